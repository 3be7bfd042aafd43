__version__ = "2.8.0+b200"
git_version = "4457f4c50cbfb85c00bc2c167ac5e4873bf5ebe2"
