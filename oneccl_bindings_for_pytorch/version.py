__version__ = "2.8.0+b200"
git_version = "a0b43a4f12145a3ce0a13b6cbe602832f2c5e41b"
