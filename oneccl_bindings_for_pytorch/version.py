__version__ = "2.8.0+b200"
git_version = "1446ecce481a152212983c6acec83772e4bc1d48"
