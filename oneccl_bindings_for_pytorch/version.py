__version__ = "2.8.0+b200"
git_version = "8dbd6f50d42db14a614b645275c693d25a32b8aa"
