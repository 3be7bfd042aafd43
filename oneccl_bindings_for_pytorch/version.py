__version__ = "2.8.0+b200"
git_version = "60d869f6482e34216bc6ea1997d8375e4bb550ab"
