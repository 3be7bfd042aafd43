__version__ = "2.8.0+b200"
git_version = "bf21273d28bdf987e048743f2dbd7f1f65ffdddb"
