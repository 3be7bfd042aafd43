__version__ = "2.8.0+b200"
git_version = "0062a956ceaa999763f2d60fc13430ca494edd86"
