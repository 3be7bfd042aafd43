__version__ = "2.8.0+b200"
git_version = "d0bdc7dd038ea40a0bc26ea7641e8c4b997dd693"
