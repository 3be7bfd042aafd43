__version__ = "2.8.0+b200"
git_version = "d32e83a6841375b2104aba14274413680d05943a"
