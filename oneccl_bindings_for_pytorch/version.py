__version__ = "2.8.0+b200"
git_version = "550a022a39385d31b7ca693999e752df1d5706b2"
