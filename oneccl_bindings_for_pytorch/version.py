__version__ = "2.8.0+b200"
git_version = "d3068b93523a41f4ef44d895d1be8cf8ff01cda8"
