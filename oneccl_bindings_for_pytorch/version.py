__version__ = "2.8.0+b200"
git_version = "3d0cdeceb6f67ae9d14cff0ef9a8b959bc8ab19b"
