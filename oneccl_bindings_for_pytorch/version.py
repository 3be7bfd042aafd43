__version__ = "2.8.0+b200"
git_version = "b0f33e28de06574a267e1f8b84341327a247b03d"
