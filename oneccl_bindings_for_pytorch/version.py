__version__ = "2.8.0+b200"
git_version = "b608ed1cbd4361b0cef7ef8057f5911ce91ffc21"
