__version__ = "2.8.0+b200"
git_version = "6d99678bac48ccd2325915631b494121a1415d29"
