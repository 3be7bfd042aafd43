__version__ = "2.8.0+b200"
git_version = "9d5c1fde7652430e1d25dbc36b3f717fba3c685d"
