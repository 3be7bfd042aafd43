__version__ = "2.8.0+b200"
git_version = "4f8681f50a5ae32deca34fd05bcf5c8c5c7d04ba"
