__version__ = "2.8.0+b200"
git_version = "9b0505d6a1cf95f2b3b1509da22ba8404fdffc16"
