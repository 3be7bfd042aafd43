__version__ = "2.8.0+b200"
git_version = "c40f7d358ad5ff5eee0493c679461c427113f7eb"
