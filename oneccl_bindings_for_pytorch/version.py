__version__ = "2.8.0+b200"
git_version = "17dd01a0b1a5546746e5196e1404f65ca4efa7cb"
