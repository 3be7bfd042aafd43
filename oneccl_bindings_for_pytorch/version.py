__version__ = "2.8.0+b200"
git_version = "1f528759742ec017cddbbc7db7215629c9ee94ad"
