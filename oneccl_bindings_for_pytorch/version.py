__version__ = "2.8.0+b200"
git_version = "954cb6ac0de02145c87d2d06ef884b6fd61a433e"
