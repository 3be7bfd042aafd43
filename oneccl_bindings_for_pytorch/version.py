__version__ = "2.8.0+b200"
git_version = "99a51b7a3789f8f8f200f74add169891669d210e"
