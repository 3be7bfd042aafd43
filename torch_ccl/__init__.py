"""Legacy alias of `oneccl_bindings_for_pytorch` (the reference's benchmark script falls back to
this name: tests/ddp_allreduce.py:50-52 of intel/torch-ccl)."""
from oneccl_bindings_for_pytorch import *  # noqa: F401,F403
from oneccl_bindings_for_pytorch import __version__, cwd, git_version, is_available  # noqa: F401
