"""B200-native `ccl` backend for torch.distributed.

Layout:
  _C          compiled extension: ProcessGroupCCL (C++), CPU shared-memory collectives, the
              sm_100a collective / GEMM / attention kernels and their launchers
  ops         fused collective + compute ops on a process group
  parallel    tensor-parallel layers, FSDP communication hooks, expert-parallel dispatch
  models      Llama-architecture decoder used by the benchmarks
  utils       environment, tuner table, statistics
"""
import torch  # noqa: F401

from . import _C  # registers backend "ccl" with torch.distributed


def stats():
    """Per-op statistics of this process: count, bytes, host time histogram, algorithms."""
    return _C.stats()


def flight_recorder():
    """Text dump of the most recent operations (also printed when a collective times out)."""
    return _C.flight_recorder()


def reparse_env():
    """Re-read the environment knobs (they are otherwise parsed once per process)."""
    _C.reparse_env()


def get_backend(group=None, device="cuda"):
    """The ProcessGroupCCL object that serves `device` tensors of `group`."""
    import torch.distributed as dist

    group = group if group is not None else dist.group.WORLD
    return group._get_backend(torch.device(device))


from . import ops  # noqa: E402,F401
