"""B200-native `ccl` backend for torch.distributed.

Layout:
  _C          compiled extension: ProcessGroupCCL (C++), CPU shared-memory collectives, the
              sm_100a collective / GEMM / attention kernels and their launchers
  ops         fused collective + compute ops on a process group (also registered as torch.ops.ccl.*)
  parallel    full-shard (ZeRO-3) engine, sequence-parallel tensor-parallel linear layers
  models      tensor-parallel Llama-architecture decoder used by the benchmarks
  utils       collective trace replay with value checks
Environment knobs, the tuning table and statistics live in the extension: see env(), stats(),
flight_recorder() below and torch_ccl_b200._C.
"""
import torch  # noqa: F401

from . import _C  # registers backend "ccl" with torch.distributed and the torch.ops.ccl.* ops


def _check_c10d_cuda_keys():
    """torch.distributed reaches this backend for CUDA tensors through torch's own `c10d::*` CUDA
    dispatcher entries (they call the Backend object of the process group). The reference has to
    register those entries itself for its device (src/ProcessGroupCCL.cpp:86-738 of intel/torch-ccl);
    here they must already exist - a torch build without them could not route a CUDA collective."""
    names = ["allreduce_", "broadcast_", "reduce_", "allgather_", "_allgather_base_", "reduce_scatter_",
             "_reduce_scatter_base_", "alltoall_", "alltoall_base_", "gather_", "scatter_", "barrier", "send", "recv_"]
    has = torch._C._dispatch_has_kernel_for_dispatch_key
    missing = [n for n in names if not has("c10d::" + n, "CUDA")]
    if missing:
        raise ImportError("this torch build has no CUDA dispatcher entries for c10d ops " + ", ".join(missing) +
                          "; the 'ccl' backend cannot serve CUDA tensors with it")


_check_c10d_cuda_keys()


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


def symm_empty(shape, dtype=torch.float32, group=None, device=None):
    """An uninitialised SYMMETRIC tensor: memory from the group's symmetric heap, mapped by every rank, so that
    all_reduce / reduce_scatter_tensor / all_gather_into_tensor on it run zero-copy over NVLink (through the NVSwitch
    reduction when the heap is bound to a multicast object, CCL_NVLS=1) instead of staging through the arena.
    Collective in order: every rank of the group must allocate the same sizes in the same order and drop them in the
    same order. The heap has CCL_SYMM_HEAP_MB megabytes (default 1024) and is created by the first allocation.
    Same as `backend.allocate_tensor(...)` of torch's Backend API."""
    shape = (shape,) if isinstance(shape, int) else tuple(shape)
    numel = 1
    for s in shape:
        numel *= int(s)
    be = get_backend(group, "cuda")
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    return be.symm_empty(numel, dtype, dev).view(shape)


def is_symmetric(tensor, group=None):
    """True if `tensor` lies wholly inside the group's symmetric heap."""
    return get_backend(group, "cuda").is_symmetric(tensor)


from . import ops  # noqa: E402,F401
