"""Replay of a ZeRO-shaped collective trace with value checks (CPU ranks here; the CUDA variant
runs with >= 2 GPUs). The reference replays tests/DeepSpeed_test/DeepSpeed.csv (491 ops: 367
broadcast, 107 reduce, 10 allreduce, 8 allgather) as a hang detector without checking values
(tests/DeepSpeed_test/testccl_cpu.py:56-100); this test keeps the op mix and checks every result."""
import pytest
import torch

from mp_util import run_ranks


def _replay(rank, world, device, rounds, dtype_name, async_op):
    from torch_ccl_b200.utils import trace_replay as tr

    text = tr.synthetic_zero_trace(world, layers=2, hidden=64, steps=2)
    text += "reduce_scatter,1000,-1\nalltoall,777,-1\n# comment\n\nbroadcast,3072,%d\n" % (world - 1)
    trace = tr.parse_trace(text, world)
    ops = [t[0] for t in trace]
    assert min(ops.count(o) for o in ("broadcast", "reduce", "allreduce", "allgather", "barrier")) > 0
    res = tr.replay(trace, rounds=rounds, device=device, dtype=getattr(torch, dtype_name), async_op=async_op)
    assert res["ops"] == rounds * len(trace) and res["checked"] > 0
    with pytest.raises(ValueError, match="root"):
        tr.parse_trace("reduce,8,%d\n" % world, world)
    with pytest.raises(ValueError, match="unknown op"):
        tr.parse_trace("allscatter,8,0\n", world)


def test_trace_replay_cpu_world4():
    run_ranks(_replay, world=4, args=("cpu", 2, "float32", False))


def test_trace_replay_cpu_async_bf16_world3():
    run_ranks(_replay, world=3, args=("cpu", 1, "bfloat16", True))


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
@pytest.mark.parametrize("dtype_name", ["float16", "bfloat16"])
def test_trace_replay_cuda(dtype_name):
    run_ranks(_replay, world=min(torch.cuda.device_count(), 8), device="cuda", args=("cuda", 3, dtype_name, False))


def test_trace_replay_cpu_world8_bf16():
    """Eight CPU ranks (the reference's own stress runs 12 local processes, testccl_cpu.py:8)."""
    run_ranks(_replay, world=8, args=("cpu", 1, "bfloat16", False), timeout=300)
