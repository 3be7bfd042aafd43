"""Exhaustive small sizes and a long mixed sequence on the single-GPU emulation of the collective
kernels (one cooperative launch plays all ranks). Inputs are small integers, exact in bf16, so
every result is compared bit for bit.

The reference relies on structural arguments for its flag protocol (triple buffering with a
counter reset one slot ahead, src/gpu/allreduce_small.h:275-285) and tests a handful of shapes
(tests/test_llm_allreduce.py:16-37); here every element count from 1 to 1030 and around 4096
crosses each vector tail, and 1500 back-to-back collectives of mixed kind and size exercise the
epoch / parity bookkeeping between kernels of different geometry."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu
SUM = 0


@pytest.fixture(scope="module")
def comm_of():
    import torch_ccl_b200._C as C

    cache = {}

    def get(world):
        if world not in cache:
            cache[world] = C.CudaComm.emulated(world, 2 << 20, 2000, 8)
        return cache[world]

    yield get
    cache.clear()


def pattern(n, r, dtype):
    return ((torch.arange(n, device="cuda", dtype=torch.int32) % 7) + r + 1).to(dtype)


def pattern_sum(n, world, dtype):
    return ((torch.arange(n, device="cuda", dtype=torch.int32) % 7) * world + world * (world + 1) // 2).to(dtype)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_every_small_size(comm_of, world):
    c = comm_of(world)
    dt = torch.bfloat16
    nmax = 4100
    src = [pattern(nmax * world, r, dt) for r in range(world)]
    want_sum = pattern_sum(nmax * world, world, dt)
    out = [torch.empty(nmax * world, device="cuda", dtype=dt) for _ in range(world)]
    bad = []
    for n in list(range(1, 1031)) + list(range(4090, 4100)):
        for algo in (1, 2):
            for o in out:
                o[:n].zero_()
            c.allreduce([s[:n] for s in src], [o[:n] for o in out], SUM, 1.0, 0, algo)
            if not all(torch.equal(o[:n], want_sum[:n]) for o in out):
                bad.append(("allreduce", algo, n))
        if n <= 520:
            # all_gather of n elements per rank, reduce_scatter down to n elements per rank
            c.all_gather([s[:n] for s in src], [[o[p * n:(p + 1) * n] for p in range(world)] for o in out])
            for o in out:
                for p in range(world):
                    if not torch.equal(o[p * n:(p + 1) * n], src[p][:n]):
                        bad.append(("all_gather", p, n))
            rs_out = [torch.empty(n, device="cuda", dtype=dt) for _ in range(world)]
            c.reduce_scatter([[s[p * n:(p + 1) * n] for p in range(world)] for s in src], rs_out, SUM, 1.0, 0)
            for r in range(world):
                if not torch.equal(rs_out[r], want_sum[r * n:(r + 1) * n]):
                    bad.append(("reduce_scatter", r, n))
        assert not bad, bad[:5]
    torch.cuda.synchronize()
    assert c.status()[0] == 0


def test_long_mixed_sequence(comm_of):
    world = 4
    c = comm_of(world)
    rng = random.Random(7)
    dt = torch.bfloat16
    nmax = 70000
    src = [pattern(nmax * world, r, dt) for r in range(world)]
    want_sum = pattern_sum(nmax * world, world, dt)
    out = [torch.empty(nmax * world, device="cuda", dtype=dt) for _ in range(world)]
    for step in range(1500):
        kind = rng.choice(["ar1", "ar2", "ag", "rs", "a2a", "bcast", "barrier"])
        n = rng.choice([1, 3, 8, 257, 4096, 20000, 65537]) if step % 3 else rng.randint(1, nmax)
        if kind in ("ar1", "ar2"):
            c.allreduce([s[:n] for s in src], [o[:n] for o in out], SUM, 1.0, 0, 1 if kind == "ar1" else 2)
            ok = all(torch.equal(o[:n], want_sum[:n]) for o in out)
        elif kind == "ag":
            c.all_gather([s[:n] for s in src], [[o[p * n:(p + 1) * n] for p in range(world)] for o in out])
            ok = all(torch.equal(o[p * n:(p + 1) * n], src[p][:n]) for o in out for p in range(world))
        elif kind == "rs":
            c.reduce_scatter([[s[p * n:(p + 1) * n] for p in range(world)] for s in src], [o[:n] for o in out], SUM, 1.0, 0)
            ok = all(torch.equal(out[r][:n], want_sum[r * n:(r + 1) * n]) for r in range(world))
        elif kind == "a2a":
            c.all_to_all([[s[p * n:(p + 1) * n] for p in range(world)] for s in src],
                         [[o[p * n:(p + 1) * n] for p in range(world)] for o in out], False)
            ok = all(torch.equal(out[r][p * n:(p + 1) * n], src[p][r * n:(r + 1) * n]) for r in range(world) for p in range(world))
        elif kind == "bcast":
            root = rng.randrange(world)
            bufs = [src[r][:n].clone() for r in range(world)]
            c.broadcast(bufs, root)
            ok = all(torch.equal(b, src[root][:n]) for b in bufs)
        else:
            c.barrier()
            ok = True
        assert ok, (step, kind, n)
    torch.cuda.synchronize()
    assert c.status()[0] == 0
