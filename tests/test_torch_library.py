"""The fused ops as dispatcher ops (`torch.ops.ccl.*`): schemas, Meta kernels (shape inference with no GPU and no
communication) and tracing under torch.compile. The CUDA kernels behind the same ops are covered by the GPU tests."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist

import oneccl_bindings_for_pytorch  # noqa: F401


@pytest.fixture
def one_rank_group():
    with tempfile.TemporaryDirectory() as d:
        store = dist.FileStore(os.path.join(d, "store"), 1)
        dist.init_process_group("ccl", store=store, rank=0, world_size=1)
        try:
            yield dist.group.WORLD
        finally:
            dist.destroy_process_group()


def test_schemas_are_registered():
    for name in ["allreduce_residual_rmsnorm", "gemm_ar_norm", "all_reduce_scaled", "reduce_scatter_cast", "all_gather_copy_out",
                 "gemm_reduce_scatter", "all_gather_gemm", "moe_dispatch", "moe_combine"]:
        op = getattr(torch.ops.ccl, name)
        schema = op.default._schema
        assert "str group" in str(schema), schema
        assert torch._C._dispatch_has_kernel_for_dispatch_key(f"ccl::{name}", "CUDA")
        assert torch._C._dispatch_has_kernel_for_dispatch_key(f"ccl::{name}", "Meta")
    assert "Tensor(a!) residual" in str(torch.ops.ccl.gemm_ar_norm.default._schema)


def test_meta_kernels_give_shapes(one_rank_group):
    g = one_rank_group.group_name
    m = dict(device="meta", dtype=torch.bfloat16)
    x, res, w = torch.empty(16, 4096, **m), torch.empty(16, 4096, **m), torch.empty(4096, **m)
    assert torch.ops.ccl.allreduce_residual_rmsnorm(x, res, w, 1e-5, g).shape == (16, 4096)
    wp = torch.empty(4096 * 8, 64, **m)
    assert torch.ops.ccl.gemm_ar_norm(wp, torch.empty(16, 512, **m), res, w, 1e-5, g).shape == (16, 4096)
    out = torch.ops.ccl.reduce_scatter_cast(torch.empty(1024, **m), torch.float32, 0.5, g)
    assert out.shape == (1024,) and out.dtype == torch.float32
    assert torch.ops.ccl.gemm_reduce_scatter(torch.empty(256, 64, **m), torch.empty(128, 64, **m), g).shape == (256, 128)
    assert torch.ops.ccl.all_gather_gemm(torch.empty(128, 64, **m), torch.empty(96, 64, **m), g).shape == (128, 96)
    rows, meta, count = torch.ops.ccl.moe_dispatch(torch.empty(32, 256, **m), torch.empty(32, 2, device="meta", dtype=torch.int32), 1, 64, g)
    assert rows.shape == (64, 256) and meta.shape == (64, 3) and count.dtype == torch.int32
    gate = torch.empty(32, 2, device="meta")
    assert torch.ops.ccl.moe_combine(rows, meta, count, gate, g).shape == (32, 256)
    # the two in-place ops return nothing and accept meta tensors
    assert torch.ops.ccl.all_reduce_scaled(torch.empty(1000, **m), 0.125, g) is None
    assert torch.ops.ccl.all_gather_copy_out(torch.empty(64, **m), [torch.empty(64, **m)], g) is None
    with pytest.raises(RuntimeError, match="one destination per rank"):
        torch.ops.ccl.all_gather_copy_out(torch.empty(64, **m), [torch.empty(40, **m), torch.empty(24, **m)], g)
    with pytest.raises(RuntimeError, match="shape mismatch"):
        torch.ops.ccl.allreduce_residual_rmsnorm(x, torch.empty(8, 4096, **m), w, 1e-5, g)


def test_ops_trace_under_torch_compile(one_rank_group):
    """A tensor-parallel MLP tail written with two of the ops compiles as ONE graph (no graph break)."""
    from torch_ccl_b200 import ops

    def block(wp, act, residual, norm_w, a, b):
        xn = ops.gemm_allreduce_residual_rmsnorm(wp, act, residual, norm_w)      # mutates residual
        y = ops.gemm_reduce_scatter(a, b)
        return xn * 2, y + 1

    m = dict(device="meta", dtype=torch.bfloat16)
    args = (torch.empty(512 * 4, 64, **m), torch.empty(8, 256, **m), torch.empty(8, 512, **m), torch.empty(512, **m),
            torch.empty(128, 64, **m), torch.empty(256, 64, **m))
    compiled = torch.compile(block, backend="eager", fullgraph=True)
    xn, y = compiled(*args)
    assert xn.shape == (8, 512) and y.shape == (128, 256) and xn.device.type == "meta"
    graphs = []

    def spy(gm, example_inputs):
        graphs.append(gm)
        return gm.forward

    torch._dynamo.reset()
    torch.compile(block, backend=spy, fullgraph=True)(*args)
    text = graphs[0].print_readable(print_output=False)
    assert "ccl.gemm_ar_norm" in text and "ccl.gemm_reduce_scatter" in text
