"""Small, fixed single-kernel workloads for profiling (one kernel family per case, a handful of
launches, inputs larger than the 126 MB L2 but only a few hundred MB on the device).

    python bench/kernel_cases.py {gemm_decode|gemm_swiglu|gemm_large|attention|addnorm} [--iters N]
    python bench/kernel_cases.py {tp8_qkv|tp8_gate_up|tp8_attention|tp8_fused_o|tp8_fused_down} [--iters N]

    python bench/kernel_cases.py {emu_oneshot|emu_twoshot|emu_reduce_scatter|emu_all_to_all|emu_symm_allreduce} [--iters N]

The emu_* cases run one collective kernel for EIGHT ranks on one GPU (one cooperative launch with gridDim.y = 8, every
rank's arena on this device): the only form in which a profiler can look at a collective kernel, since kernels of
different ranks wait on one another. Traffic that crosses NVLink in a real run shows up as L2 / DRAM traffic here.

The tp8_* cases are the kernels of one layer of the tensor-parallel decode step at the shapes ONE rank of
eight sees (Llama-7B, batch 16, 1024-token context), on a one-rank communicator: what a rank computes when
no time is spent waiting for peers.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch_ccl_b200._C as C  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--iters", type=int, default=6)
    ap.add_argument("--splitk", type=int, default=0, help="tp8_* GEMM cases: split-K factor (0 = the library's choice)")
    a = ap.parse_args()
    dev = "cuda"
    bf = dict(device=dev, dtype=torch.bfloat16)
    if a.case == "gemm_decode":  # Llama-7B QKV projection at batch 16 (weights stream from HBM)
        ws = [torch.randn(12288, 4096, **bf) * 0.02 for _ in range(3)]
        x = torch.randn(16, 4096, **bf)
        out = torch.empty(16, 12288, **bf)
        fn = lambda i: C.gemm_bf16_tn(ws[i % 3], x, out, True, 0, 0, 16)
    elif a.case == "gemm_swiglu":  # gate/up projection with the fused SwiGLU epilogue
        ws = [torch.randn(22016, 4096, **bf) * 0.02 for _ in range(2)]
        x = torch.randn(16, 4096, **bf)
        out = torch.empty(16, 11008, **bf)
        fn = lambda i: C.gemm_bf16_tn(ws[i % 2], x, out, True, 11008, 0, 16)
    elif a.case == "gemm_large":  # compute-bound
        A = torch.randn(8192, 4096, **bf)
        B = torch.randn(8192, 4096, **bf)
        out = torch.empty(8192, 8192, **bf)
        fn = lambda i: C.gemm_bf16_tn(A, B, out, False, 0, 1, 0)
    elif a.case == "attention":  # batch 16 x 32 heads over a 1024-token cache (268 MB of K/V)
        B, nh, S = 16, 32, 1280
        qkv = torch.randn(B, 3 * nh * 128, **bf)
        kc = torch.randn(B, nh, S, 128, **bf)
        vc = torch.randn(B, nh, S, 128, **bf)
        pos = torch.full((B,), 1024, device=dev, dtype=torch.int32)
        inv = 1.0 / (10000.0 ** (torch.arange(0, 128, 2, device=dev).float() / 128))
        ang = torch.arange(S, device=dev).float()[:, None] * inv[None]
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
        out = torch.empty(B, nh * 128, **bf)
        ns = C.decode_attention_default_splits(B, nh, S)
        scratch = torch.zeros(C.decode_attention_scratch_bytes(B, nh, ns) // 4 + 1, device=dev)
        cnt = torch.zeros(B * nh, device=dev, dtype=torch.int32)
        fn = lambda i: C.decode_attention(qkv, kc, vc, pos, cos, sin, out, scratch, cnt, nh, nh, ns)
    elif a.case == "addnorm":
        comm = C.CudaComm.create(None, 0, 1, 1 << 20, 1000, "ccl/case")
        x = torch.randn(16, 4096, **bf)
        res = torch.randn(16, 4096, **bf)
        w = torch.ones(4096, **bf)
        out = torch.empty(16, 4096, **bf)
        fn = lambda i: comm.allreduce_residual_rmsnorm([x], [res], [w], [out], 1e-5)
    elif a.case in ("tp8_qkv", "tp8_gate_up", "tp8_fused_o", "tp8_fused_down"):
        from torch_ccl_b200.ops import pack_weight

        x16 = torch.randn(16, 4096, **bf)
        if a.case == "tp8_qkv":  # 4 + 4 + 4 heads: 12.6 MB of weights
            ws = [pack_weight(torch.randn(1536, 4096, **bf) * 0.02) for _ in range(12)]
            out = torch.empty(16, 1536, **bf)
            fn = lambda i: C.gemm_bf16_tn(ws[i % 12], x16, out, True, 0, a.splitk, 16, 1536)
        elif a.case == "tp8_gate_up":  # 1376 + 1376 rows with the SwiGLU epilogue: 22.5 MB of weights
            pad = (1376 + 127) // 128 * 128
            ws = [torch.cat([pack_weight(torch.randn(1376, 4096, **bf) * 0.02), pack_weight(torch.randn(1376, 4096, **bf) * 0.02)]) for _ in range(8)]
            out = torch.empty(16, 1376, **bf)
            fn = lambda i: C.gemm_bf16_tn(ws[i % 8], x16, out, True, pad, a.splitk, 16, 1376)
        else:  # row-parallel projection + (one-rank) all_reduce + residual + norm in one launch
            K = 512 if a.case == "tp8_fused_o" else 1376
            comm = C.CudaComm.create(None, 0, 1, 1 << 20, 1000, "ccl/case")
            n = 40 if K == 512 else 16
            ws = [pack_weight(torch.randn(4096, K, **bf) * 0.02) for _ in range(n)]
            xk = torch.randn(16, K, **bf)
            res = torch.randn(16, 4096, **bf)
            wn = torch.ones(4096, **bf)
            out = torch.empty(16, 4096, **bf)
            fn = lambda i: comm.gemm_ar_norm([ws[i % n]], [xk], [res], [wn], [out], 1e-5, a.splitk)
    elif a.case.startswith("emu_"):
        W = 8
        comm = C.CudaComm.emulated(W, 64 << 20, 2000, 16)
        nbytes = (64 << 10) if a.case == "emu_oneshot" else (8 << 20)
        n = nbytes // 2
        if a.case in ("emu_oneshot", "emu_twoshot"):
            comm.set_oneshot_max_bytes((1 << 30) if a.case == "emu_oneshot" else 1)
            xs = [torch.randn(n, **bf) for _ in range(W)]
            outs = [torch.empty(n, **bf) for _ in range(W)]
            fn = lambda i: comm.allreduce(xs, outs)
        elif a.case == "emu_symm_allreduce":
            comm.set_symm_min_bytes(0)
            xs = [t.view(torch.bfloat16) for t in comm.symm_empty(nbytes)]
            for t in xs:
                t.normal_()
            fn = lambda i: comm.allreduce(xs, xs)
        elif a.case == "emu_reduce_scatter":
            ins = [list(torch.randn(n, **bf).chunk(W)) for _ in range(W)]
            outs = [torch.empty(n // W, **bf) for _ in range(W)]
            fn = lambda i: comm.reduce_scatter(ins, outs)
        elif a.case == "emu_all_to_all":
            ins = [list(torch.randn(n, **bf).chunk(W)) for _ in range(W)]
            outs = [list(torch.empty(n, **bf).chunk(W)) for _ in range(W)]
            fn = lambda i: comm.all_to_all(ins, outs)
        else:
            raise SystemExit("unknown case")
    elif a.case == "tp8_attention":  # 16 sequences x 4 heads over a 1024-token cache; caches cycled through > L2
        B, nh, S = 16, 4, 1280
        qkv = torch.randn(B, 3 * nh * 128, **bf)
        caches = [(torch.randn(B, nh, S, 128, **bf), torch.randn(B, nh, S, 128, **bf)) for _ in range(5)]
        pos = torch.full((B,), 1024, device=dev, dtype=torch.int32)
        inv = 1.0 / (10000.0 ** (torch.arange(0, 128, 2, device=dev).float() / 128))
        ang = torch.arange(S, device=dev).float()[:, None] * inv[None]
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
        out = torch.empty(B, nh * 128, **bf)
        ns = C.decode_attention_default_splits(B, nh, S)
        scratch = torch.zeros(C.decode_attention_scratch_bytes(B, nh, ns) // 4 + 1, device=dev)
        cnt = torch.zeros(B * nh, device=dev, dtype=torch.int32)
        fn = lambda i: C.decode_attention(qkv, caches[i % 5][0], caches[i % 5][1], pos, cos, sin, out, scratch, cnt, nh, nh, ns)
    else:
        raise SystemExit("unknown case")
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    s.record()
    for i in range(a.iters):
        fn(i)
    e.record()
    torch.cuda.synchronize()
    print(f"{a.case}{' splitk ' + str(a.splitk) if a.splitk else ''}: {s.elapsed_time(e) / a.iters * 1e3:.2f} us per launch")


if __name__ == "__main__":
    main()
