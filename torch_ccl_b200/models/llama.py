"""Tensor-parallel Llama-architecture decoder for serving benchmarks and tests.

Every hot op of a decode step is a kernel of this repository:

  * projections: the tcgen05 bf16 GEMM in swap-AB form (weights on the 128-row UMMA M side, the
    few activation rows on the N side), split-K over a thread-block cluster, SwiGLU fused into
    the gate/up projection;
  * attention: fused RoPE + KV-cache append + split-KV decode attention;
  * the two all_reduces per layer: one-shot peer-memory all_reduce fused with the residual add
    and the following RMSNorm (the pattern the reference's LLM all-reduce path targets,
    tests/test_allreduce.py:51-67 and src/gpu/allreduce_small.h of intel/torch-ccl).

The whole step is captured in one CUDA graph. Weights are random N(0, 0.02) in bf16, generated
from per-matrix seeds so that every tensor-parallel degree shards the same full model.
"""
import math
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .. import _C
from ..ops import pack_weight, unpack_weight


@dataclass
class LlamaConfig:
    vocab: int = 32000
    hidden: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 32
    inter: int = 11008
    head_dim: int = 128
    eps: float = 1e-5
    rope_theta: float = 10000.0

    @staticmethod
    def llama7b():
        return LlamaConfig()

    @staticmethod
    def tiny(n_layers=2):
        return LlamaConfig(vocab=1024, hidden=512, n_layers=n_layers, n_heads=4, n_kv_heads=4, inter=1408)


def _rand(shape, seed, device, std=0.02):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).to(torch.bfloat16)


class _Comm:
    """The fused ops of the process group's CUDA communicator, or single-GPU stand-ins.

    collective="nccl" is the comparison arm: the same model and kernels, but every all_reduce /
    all_gather goes through a torch.distributed NCCL group and the residual add + RMSNorm runs as a
    separate local kernel afterwards (what a model on the stock backend does)."""

    def __init__(self, group, device, collective="ccl"):
        self.world = dist.get_world_size(group) if (group is not None or dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.direct = None
        self.backend = None
        self.nccl = None
        if self.world > 1 and collective == "nccl":
            ranks = dist.get_process_group_ranks(group) if group is not None else list(range(self.world))
            self.nccl = dist.new_group(ranks=ranks, backend="nccl")
            self.direct = _C.CudaComm.create(None, 0, 1, 1 << 20, 1000, "ccl/local-norm")
        elif self.world > 1:
            from .. import get_backend

            self.backend = get_backend(group, "cuda")
        else:
            # one-rank communicator: the fused norm kernel degenerates to add + rmsnorm
            self.direct = _C.CudaComm.create(None, 0, 1, 1 << 20, 1000, "ccl/single")

    def ar_res_norm(self, x, residual, weight, out, eps):
        if self.backend is not None:
            self.backend.fused_allreduce_residual_rmsnorm(x, residual, weight, out, eps)
        else:
            if self.nccl is not None:
                dist.all_reduce(x, group=self.nccl)
            self.direct.allreduce_residual_rmsnorm([x], [residual], [weight], [out], eps)

    def embed_norm(self, tokens, table, vocab_base, residual, weight, out, eps):
        """residual <- all_reduce(vocab-parallel embedding of `tokens`); out = rmsnorm(residual) * weight.
        One kernel: the lookup is the producer side of the fused all_reduce + norm."""
        if self.backend is not None:
            self.backend.fused_allreduce_residual_rmsnorm(table, residual, weight, out, eps, tokens, vocab_base, True)
        else:
            self.direct.allreduce_residual_rmsnorm([table], [residual], [weight], [out], eps, [tokens], [vocab_base], True)

    def fits_gemm_ar_norm(self, like, rows, hidden, k):
        if self.nccl is not None:
            return False
        if self.backend is not None:
            return self.backend.fits_gemm_ar_norm(like, rows, hidden, k)
        return self.direct.fits_gemm_ar_norm(rows, hidden, k)

    def gemm_ar_norm(self, w_packed, x, residual, weight, out, eps, splitk=0):
        """residual += all_reduce(x @ w^T); out = rmsnorm(residual) * weight, in ONE kernel."""
        if self.backend is not None:
            self.backend.fused_gemm_ar_norm(w_packed, x, residual, weight, out, eps, splitk)
        else:
            self.direct.gemm_ar_norm([w_packed], [x], [residual], [weight], [out], eps, splitk)

    def sample(self, logits, next_tokens, tokens, positions):
        """Greedy sampling over the vocabulary shards: arg-max, all-gather of the per-rank winners
        and the bookkeeping for the next step (tokens <- winner, positions += 1) in one kernel."""
        if self.backend is not None:
            self.backend.fused_sample_allgather(logits, next_tokens, tokens, positions)
        else:
            self.direct.sample_allgather([logits], [next_tokens], [tokens], [positions])

    def all_reduce(self, t):
        if self.backend is not None:
            self.backend.fused_allreduce(t, 1.0)
        elif self.nccl is not None:
            dist.all_reduce(t, group=self.nccl)

    def all_gather(self, shard, out):
        if self.backend is not None:
            self.backend.fused_all_gather_copy_out(shard, list(out.chunk(self.world)))
        elif self.nccl is not None:
            dist.all_gather_into_tensor(out.view(-1), shard.contiguous().view(-1), group=self.nccl)
        else:
            out.copy_(shard.view_as(out))


class TPLlamaDecoder:
    """Llama decoder sharded `world`-way by attention head and FFN column (Megatron layout)."""

    def __init__(self, cfg: LlamaConfig, max_batch=16, max_seq=2048, group=None, device=None, seed=0, collective="ccl",
                 fused=True):
        """fused=True (default): 5 kernels per layer - qkv GEMM, attention, o_proj GEMM + all_reduce +
        residual + norm in one launch, gate/up GEMM + SwiGLU, down_proj GEMM + all_reduce + residual +
        norm in one launch - plus embedding + first norm, lm_head and the sampling kernel per step.
        fused=False: the projections, the all_reduce + norm and the sampling run as separate kernels
        (7 per layer); kept for A/B measurements. collective="nccl" implies fused=False."""
        self.cfg = cfg
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.comm = _Comm(group, self.device, collective)
        self.fused = bool(fused) and collective == "ccl"
        W, r = self.comm.world, self.comm.rank
        self.world, self.rank = W, r
        assert cfg.n_heads % W == 0 and cfg.n_kv_heads % W == 0 and cfg.inter % (8 * W) == 0 and cfg.vocab % W == 0
        assert cfg.head_dim == 128, "decode attention kernel is specialised for head_dim 128"
        self.max_batch, self.max_seq = max_batch, max_seq
        self.nh = cfg.n_heads // W
        self.nkv = cfg.n_kv_heads // W
        self.inter = cfg.inter // W
        self.vshard = cfg.vocab // W
        hd, H = cfg.head_dim, cfg.hidden
        dev = self.device
        self.layers = []
        for li in range(cfg.n_layers):
            s = seed * 100003 + li * 16
            wq = _rand((cfg.n_heads * hd, H), s + 1, dev)[r * self.nh * hd:(r + 1) * self.nh * hd]
            wk = _rand((cfg.n_kv_heads * hd, H), s + 2, dev)[r * self.nkv * hd:(r + 1) * self.nkv * hd]
            wv = _rand((cfg.n_kv_heads * hd, H), s + 3, dev)[r * self.nkv * hd:(r + 1) * self.nkv * hd]
            wo = _rand((H, cfg.n_heads * hd), s + 4, dev)[:, r * self.nh * hd:(r + 1) * self.nh * hd]
            wg = _rand((cfg.inter, H), s + 5, dev)[r * self.inter:(r + 1) * self.inter]
            wu = _rand((cfg.inter, H), s + 6, dev)[r * self.inter:(r + 1) * self.inter]
            wd = _rand((H, cfg.inter), s + 7, dev)[:, r * self.inter:(r + 1) * self.inter]
            # weights are kept pre-tiled for streaming (see ops.pack_weight); gate and up are padded
            # to whole 128-row tiles separately so that the SwiGLU pairs line up tile by tile
            self.layers.append(dict(
                wqkv=pack_weight(torch.cat([wq, wk, wv])), wo=pack_weight(wo),
                wgu=torch.cat([pack_weight(wg), pack_weight(wu)]), wd=pack_weight(wd),
                attn_norm=torch.ones(H, device=dev, dtype=torch.bfloat16),
                mlp_norm=torch.ones(H, device=dev, dtype=torch.bfloat16),
                k=torch.zeros(max_batch, self.nkv, max_seq, hd, device=dev, dtype=torch.bfloat16),
                v=torch.zeros(max_batch, self.nkv, max_seq, hd, device=dev, dtype=torch.bfloat16)))
            del wq, wk, wv, wo, wg, wu, wd
        self.embed = _rand((cfg.vocab, H), seed * 100003 + 900001, dev)[r * self.vshard:(r + 1) * self.vshard].contiguous()
        self.lm_head = pack_weight(_rand((cfg.vocab, H), seed * 100003 + 900002, dev)[r * self.vshard:(r + 1) * self.vshard])
        self.inter_pad = (self.inter + 127) // 128 * 128
        self.qkv_rows = (self.nh + 2 * self.nkv) * hd
        self.final_norm = torch.ones(H, device=dev, dtype=torch.bfloat16)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, device=dev, dtype=torch.float32) / hd))
        ang = torch.arange(max_seq, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos().contiguous(), ang.sin().contiguous()
        # persistent decode buffers (the CUDA graph captures their addresses)
        B = max_batch
        bf = dict(device=dev, dtype=torch.bfloat16)
        self.tokens = torch.zeros(B, device=dev, dtype=torch.int64)
        self.positions = torch.zeros(B, device=dev, dtype=torch.int32)
        self.next_tokens = torch.zeros(B, device=dev, dtype=torch.int64)
        self.h = torch.zeros(B, H, **bf)
        self.x = torch.zeros(B, H, **bf)
        self.xn = torch.zeros(B, H, **bf)
        self.qkv = torch.zeros(B, (self.nh + 2 * self.nkv) * hd, **bf)
        self.attn = torch.zeros(B, self.nh * hd, **bf)
        self.act = torch.zeros(B, self.inter, **bf)
        self.logits = torch.zeros(B, self.vshard, device=dev, dtype=torch.float32)
        self.nsplit = _C.decode_attention_default_splits(B, self.nh, max_seq)
        self.scratch = torch.zeros(max(1, _C.decode_attention_scratch_bytes(B, self.nh, self.nsplit) // 4), device=dev)
        self.counters = torch.zeros(B * self.nh, device=dev, dtype=torch.int32)
        self.best = torch.zeros(W, B, 2, device=dev, dtype=torch.float32)
        self.my_best = torch.zeros(B, 2, device=dev, dtype=torch.float32)
        self.graph = None
        self.graph_batch = None
        # (the unfused path also runs ~20 small torch kernels per step that are not counted here)
        self.kernels_per_step = cfg.n_layers * 5 + 3 if self.fused else cfg.n_layers * 7 + 2 + (1 if W > 1 else 0)
        self._pin_in = None
        self._pin_out = None

    # ------------------------------------------------------------------------------------
    def _gemm_t(self, w, x, out, rows, dual=0, splitk=0):
        """out[b, n] = x[b, :] @ W[n, :]^T with the pre-tiled weights on the UMMA M side."""
        b = x.shape[0]
        bn = 16 if b <= 16 else (32 if b <= 32 else (64 if b <= 64 else 128))
        _C.gemm_bf16_tn(w, x, out, True, dual, 1 if b > 64 else splitk, bn, rows)

    def dense_weights(self, L):
        """Row-major copies of a layer's weights (oracle / debugging only)."""
        H, hd = self.cfg.hidden, self.cfg.head_dim
        half = L["wgu"].shape[0] // 2
        return dict(wqkv=unpack_weight(L["wqkv"], self.qkv_rows, H), wo=unpack_weight(L["wo"], H, self.nh * hd),
                    wg=unpack_weight(L["wgu"][:half], self.inter, H), wu=unpack_weight(L["wgu"][half:], self.inter, H),
                    wd=unpack_weight(L["wd"], H, self.inter))

    def _embed_partial(self, tokens, out):
        """Vocab-parallel embedding: rows outside this rank's shard contribute zeros."""
        idx = tokens - self.rank * self.vshard
        ok = (idx >= 0) & (idx < self.vshard)
        rows = self.embed.index_select(0, idx.clamp(0, self.vshard - 1))
        out.copy_(rows * ok[:, None].to(rows.dtype))

    def _decode_body(self, B):
        if self.fused and self.comm.fits_gemm_ar_norm(self.h, B, self.cfg.hidden, self.inter):
            return self._decode_body_fused(B)
        return self._decode_body_unfused(B)

    def _decode_body_fused(self, B):
        cfg = self.cfg
        tokens, h, xn = self.tokens[:B], self.h[:B], self.xn[:B]
        qkv, attn, act = self.qkv[:B], self.attn[:B], self.act[:B]
        self.comm.embed_norm(tokens, self.embed, self.rank * self.vshard, h, self.layers[0]["attn_norm"], xn, cfg.eps)
        for li, L in enumerate(self.layers):
            self._gemm_t(L["wqkv"], xn, qkv, self.qkv_rows)
            _C.decode_attention(qkv, L["k"], L["v"], self.positions[:B], self.cos, self.sin, attn, self.scratch,
                                self.counters, self.nh, self.nkv, self.nsplit)
            self.comm.gemm_ar_norm(L["wo"], attn, h, L["mlp_norm"], xn, cfg.eps)
            self._gemm_t(L["wgu"], xn, act, self.inter, dual=self.inter_pad)
            nw = self.layers[li + 1]["attn_norm"] if li + 1 < cfg.n_layers else self.final_norm
            self.comm.gemm_ar_norm(L["wd"], act, h, nw, xn, cfg.eps)
        self._gemm_t(self.lm_head, xn, self.logits[:B], self.vshard)
        # feeds the sampled ids back into self.tokens and advances the positions: steady state is a pure replay
        self.comm.sample(self.logits[:B], self.next_tokens[:B], tokens, self.positions[:B])

    def _decode_body_unfused(self, B):
        cfg = self.cfg
        tokens, h, x, xn = self.tokens[:B], self.h[:B], self.x[:B], self.xn[:B]
        qkv, attn, act = self.qkv[:B], self.attn[:B], self.act[:B]
        self._embed_partial(tokens, x)
        h.zero_()
        self.comm.ar_res_norm(x, h, self.layers[0]["attn_norm"], xn, cfg.eps)
        for li, L in enumerate(self.layers):
            self._gemm_t(L["wqkv"], xn, qkv, self.qkv_rows)
            _C.decode_attention(qkv, L["k"], L["v"], self.positions[:B], self.cos, self.sin, attn, self.scratch,
                                self.counters, self.nh, self.nkv, self.nsplit)
            self._gemm_t(L["wo"], attn, x, cfg.hidden)
            self.comm.ar_res_norm(x, h, L["mlp_norm"], xn, cfg.eps)
            self._gemm_t(L["wgu"], xn, act, self.inter, dual=self.inter_pad)
            self._gemm_t(L["wd"], act, x, cfg.hidden)
            nw = self.layers[li + 1]["attn_norm"] if li + 1 < cfg.n_layers else self.final_norm
            self.comm.ar_res_norm(x, h, nw, xn, cfg.eps)
        self._gemm_t(self.lm_head, xn, self.logits[:B], self.vshard)
        val, idx = self.logits[:B].max(dim=-1)
        if self.world > 1:
            self.my_best[:B, 0] = val
            self.my_best[:B, 1] = (idx + self.rank * self.vshard).to(torch.float32)
            self.comm.all_gather(self.my_best, self.best)
            win = self.best[:, :B, 0].argmax(dim=0)
            self.next_tokens[:B] = self.best[:, :B, 1].gather(0, win[None, :])[0].to(torch.int64)
        else:
            self.next_tokens[:B] = idx
        self.positions[:B] += 1
        self.tokens[:B] = self.next_tokens[:B]  # feed the sampled ids back: steady state is a pure replay

    def capture(self, B):
        """Capture one decode step for batch size B in a CUDA graph."""
        assert B <= self.max_batch
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        saved_pos = self.positions.clone()
        saved_tok = self.tokens.clone()  # the step feeds its sampled ids back into self.tokens
        with torch.cuda.stream(s):
            for _ in range(2):  # warm-up outside capture (lazy inits, tensor-map cache)
                self._decode_body(B)
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        self.positions.copy_(saved_pos)
        self.tokens.copy_(saved_tok)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            self._decode_body(B)
        self.graph, self.graph_batch = g, B
        torch.cuda.synchronize(self.device)
        return g

    def decode_step(self, B=None):
        """One token for each of the B sequences: reads self.tokens / self.positions, writes
        self.next_tokens and advances the positions. Device-side only."""
        B = B or self.graph_batch or self.max_batch
        if self.graph is not None and self.graph_batch == B:
            self.graph.replay()
        else:
            self._decode_body(B)
        return self.next_tokens[:B]

    def decode_step_host(self, tokens_pinned, out_pinned):
        """End-to-end step for a serving loop: token ids come from pinned host memory and the
        sampled ids are read back to pinned host memory."""
        B = tokens_pinned.numel()
        self.tokens[:B].copy_(tokens_pinned, non_blocking=True)
        self.decode_step(B)
        out_pinned.copy_(self.next_tokens[:B], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return out_pinned

    # ------------------------------------------------------------------------------------
    def prefill(self, prompt, chunk_seqs=None):
        """Runs the prompt [B, S] through the model, fills the KV caches and leaves the first generated
        token in self.tokens. All sequences of a chunk go through every layer together ([chunk * S]
        rows per GEMM): the same tcgen05 GEMM in its row-major form, the staged all_reduce fused with
        residual add + norm (in slices that fit the communicator's staging arena), and torch's
        scaled_dot_product_attention for the causal attention over the prompt itself.
        `chunk_seqs` bounds the sequences per pass (default: as many as keep a pass under ~32k rows)."""
        cfg = self.cfg
        B, S = prompt.shape
        hd, H = cfg.head_dim, cfg.hidden
        dev = self.device
        bf = dict(device=dev, dtype=torch.bfloat16)
        cos = self.cos[:S].to(torch.bfloat16)[None, :, None, :]
        sin = self.sin[:S].to(torch.bfloat16)[None, :, None, :]

        def rope(t):  # [n, S, heads, hd]
            t1, t2 = t[..., : hd // 2], t[..., hd // 2:]
            return torch.cat([t1 * cos - t2 * sin, t2 * cos + t1 * sin], dim=-1)

        cap_rows = 1024 if self.world > 1 else 1 << 30  # rows per fused-norm launch (staging capacity)
        per = chunk_seqs or max(1, 32768 // S)
        for b0 in range(0, B, per):
            n = min(per, B - b0)
            R = n * S
            toks = prompt[b0:b0 + n].reshape(-1).to(dev)
            x = torch.empty(R, H, **bf)
            self._embed_partial(toks, x)
            h = torch.zeros(R, H, **bf)
            xn = torch.empty(R, H, **bf)

            def norm_step(w):
                for r0 in range(0, R, cap_rows):
                    r1 = min(R, r0 + cap_rows)
                    self.comm.ar_res_norm(x[r0:r1], h[r0:r1], w, xn[r0:r1], cfg.eps)

            norm_step(self.layers[0]["attn_norm"])
            qkv = torch.empty(R, (self.nh + 2 * self.nkv) * hd, **bf)
            attn = torch.empty(R, self.nh * hd, **bf)
            act = torch.empty(R, self.inter, **bf)
            for li, L in enumerate(self.layers):
                self._gemm_t(L["wqkv"], xn, qkv, self.qkv_rows)
                q = rope(qkv[:, : self.nh * hd].view(n, S, self.nh, hd))
                k = rope(qkv[:, self.nh * hd:(self.nh + self.nkv) * hd].view(n, S, self.nkv, hd))
                v = qkv[:, (self.nh + self.nkv) * hd:].view(n, S, self.nkv, hd)
                L["k"][b0:b0 + n, :, :S] = k.transpose(1, 2)
                L["v"][b0:b0 + n, :, :S] = v.transpose(1, 2)
                o = torch.nn.functional.scaled_dot_product_attention(
                    q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                    enable_gqa=self.nh != self.nkv)
                attn.copy_(o.transpose(1, 2).reshape(R, self.nh * hd))
                self._gemm_t(L["wo"], attn, x, cfg.hidden)
                norm_step(L["mlp_norm"])
                self._gemm_t(L["wgu"], xn, act, self.inter, dual=self.inter_pad)
                self._gemm_t(L["wd"], act, x, cfg.hidden)
                nw = self.layers[li + 1]["attn_norm"] if li + 1 < cfg.n_layers else self.final_norm
                norm_step(nw)
            last = xn.view(n, S, H)[:, S - 1].contiguous()
            logits = torch.empty(n, self.vshard, device=dev, dtype=torch.float32)
            self._gemm_t(self.lm_head, last, logits, self.vshard)
            val, idx = logits.max(dim=-1)
            if self.world > 1:
                mine = torch.stack([val, (idx + self.rank * self.vshard).float()], dim=-1).contiguous()
                allb = torch.empty(self.world, n, 2, device=dev)
                self.comm.all_gather(mine, allb)
                win = allb[:, :, 0].argmax(dim=0)
                idx = allb[:, :, 1].gather(0, win[None, :])[0].to(torch.int64)
            self.tokens[b0:b0 + n] = idx
        self.positions[:B] = S
        torch.cuda.synchronize(dev)

    # ------------------------------------------------------------------------------------
    def reference_decode_step(self, B):
        """Plain PyTorch fp32 restatement of one decode step on this rank's shard plus
        torch.distributed all_reduces; the oracle of the numerics tests. Does not touch the
        caches or the positions; returns the logits shard [B, vocab / world] of the next token."""
        cfg = self.cfg
        hd = cfg.head_dim
        tokens = self.tokens[:B]
        pos = self.positions[:B].long()

        def allreduce(t):
            if self.world > 1:
                t = t.clone()
                self.comm.all_reduce(t)
            return t

        def rms(t, w):
            tf = t.float()
            n = (tf * torch.rsqrt(tf.pow(2).mean(-1, keepdim=True) + cfg.eps)).to(torch.bfloat16)
            return (n.float() * w.float()).to(torch.bfloat16)

        x = torch.empty(B, cfg.hidden, device=self.device, dtype=torch.bfloat16)
        self._embed_partial(tokens, x)
        h = allreduce(x)
        cos = self.cos[pos][:, None, :]
        sin = self.sin[pos][:, None, :]

        def rope(t):  # [B, heads, hd] fp32
            t1, t2 = t[..., : hd // 2], t[..., hd // 2:]
            return torch.cat([t1 * cos - t2 * sin, t2 * cos + t1 * sin], dim=-1)

        xn = rms(h, self.layers[0]["attn_norm"])
        for li, L in enumerate(self.layers):
            D = self.dense_weights(L)
            qkv = (xn.float() @ D["wqkv"].float().t()).to(torch.bfloat16).float()
            q = rope(qkv[:, : self.nh * hd].view(B, self.nh, hd))
            k = rope(qkv[:, self.nh * hd:(self.nh + self.nkv) * hd].view(B, self.nkv, hd)).to(torch.bfloat16).float()
            v = qkv[:, (self.nh + self.nkv) * hd:].view(B, self.nkv, hd)
            outs = []
            for b in range(B):
                p = int(pos[b])
                kk = torch.cat([L["k"][b, :, :p].float(), k[b][:, None, :]], dim=1)  # [nkv, p+1, hd]
                vv = torch.cat([L["v"][b, :, :p].float(), v[b][:, None, :]], dim=1)
                rep = self.nh // self.nkv
                kk = kk.repeat_interleave(rep, 0)
                vv = vv.repeat_interleave(rep, 0)
                s = torch.einsum("hd,htd->ht", q[b], kk) / math.sqrt(hd)
                outs.append(torch.einsum("ht,htd->hd", s.softmax(-1), vv).reshape(-1))
            attn = torch.stack(outs).to(torch.bfloat16)
            o = allreduce((attn.float() @ D["wo"].float().t()).to(torch.bfloat16))
            h = (o.float() + h.float()).to(torch.bfloat16)
            xn = rms(h, L["mlp_norm"])
            act = (torch.nn.functional.silu(xn.float() @ D["wg"].float().t()) * (xn.float() @ D["wu"].float().t())).to(torch.bfloat16)
            d = allreduce((act.float() @ D["wd"].float().t()).to(torch.bfloat16))
            h = (d.float() + h.float()).to(torch.bfloat16)
            nw = self.layers[li + 1]["attn_norm"] if li + 1 < cfg.n_layers else self.final_norm
            xn = rms(h, nw)
        return xn.float() @ unpack_weight(self.lm_head, self.vshard, cfg.hidden).float().t()
