"""Comparison arm of the headline benchmark: the same tensor-parallel Llama decode step written in
plain PyTorch on the stock stack - torch.matmul (cuBLAS) for every projection,
scaled_dot_product_attention over the KV cache, torch.nn.functional.rms_norm, eager RoPE and
KV append, torch.distributed all_reduce / all_gather on an NCCL group - captured in one CUDA
graph like the repo's own arm. None of this repository's kernels run here. Same shapes, same
sharding (heads and FFN columns split over the ranks, vocabulary-parallel embedding and lm_head),
same batch, same context length, random N(0, 0.02) bf16 weights.

This is the A/B switch the reference ships in its own sweeps (the same script on the `nccl`
backend: tests/ddp_allreduce.py:54-59 of intel/torch-ccl) applied to its tensor-parallel decode
loop (tests/test_allreduce.py:49-76)."""
import torch
import torch.distributed as dist
import torch.nn.functional as F


class TorchTPDecoder:
    def __init__(self, cfg, batch, context, kv_len, group=None, device=None, seed=0):
        self.cfg = cfg
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.group = group
        W, dev = self.world, self.device
        H, hd = cfg.hidden, cfg.head_dim
        self.nh, self.nkv, self.inter, self.vshard = cfg.n_heads // W, cfg.n_kv_heads // W, cfg.inter // W, cfg.vocab // W
        g = torch.Generator(device=dev)
        g.manual_seed(seed * 7919 + self.rank)

        def rnd(*shape):
            return (torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)

        self.layers = []
        for _ in range(cfg.n_layers):
            self.layers.append(dict(
                wqkv=rnd((self.nh + 2 * self.nkv) * hd, H), wo=rnd(H, self.nh * hd), wg=rnd(self.inter, H), wu=rnd(self.inter, H),
                wd=rnd(H, self.inter), n1=torch.ones(H, device=dev, dtype=torch.bfloat16), n2=torch.ones(H, device=dev, dtype=torch.bfloat16),
                # the cache holds a random "prompt": decode speed does not depend on its values
                k=rnd(batch, self.nkv, kv_len, hd), v=rnd(batch, self.nkv, kv_len, hd)))
        self.embed = rnd(self.vshard, H)
        self.lm_head = rnd(self.vshard, H)
        self.final_norm = torch.ones(H, device=dev, dtype=torch.bfloat16)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, device=dev, dtype=torch.float32) / hd))
        ang = torch.arange(kv_len, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
        self.batch, self.kv_len = batch, kv_len
        self.tokens = torch.randint(0, cfg.vocab, (batch,), device=dev)
        self.next_tokens = torch.zeros(batch, device=dev, dtype=torch.int64)
        self.positions = torch.full((batch,), context, device=dev, dtype=torch.int64)
        self.rows = torch.arange(batch, device=dev)
        self.kpos = torch.arange(kv_len, device=dev)
        self.graph = None

    def _all_reduce(self, t):
        if self.world > 1:
            dist.all_reduce(t, group=self.group)

    def _body(self):
        cfg, B, hd = self.cfg, self.batch, self.cfg.head_dim
        tok = self.tokens - self.rank * self.vshard
        ok = (tok >= 0) & (tok < self.vshard)
        h = self.embed[tok.clamp(0, self.vshard - 1)] * ok[:, None].to(torch.bfloat16)
        self._all_reduce(h)
        pos = self.positions
        cos, sin = self.cos[pos][:, None, :], self.sin[pos][:, None, :]
        mask = (self.kpos[None, :] <= pos[:, None])[:, None, None, :]

        def rope(t):
            t1, t2 = t[..., : hd // 2], t[..., hd // 2:]
            return torch.cat([t1 * cos - t2 * sin, t2 * cos + t1 * sin], dim=-1)

        for L in self.layers:
            xn = F.rms_norm(h, (cfg.hidden,), L["n1"], cfg.eps)
            qkv = xn @ L["wqkv"].t()
            q = rope(qkv[:, : self.nh * hd].view(B, self.nh, hd))
            k = rope(qkv[:, self.nh * hd:(self.nh + self.nkv) * hd].view(B, self.nkv, hd))
            v = qkv[:, (self.nh + self.nkv) * hd:].view(B, self.nkv, hd)
            L["k"][self.rows, :, pos] = k
            L["v"][self.rows, :, pos] = v
            o = F.scaled_dot_product_attention(q[:, :, None, :], L["k"], L["v"], attn_mask=mask, enable_gqa=self.nh != self.nkv)
            o = o.reshape(B, self.nh * hd) @ L["wo"].t()
            self._all_reduce(o)
            h = h + o
            xn = F.rms_norm(h, (cfg.hidden,), L["n2"], cfg.eps)
            d = (F.silu(xn @ L["wg"].t()) * (xn @ L["wu"].t())) @ L["wd"].t()
            self._all_reduce(d)
            h = h + d
        logits = (F.rms_norm(h, (cfg.hidden,), self.final_norm, cfg.eps) @ self.lm_head.t()).float()
        val, idx = logits.max(dim=-1)
        if self.world > 1:
            mine = torch.stack([val, (idx + self.rank * self.vshard).float()], dim=-1)
            allb = torch.empty(self.world, B, 2, device=self.device)
            dist.all_gather_into_tensor(allb, mine, group=self.group)
            win = allb[:, :, 0].argmax(dim=0)
            idx = allb[:, :, 1].gather(0, win[None, :])[0].to(torch.int64)
        self.next_tokens.copy_(idx)
        self.tokens.copy_(idx)
        self.positions += 1

    def capture(self):
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        saved = self.positions.clone(), self.tokens.clone()
        with torch.cuda.stream(s), torch.no_grad():
            for _ in range(2):
                self._body()
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        self.positions.copy_(saved[0])
        self.tokens.copy_(saved[1])
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s), torch.no_grad():
            self._body()
        self.graph = g
        torch.cuda.synchronize(self.device)

    def decode_step(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            with torch.no_grad():
                self._body()
        return self.next_tokens

    def decode_step_host(self, tokens_pinned, out_pinned):
        self.tokens.copy_(tokens_pinned, non_blocking=True)
        self.decode_step()
        out_pinned.copy_(self.next_tokens, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return out_pinned


def step_bytes(cfg, batch, context):
    """Bytes one decode step must stream from HBM over all ranks: every weight once plus the KV cache."""
    H, hd = cfg.hidden, cfg.head_dim
    per_layer = H * ((cfg.n_heads + 2 * cfg.n_kv_heads) * hd + cfg.n_heads * hd + 3 * cfg.inter)
    weights = 2 * (cfg.n_layers * per_layer + H * cfg.vocab)
    kv = 2 * cfg.n_layers * batch * cfg.n_kv_heads * hd * 2 * (context + 1)
    return weights + kv
