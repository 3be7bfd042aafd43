"""Full-shard data parallelism (ZeRO-3 style) built on the fused collectives of the `ccl` backend.

Every wrapped unit (typically one transformer layer) keeps only its 1/world shard of a flat bf16
parameter, an fp32 master copy of that shard and an fp32 gradient shard. Around the unit's compute:

  * un-shard: ONE all_gather whose pieces land directly in the unit's full flat parameter buffer
    (`ops.all_gather_copy_out`; the module's parameters are views of that buffer, so there is no
    copy-out pass afterwards);
  * gradients accumulate in views of one flat bf16 gradient buffer; ONE reduce_scatter then sums
    them over the ranks, averages, and writes fp32 into the gradient shard in the same kernel
    (`ops.reduce_scatter_cast`: no separate divide and no separate cast).

Activations inside a unit are recomputed in backward (the unit runs under no_grad in forward), so
only unit boundaries are kept. The all_gather of the next unit (previous unit in backward) is
prefetched on a side stream while the current unit computes.

`comm="c10d"` runs the same schedule with plain torch.distributed calls (all_gather_into_tensor,
reduce_scatter_tensor, then divide and cast) on any backend; it is the comparison arm of the
benchmarks and the oracle of the tests.

The reference enables FSDP only as a workload on top of its collectives (tests/test_fsdp.py:113-180
of intel/torch-ccl wraps a CNN in torch's FSDP); torch's own FSDP also runs unmodified on this
backend. This engine exists to exercise the fused reduce_scatter / all_gather kernels.
"""
import torch
import torch.distributed as dist

from .. import ops


class _SymmPool:
    """Two symmetric buffers (memory of the group's symmetric heap, mapped by every rank) used in
    turn by consecutive units, so that the collectives on them run zero-copy: the all_gather writes
    straight into every rank's parameter buffer and the reduce_scatter reads the peers' gradient
    buffers in place (through the NVSwitch reduction when the heap is bound to a multicast object).
    `free[slot]` is the event after which the slot may be overwritten."""

    def __init__(self, numel, dtype, group, slots=2):
        from .. import symm_empty

        self.bufs = [symm_empty(numel, dtype, group=group) for _ in range(slots)]
        self.free = [None] * slots


class ShardedUnit:
    def __init__(self, module, group=None, comm="ccl", param_dtype=torch.bfloat16):
        self.module = module
        self.group = group
        self.comm = comm
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.params = [p for p in module.parameters()]
        dev = self.params[0].device
        self.device = dev
        self.dtype = param_dtype
        self.meta = []
        off = 0
        for p in self.params:
            self.meta.append((off, p.numel(), p.shape))
            off += p.numel()
        align = self.world * 8  # shards stay 16-byte aligned
        self.total = off
        self.padded = (off + align - 1) // align * align
        self.shard_numel = self.padded // self.world
        flat = torch.zeros(self.padded, device=dev, dtype=param_dtype)
        for p, (o, n, _) in zip(self.params, self.meta):
            flat[o:o + n] = p.data.to(param_dtype).view(-1)
        lo = self.rank * self.shard_numel
        self.shard = flat[lo:lo + self.shard_numel].clone()
        self.master = self.shard.float()               # fp32 master weights of the shard
        self.grad_shard = torch.zeros_like(self.master)  # fp32 gradient of the shard
        self._rs_out = torch.empty_like(self.master)
        del flat
        for p in self.params:
            p.data = torch.empty(0, device=dev, dtype=param_dtype)
        self.full = None
        self.gfull = None
        self.ready = None  # event: gathered parameters are complete
        self.ppool = self.gpool = None  # symmetric buffer pools of the engine (optional)
        self.slot = 0

    # -- parameters ---------------------------------------------------------------------------
    def gather(self, stream):
        """All-gather the flat parameter; parameters become views of the gathered buffer."""
        if self.full is not None:
            return
        cur = torch.cuda.current_stream(self.device)
        s = stream
        with torch.cuda.stream(s):
            if self.ppool is not None:
                if self.ppool.free[self.slot] is not None:
                    s.wait_event(self.ppool.free[self.slot])  # the unit that used this slot before has finished computing
                full = self.ppool.bufs[self.slot][: self.padded]
            else:
                full = torch.empty(self.padded, device=self.device, dtype=self.dtype)
            if self.comm == "ccl":
                ops.all_gather_copy_out(self.shard, list(full.chunk(self.world)), group=self.group)
            else:
                dist.all_gather_into_tensor(full, self.shard, group=self.group)
            self.ready = torch.cuda.Event()
            self.ready.record(s)
        if self.ppool is None:
            full.record_stream(cur)
        self.full = full
        for p, (o, n, shape) in zip(self.params, self.meta):
            p.data = full[o:o + n].view(shape)

    def wait_ready(self):
        if self.ready is not None:
            torch.cuda.current_stream(self.device).wait_event(self.ready)

    def release(self):
        if self.ppool is not None and self.full is not None:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self.ppool.free[self.slot] = ev
        self.full = None
        self.ready = None
        for p in self.params:
            p.data = torch.empty(0, device=self.device, dtype=self.dtype)

    # -- gradients ----------------------------------------------------------------------------
    def prepare_grads(self):
        if self.gpool is not None:
            if self.gpool.free[self.slot] is not None:
                torch.cuda.current_stream(self.device).wait_event(self.gpool.free[self.slot])  # its last reduce_scatter is done
            self.gfull = self.gpool.bufs[self.slot][: self.padded]
            self.gfull.zero_()
        else:
            self.gfull = torch.zeros(self.padded, device=self.device, dtype=self.dtype)
        for p, (o, n, shape) in zip(self.params, self.meta):
            p.grad = self.gfull[o:o + n].view(shape)

    def reduce_grads(self, stream):
        """grad_shard += mean over ranks of this rank's piece of the flat gradient (fp32).

        Runs on `stream` — the same stream as the parameter gathers: the kernels of one
        communicator must never run concurrently, so all of the engine's collectives share one
        stream and are ordered against the compute stream with events."""
        cur = torch.cuda.current_stream(self.device)
        done = torch.cuda.Event()
        done.record(cur)
        gfull = self.gfull
        with torch.cuda.stream(stream):
            stream.wait_event(done)
            if self.comm == "ccl":
                ops.reduce_scatter_cast(gfull, self._rs_out, scale=1.0 / self.world, group=self.group)
                self.grad_shard += self._rs_out
            else:
                tmp = torch.empty(self.shard_numel, device=self.device, dtype=self.dtype)
                dist.reduce_scatter_tensor(tmp, gfull, group=self.group)
                self.grad_shard += tmp.float() / self.world
            if self.gpool is not None:
                ev = torch.cuda.Event()
                ev.record(stream)
                self.gpool.free[self.slot] = ev
        if self.gpool is None:
            gfull.record_stream(stream)
        for p in self.params:
            p.grad = None
        self.gfull = None

    def optimizer_views(self):
        """(fp32 master shard with .grad set) for an optimizer; call `sync_shard` after the step."""
        self.master.grad = self.grad_shard
        return self.master

    def sync_shard(self):
        self.shard.copy_(self.master)
        self.grad_shard.zero_()


class _UnitFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, anchor, engine, index):
        unit = engine.units[index]
        unit.gather(engine.comm_stream)
        unit.wait_ready()
        if index + 1 < len(engine.units):
            engine.units[index + 1].gather(engine.comm_stream)  # prefetch
        with torch.no_grad():
            y = unit.module(x)
        unit.release()
        ctx.engine, ctx.index = engine, index
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, gy):
        engine, index = ctx.engine, ctx.index
        unit = engine.units[index]
        (x,) = ctx.saved_tensors
        unit.gather(engine.comm_stream)
        unit.wait_ready()
        if index > 0:
            engine.units[index - 1].gather(engine.comm_stream)  # prefetch for the previous unit
        unit.prepare_grads()
        with torch.enable_grad():
            xd = x.detach().requires_grad_(x.is_floating_point())
            y = unit.module(xd)
        torch.autograd.backward(y, gy)
        unit.reduce_grads(engine.comm_stream)
        unit.release()
        return (xd.grad if xd.requires_grad else None), None, None, None


class FullyShardedSequential:
    """A chain of modules, each sharded as one unit: y = m_n(...m_1(x))."""

    def __init__(self, modules, group=None, comm="ccl", param_dtype=torch.bfloat16, comm_blocks=None, symmetric=False):
        """comm_blocks: CTA cap of the collective kernels of this group's communicator. The gathers and
        reduce_scatters of this engine run NEXT TO the units' compute; with the default cap (256 CTAs of
        512 threads) they take every SM away from the GEMMs they are supposed to hide behind. A cap of
        32-64 leaves most of the GPU to the compute while the NVLink transfer still runs near full rate.
        The setting applies to every collective of the group (all ranks must pass the same value).
        symmetric: keep the gathered parameters and the flat gradients in two pairs of buffers from the
        group's symmetric heap (CCL_SYMM_HEAP_MB must hold four buffers of the largest unit), so that both
        collectives run zero-copy over NVLink instead of staging through the arena."""
        self.units = [ShardedUnit(m, group, comm, param_dtype) for m in modules]
        if comm == "ccl" and symmetric and self.units[0].world > 1:
            biggest = max(u.padded for u in self.units)
            ppool = _SymmPool(biggest, param_dtype, group)
            gpool = _SymmPool(biggest, param_dtype, group)
            for i, u in enumerate(self.units):
                u.ppool, u.gpool, u.slot = ppool, gpool, i % 2
        if comm == "ccl" and comm_blocks:
            from .. import get_backend

            get_backend(group, "cuda").set_cuda_tuning(self.units[0].shard, {"max_blocks": int(comm_blocks)})
        self.comm_stream = torch.cuda.Stream()
        self.anchor = torch.zeros((), device=self.units[0].device, requires_grad=True)
        self.group = group

    def __call__(self, x):
        # `anchor` requires grad, so every unit's backward runs even when the chain starts from
        # token ids (which cannot carry gradients themselves)
        for i in range(len(self.units)):
            x = _UnitFn.apply(x, self.anchor, self, i)
        return x

    def finish_backward(self):
        """The gradient reduce_scatters run on the communication stream: join it."""
        torch.cuda.current_stream(self.units[0].device).wait_stream(self.comm_stream)

    def master_params(self):
        """fp32 master shards with their gradient shards attached (call after backward)."""
        self.finish_backward()
        return [u.optimizer_views() for u in self.units]

    def after_step(self):
        for u in self.units:
            u.sync_shard()
        # the next forward's gathers (communication stream) must see the updated shards
        self.comm_stream.wait_stream(torch.cuda.current_stream(self.units[0].device))

    # -- checkpoints ------------------------------------------------------------------------------
    def sharded_state_dict(self):
        """This rank's part of a checkpoint: the fp32 master shard of every unit (CPU tensors).

        Every rank saves its own file; no communication. Reload with `load_sharded_state_dict` on
        the same world size. (The reference only shows `model.state_dict()` + `torch.save` after a
        barrier in its FSDP example, tests/test_fsdp.py:172-178.)"""
        w, r = self.units[0].world, self.units[0].rank
        return {"world": w, "rank": r,
                "units": [{"numel": u.total, "padded": u.padded, "master": u.master.detach().cpu().clone()} for u in self.units]}

    def load_sharded_state_dict(self, sd):
        w, r = self.units[0].world, self.units[0].rank
        if sd["world"] != w or sd["rank"] != r or len(sd["units"]) != len(self.units):
            raise ValueError("sharded checkpoint of rank %d/%d with %d units does not fit rank %d/%d with %d units"
                             % (sd["rank"], sd["world"], len(sd["units"]), r, w, len(self.units)))
        for u, e in zip(self.units, sd["units"]):
            if e["numel"] != u.total or e["padded"] != u.padded:
                raise ValueError("sharded checkpoint: unit size mismatch")
            u.master.copy_(e["master"])
            u.sync_shard()
        self.comm_stream.wait_stream(torch.cuda.current_stream(self.units[0].device))

    def full_state_dict(self, dst=0):
        """Consolidated fp32 parameters {"<unit>.<name>": tensor} on rank `dst` (None elsewhere):
        one all_gather of the master shards per unit through torch.distributed."""
        self.finish_backward()  # gradient reduce_scatters may still be running on the communication stream
        out = {} if self.units[0].rank == dst else None
        for i, u in enumerate(self.units):
            full = torch.empty(u.padded, device=u.device, dtype=torch.float32)
            dist.all_gather_into_tensor(full, u.master, group=self.group)
            if out is not None:
                for (name, _), (o, n, shape) in zip(u.module.named_parameters(), u.meta):
                    out["%d.%s" % (i, name)] = full[o:o + n].view(shape).cpu()
        return out
