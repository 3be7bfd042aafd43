"""Collectives over a two-level rank layout: `ranks_per_node` ranks share a node-local group, and the ranks with the same
local index on every node share a cross-node group.

The CUDA communicator of this backend spans the GPUs of ONE node (peer memory over NVLink / NVSwitch). A job on several
nodes therefore keeps its bandwidth-heavy traffic inside the node-local `ccl` groups and crosses nodes with 1/ranks_per_node
of the data, through whichever backend serves the cross groups (NCCL over the network, or `ccl` itself when the "nodes" are
slices of one machine, which is how the tests run it):

    all_reduce      = reduce_scatter inside the node -> all_reduce across nodes -> all_gather inside the node
    broadcast       = across nodes between the ranks with the root's local index -> inside every node
    all_gather      = inside the node -> across nodes (node-major order, i.e. the order of the global ranks)
    reduce_scatter  = across nodes on the node-sized slices -> inside the node

The reference gets the same effect from oneCCL's own topology-aware algorithms below its API (its binding only hands the
global communicator to the library, src/ccl_comm_collector.cpp:10-45); here the composition is explicit and the groups are
ordinary `torch.distributed` groups.
"""
import torch
import torch.distributed as dist


class HierarchicalGroups:
    """Builds the node and cross groups (collective: every rank of the default group must construct it, with the same
    arguments) and runs the composed collectives on contiguous tensors."""

    def __init__(self, ranks_per_node, intra_backend=None, cross_backend=None):
        world, rank = dist.get_world_size(), dist.get_rank()
        if ranks_per_node < 1 or world % ranks_per_node != 0:
            raise ValueError(f"ranks_per_node={ranks_per_node} does not divide the world size {world}")
        self.world, self.rank = world, rank
        self.per = ranks_per_node
        self.nodes = world // ranks_per_node
        self.node, self.local = rank // ranks_per_node, rank % ranks_per_node
        self.intra = self.cross = None
        # new_group is collective over the default group: every rank creates every group, in the same order
        for n in range(self.nodes):
            g = dist.new_group(list(range(n * self.per, (n + 1) * self.per)), backend=intra_backend)
            if n == self.node:
                self.intra = g
        for l in range(self.per):
            g = dist.new_group([n * self.per + l for n in range(self.nodes)], backend=cross_backend)
            if l == self.local:
                self.cross = g

    def all_reduce(self, tensor, op=dist.ReduceOp.SUM):
        """In place. The element count is padded up to a multiple of ranks_per_node internally."""
        if not tensor.is_contiguous():
            tmp = tensor.contiguous()
            self.all_reduce(tmp, op=op)
            tensor.copy_(tmp)
            return
        if self.nodes == 1:
            return dist.all_reduce(tensor, op=op, group=self.intra)
        if self.per == 1:
            return dist.all_reduce(tensor, op=op, group=self.cross)
        flat = tensor.view(-1)
        n = flat.numel()
        shard_n = (n + self.per - 1) // self.per
        if shard_n * self.per != n:
            padded = flat.new_zeros(shard_n * self.per)
            padded[:n] = flat
        else:
            padded = flat
        shard = torch.empty(shard_n, dtype=flat.dtype, device=flat.device)
        dist.reduce_scatter_tensor(shard, padded, op=op, group=self.intra)
        dist.all_reduce(shard, op=op, group=self.cross)
        dist.all_gather_into_tensor(padded, shard, group=self.intra)
        if padded is not flat:
            flat.copy_(padded[:n])

    def broadcast(self, tensor, src):
        src_node, src_local = src // self.per, src % self.per
        if self.nodes > 1 and self.local == src_local:
            dist.broadcast(tensor, src=src, group=self.cross)
        if self.per > 1:
            dist.broadcast(tensor, src=self.node * self.per + src_local, group=self.intra)

    def all_gather_into_tensor(self, output, input):
        """output[r * n:(r + 1) * n] = rank r's input, for the global ranks r in order."""
        n = input.numel()
        out = output.reshape(-1)
        if self.nodes == 1:
            return dist.all_gather_into_tensor(out, input.reshape(-1), group=self.intra)
        node_part = out[self.node * self.per * n:(self.node + 1) * self.per * n]
        dist.all_gather_into_tensor(node_part, input.reshape(-1), group=self.intra)
        # every local index forwards the same node-sized block; one of them per node would be enough, all of them keep
        # the call symmetric and cost the same time
        dist.all_gather_into_tensor(out, node_part.clone(), group=self.cross)

    def reduce_scatter_tensor(self, output, input, op=dist.ReduceOp.SUM):
        """output = slice `rank` of the reduction of the ranks' inputs (input has world * output.numel() elements)."""
        n = output.numel()
        inp = input.reshape(-1)
        if self.nodes == 1:
            return dist.reduce_scatter_tensor(output.reshape(-1), inp, op=op, group=self.intra)
        # across nodes first: this rank's cross group reduces the node-sized slices, rank `node` of it keeps slice `node`
        node_slice = torch.empty(self.per * n, dtype=inp.dtype, device=inp.device)
        dist.reduce_scatter_tensor(node_slice, inp, op=op, group=self.cross)
        dist.reduce_scatter_tensor(output.reshape(-1), node_slice, op=op, group=self.intra)
