"""torch's own FullyShardedDataParallel and DistributedDataParallel running on the `ccl` backend.

The reference's FSDP test wraps an MNIST CNN, trains three batches and prints the loss without
asserting anything (tests/test_fsdp.py:113-180 of intel/torch-ccl; it needs torchvision and a
download). Here a small MLP on seeded random data takes two SGD steps under FSDP and must end with
the parameters of a single-process run on the union of the ranks' batches."""
import pytest
import torch
import torch.distributed as dist

from mp_util import run_ranks


def _data(rank, n, salt=0):
    g = torch.Generator().manual_seed(99 + 31 * rank + salt)
    return torch.randn(n, generator=g)


def _torch_fsdp(rank, world, device):
    import torch.nn as nn
    from torch.distributed.fsdp import FullyShardedDataParallel as FSDP

    dev = torch.device("cuda", torch.cuda.current_device()) if device == "cuda" else torch.device("cpu")

    def make():
        torch.manual_seed(0)
        return nn.Sequential(nn.Linear(32, 64), nn.Tanh(), nn.Linear(64, 8)).to(dev)

    model = FSDP(make(), device_id=dev)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    ref = make()
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
    losses = []
    for step in range(2):
        xs = [_data(r, 8 * 32, salt=step).view(8, 32).to(dev) for r in range(world)]
        opt.zero_grad()
        loss = model(xs[rank]).pow(2).mean()
        loss.backward()
        opt.step()
        losses.append(float(loss))
        ropt.zero_grad()
        (sum(ref(x).pow(2).mean() for x in xs) / world).backward()
        ropt.step()
    with FSDP.summon_full_params(model):
        for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
            torch.testing.assert_close(p.detach(), q.detach(), rtol=1e-4, atol=1e-5, msg=n)
    # the sharded state can be consolidated after a barrier, like the reference's --save-model path
    dist.barrier()
    with FSDP.summon_full_params(model):
        sd = {k: v.detach().cpu().clone() for k, v in model.state_dict().items()}
    assert len(sd) == 4


def _torch_fsdp2(rank, world, device):
    """FSDP2 (`fully_shard`, DTensor-based) uses the *_tensor_coalesced collectives of the backend."""
    import torch.nn as nn
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    dev = torch.device("cuda", torch.cuda.current_device()) if device == "cuda" else torch.device("cpu")

    def make():
        torch.manual_seed(0)
        return nn.Sequential(nn.Linear(32, 64), nn.Tanh(), nn.Linear(64, 8)).to(dev)

    model = make()
    mesh = init_device_mesh(device, (world,))
    for layer in model:
        if isinstance(layer, nn.Linear):
            fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    ref = make()
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
    for step in range(2):
        xs = [_data(r, 8 * 32, salt=step).view(8, 32).to(dev) for r in range(world)]
        opt.zero_grad()
        model(xs[rank]).pow(2).mean().backward()
        opt.step()
        ropt.zero_grad()
        (sum(ref(x).pow(2).mean() for x in xs) / world).backward()
        ropt.step()
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        torch.testing.assert_close(p.full_tensor().detach(), q.detach(), rtol=1e-4, atol=1e-5, msg=n)
    dist.barrier()


def test_torch_fsdp2_cpu_world2():
    run_ranks(_torch_fsdp2, world=2, args=("cpu",))


@pytest.mark.gpu
@pytest.mark.multigpu
def test_torch_fsdp2_cuda():
    run_ranks(_torch_fsdp2, world=min(torch.cuda.device_count(), 8), device="cuda", args=("cuda",), env={"NCCL_NVLS_ENABLE": "0"}, timeout=150)


def test_torch_fsdp_cpu_world2():
    run_ranks(_torch_fsdp, world=2, args=("cpu",))


@pytest.mark.gpu
@pytest.mark.multigpu
def test_torch_fsdp_cuda():
    run_ranks(_torch_fsdp, world=min(torch.cuda.device_count(), 8), device="cuda", args=("cuda",), env={"NCCL_NVLS_ENABLE": "0"}, timeout=150)
