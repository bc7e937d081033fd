"""Process-group plumbing: one process per GPU (torchrun style), NCCL on GPUs / gloo on CPU ranks.

``init_from_env`` reads RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT, creates the default
group with a bounded timeout (a rank that never joins ends the others' next collective with an error
instead of a hang), and returns the ``ParallelCtx`` the decoder uses. ``comm="fused"`` additionally
sets up the symmetric-memory communicator whose kernels do the reductions over NVLink peer loads.
"""
from __future__ import annotations

import datetime
import os
from typing import Optional

import torch

from .context import ParallelCtx


def no_multicast_default():
    """Call before the first symmetric-memory rendezvous of a process. By default no kernel of this library uses
    multimem, so the buffers need no NVLink multicast binding (``LB_MULTIMEM=1`` turns the multimem form of the
    prompt-sized reduction on and with it the binding); a rank that dies while its memory is bound to a multicast object
    can raise NVLink faults on its peers' GPUs. ``TORCH_SYMM_MEM_DISABLE_MULTICAST=0`` in the environment keeps
    PyTorch's default."""
    if os.environ.get("LB_MULTIMEM", "0") == "1":
        # opt-in: the prompt-sized reduction uses multimem.ld_reduce / multimem.st through the NVLink multicast
        # mapping of the symmetric buffer, which the rendezvous then has to create
        os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "0"
        return
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


def env_world():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def init_from_env(device: Optional[str] = None, comm: str = "fused", expert_parallel: bool = False,
                  timeout_s: float = 120.0, max_rows: int = 8192, hidden: int = 0) -> ParallelCtx:
    import torch.distributed as dist
    rank, local_rank, world = env_world()
    if world == 1:
        return ParallelCtx.single()
    use_cuda = (device or "cuda").startswith("cuda") and torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        kwargs = {}
        if use_cuda:
            kwargs["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    symm = None
    no_multicast_default()
    if comm == "fused" and use_cuda:
        from .symm import SymmComm
        symm = SymmComm(dist.group.WORLD, rank, world, torch.device("cuda", local_rank), max_rows, hidden)
    elif comm == "fused":
        comm = "nccl"
    return ParallelCtx(rank, world, dist.group.WORLD, expert_parallel, comm, symm)


def barrier():
    import torch.distributed as dist
    if dist.is_initialized():
        dist.barrier()


def all_reduce_max(x: float, device) -> float:
    import torch.distributed as dist
    if not dist.is_initialized():
        return x
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
