"""Process-group state: one process per GPU, ``torch.distributed`` (NCCL on GPUs, gloo on CPU) for
the plumbing, a gloo twin group for host-side control messages.

Counterpart of vllm/distributed/parallel_state.py:802-949. Only tensor parallelism is modelled:
the TokenWeave path of the reference runs TP=4/8 with PP=DP=1 (its V1 multiprocess executor asserts
world_size == tp, vllm/v1/executor/multiproc_executor.py:56-59).
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class TPState:
    rank: int = 0
    world_size: int = 1
    local_rank: int = 0
    device: torch.device = torch.device("cpu")
    group: Optional[dist.ProcessGroup] = None       # device collectives (NCCL / gloo)
    cpu_group: Optional[dist.ProcessGroup] = None   # host control plane (gloo)
    owns_process_group: bool = False


_STATE = TPState()


def get_tp() -> TPState:
    return _STATE


def tp_rank() -> int:
    return _STATE.rank


def tp_world_size() -> int:
    return _STATE.world_size


_init_generation = 0


def _generation_store(init_method: str, rank: int, world_size: int, timeout_s: float):
    """Rendezvous store for ``tcp://host:port`` with a per-initialisation key prefix.

    A process that builds several engines one after another re-initialises the process group against
    the same TCP store (under ``torch.distributed.run`` the launcher's store outlives every group),
    and torch restarts its group counter on destroy, so the second group would find the first one's
    keys — a stale NCCL unique id among them, which a rank that runs ahead of rank 0 then reads.
    Prefixing every generation's keys keeps them apart."""
    global _init_generation
    if not init_method.startswith("tcp://"):
        return None
    host, _, port = init_method[len("tcp://"):].partition(":")
    gen = _init_generation
    _init_generation += 1
    agent_store = os.environ.get("TORCHELASTIC_USE_AGENT_STORE", "") == "True"
    base = dist.TCPStore(host, int(port), world_size, is_master=(rank == 0 and not agent_store),
                         timeout=datetime.timedelta(seconds=timeout_s), wait_for_workers=False)
    return dist.PrefixStore(f"tw_init_{gen}", base)


def init_distributed(rank: int, world_size: int, local_rank: Optional[int] = None, device: str = "auto",
                     init_method: Optional[str] = None, timeout_s: float = 600.0) -> TPState:
    """Join (or create) the job's process group and bind this process to its GPU."""
    global _STATE
    local_rank = rank if local_rank is None else local_rank
    use_cuda = (device == "cuda") or (device == "auto" and torch.cuda.is_available())
    if use_cuda:
        torch.cuda.set_device(local_rank)
        dev = torch.device("cuda", local_rank)
    else:
        dev = torch.device("cpu")
    owns = False
    group = cpu_group = None
    if world_size > 1:
        if not dist.is_initialized():
            if init_method is None:
                addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
                port = os.environ.get("MASTER_PORT", "29611")
                init_method = f"tcp://{addr}:{port}"
            kwargs = dict(backend="nccl" if use_cuda else "gloo", rank=rank, world_size=world_size,
                          timeout=datetime.timedelta(seconds=timeout_s))
            if use_cuda:
                kwargs["device_id"] = dev
            store = _generation_store(init_method, rank, world_size, timeout_s)
            if store is not None:
                kwargs["store"] = store
            else:
                kwargs["init_method"] = init_method
            dist.init_process_group(**kwargs)
            owns = True
        group = dist.group.WORLD
        cpu_group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s)) if use_cuda else group
    _STATE = TPState(rank, world_size, local_rank, dev, group, cpu_group, owns)
    return _STATE


def set_single_process(device: torch.device) -> TPState:
    global _STATE
    _STATE = TPState(0, 1, device.index or 0, device, None, None, False)
    return _STATE


def destroy_distributed() -> None:
    global _STATE
    if _STATE.owns_process_group and dist.is_initialized():
        dist.destroy_process_group()
    _STATE = TPState()


def cpu_barrier() -> None:
    if _STATE.cpu_group is not None:
        dist.barrier(group=_STATE.cpu_group)


def broadcast_object(obj, src: int = 0):
    if _STATE.world_size == 1:
        return obj
    box = [obj]
    dist.broadcast_object_list(box, src=src, group=_STATE.cpu_group)
    return box[0]
