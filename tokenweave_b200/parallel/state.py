"""Process-group state: one process per GPU, ``torch.distributed`` (NCCL on GPUs, gloo on CPU) for
the plumbing, a gloo twin group for host-side control messages.

Counterpart of vllm/distributed/parallel_state.py:802-949. The job's ranks form ``pp`` pipeline stages
of ``tp`` tensor-parallel ranks each (stage ``s`` = global ranks ``[s * tp, (s + 1) * tp)``, the layout of
``parallel_state.py:906-933``). ``TPState.rank`` / ``world_size`` / ``group`` always describe the
tensor-parallel group of this process, so everything written for TP runs unchanged inside a stage;
activations cross stage boundaries with point-to-point sends between equal tensor-parallel ranks.
The TokenWeave runs of the reference use TP = 4 / 8 with PP = 1.
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
    # pipeline parallelism (1 stage: everything below is the identity)
    pp_rank: int = 0
    pp_size: int = 1
    global_rank: int = 0
    global_size: int = 1
    world_cpu_group: Optional[dist.ProcessGroup] = None   # host control plane over all stages

    @property
    def is_first_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_stage(self) -> bool:
        return self.pp_rank == self.pp_size - 1


_STATE = TPState()
_SUBGROUPS: list = []       # groups made by new_group here, destroyed (newest first) before the world group


def _new_group(*args, **kwargs):
    g = dist.new_group(*args, **kwargs)
    _SUBGROUPS.append(g)
    return g


def get_tp() -> TPState:
    return _STATE


def tp_rank() -> int:
    return _STATE.rank


def tp_world_size() -> int:
    return _STATE.world_size


_init_generation = 0
_BASE_STORES: dict = {}


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
    # one store (server on rank 0, one client connection elsewhere) per address for the life of the process:
    # a second engine in the same process finds it again instead of binding the port a second time
    key = (host, int(port), rank, world_size)
    base = _BASE_STORES.get(key)
    if base is None:
        base = dist.TCPStore(host, int(port), world_size, is_master=(rank == 0 and not agent_store),
                             timeout=datetime.timedelta(seconds=timeout_s), wait_for_workers=False)
        _BASE_STORES[key] = base
    return dist.PrefixStore(f"tw_init_{gen}", base)


def init_distributed(rank: int, world_size: int, local_rank: Optional[int] = None, device: str = "auto",
                     init_method: Optional[str] = None, timeout_s: float = 600.0,
                     tp_size: Optional[int] = None) -> TPState:
    """Join (or create) the job's process group and bind this process to its GPU. ``tp_size`` smaller than
    ``world_size`` makes ``world_size / tp_size`` pipeline stages."""
    global _STATE
    tp_size = world_size if tp_size is None else tp_size
    if world_size % tp_size:
        raise ValueError(f"world size {world_size} is not a multiple of the tensor-parallel size {tp_size}")
    pp_size = world_size // tp_size
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
        cpu_group = _new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s)) if use_cuda else group
    if pp_size == 1:
        _STATE = TPState(rank, world_size, local_rank, dev, group, cpu_group, owns, global_rank=rank,
                         global_size=world_size, world_cpu_group=cpu_group)
        return _STATE
    # several stages: one tensor-parallel group (and its gloo twin) per stage; every rank creates all of them,
    # in the same order, as torch.distributed requires
    world_cpu, tp_group, tp_cpu = cpu_group, None, None
    if tp_size > 1:
        for s in range(pp_size):
            ranks = list(range(s * tp_size, (s + 1) * tp_size))
            g = _new_group(ranks, backend="nccl" if use_cuda else "gloo", timeout=datetime.timedelta(seconds=timeout_s))
            cg = _new_group(ranks, backend="gloo", timeout=datetime.timedelta(seconds=timeout_s)) if use_cuda else g
            if rank in ranks:
                tp_group, tp_cpu = g, cg
    _STATE = TPState(rank % tp_size, tp_size, local_rank, dev, tp_group, tp_cpu, owns, pp_rank=rank // tp_size,
                     pp_size=pp_size, global_rank=rank, global_size=world_size, world_cpu_group=world_cpu)
    return _STATE


def send_to_next_stage(*tensors: torch.Tensor) -> None:
    """Hand tensors to the same tensor-parallel rank of the next pipeline stage (blocking sends, in order)."""
    dst = _STATE.global_rank + _STATE.world_size
    for t in tensors:
        dist.send(t, dst=dst)


def recv_from_prev_stage(*tensors: torch.Tensor) -> None:
    src = _STATE.global_rank - _STATE.world_size
    for t in tensors:
        dist.recv(t, src=src)


def broadcast_from_last_stage(obj):
    """The step result lives on the last stage; every rank of the job gets a copy (host control plane)."""
    if _STATE.pp_size == 1:
        return obj
    box = [obj]
    dist.broadcast_object_list(box, src=(_STATE.pp_size - 1) * _STATE.world_size, group=_STATE.world_cpu_group)
    return box[0]


def set_single_process(device: torch.device) -> TPState:
    global _STATE
    _STATE = TPState(0, 1, device.index or 0, device, None, None, False)
    return _STATE


def destroy_distributed() -> None:
    """Leave the job's process groups. Every rank first meets the others on the host control plane, so no
    rank tears its sockets down while a peer still has traffic (or a gloo worker thread) on them; the
    sub-groups go before the world group they were carved from."""
    global _STATE
    if _STATE.owns_process_group and dist.is_initialized():
        try:
            if _STATE.world_cpu_group is not None:
                dist.barrier(group=_STATE.world_cpu_group, async_op=True).wait(datetime.timedelta(seconds=20))
        except Exception:            # a peer that died or hangs: do not wait for it
            pass
        while _SUBGROUPS:
            g = _SUBGROUPS.pop()
            try:
                dist.destroy_process_group(g)
            except Exception:
                pass
        dist.destroy_process_group()
    _SUBGROUPS.clear()
    _STATE = TPState()


def cpu_barrier() -> None:
    if _STATE.cpu_group is not None:
        dist.barrier(group=_STATE.cpu_group)


def broadcast_object(obj, src: int = 0):
    """Broadcast inside the tensor-parallel group; ``src`` is a rank of that group."""
    if _STATE.world_size == 1:
        return obj
    box = [obj]
    dist.broadcast_object_list(box, src=dist.get_global_rank(_STATE.cpu_group, src), group=_STATE.cpu_group)
    return box[0]
