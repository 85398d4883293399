"""Process bootstrap and pickled-object collectives for the single-axis (HF-style) runner.

Parity: llm/utils/env/hf_dist_helper.py:12-331 — rank / world discovery from the launcher's
environment (torchrun, slurm, Open MPI, MVAPICH), ``setup_distributed`` (nccl or gloo), and
``all_gather`` / ``gather_pk`` / ``broadcast_object`` of arbitrary Python objects over a lazily
created **gloo** side group (so no GPU memory or NCCL kernels are used for control data).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

_GLOO = None


def env_rank_world():
    e = os.environ
    for rk, wk, lk in (("RANK", "WORLD_SIZE", "LOCAL_RANK"), ("SLURM_PROCID", "SLURM_NTASKS", "SLURM_LOCALID"),
                       ("OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_RANK"),
                       ("MV2_COMM_WORLD_RANK", "MV2_COMM_WORLD_SIZE", "MV2_COMM_WORLD_LOCAL_RANK")):
        if rk in e and wk in e:
            return int(e[rk]), int(e[wk]), int(e.get(lk, 0))
    return 0, 1, 0


def get_rank():
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else env_rank_world()[0]


def get_world_size():
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else env_rank_world()[1]


def get_local_rank():
    return env_rank_world()[2]


def barrier():
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def setup_distributed(port=13333, launcher="torch", backend="nccl"):
    from .grid import initialize_distributed
    if backend == "nccl" and not torch.cuda.is_available():
        backend = "gloo"
    return initialize_distributed(1, 1, backend=backend, launcher=launcher, port=port)


def _gloo_group():
    global _GLOO
    if _GLOO is None:
        _GLOO = dist.group.WORLD if dist.get_backend() == "gloo" else dist.new_group(backend="gloo")
    return _GLOO


def all_gather_object(obj):
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return [obj]
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, obj, group=_gloo_group())
    return out


all_gather = all_gather_object


def gather_pk(obj, dst=0):
    parts = all_gather_object(obj)
    return parts if get_rank() == dst else None


def broadcast_object(obj, src=0):
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return obj
    box = [obj if get_rank() == src else None]
    dist.broadcast_object_list(box, src=src, group=_gloo_group())
    return box[0]
