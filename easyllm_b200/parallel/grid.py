"""3D process grid: tensor (TP) × pipeline (PP) × data (DP) parallel groups.

Rank layout parity with llm/utils/env/dist_env/dist_helper.py:58-176:
``rank = pp · (DP·TP) + dp · TP + tp``; TP groups are contiguous ranks, DP groups stride TP
inside one pipeline block, PP groups stride ``world / PP``, MODEL groups hold every
(tp, pp) of one dp index, EMBEDDING groups hold the first and last stage of each pipe.

``grid_layout`` is a pure function (no process group needed) so the tables can be checked
on one CPU process; ``ParallelGrid`` materialises the groups with ``torch.distributed``
(NCCL on GPUs, gloo on CPU).  On one 8×B200 box every group rides NVSwitch, so group
placement never has to account for link topology — only for which ranks share a kernel's
symmetric-memory heap (the TP group and the DP group).
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class GridLayout:
    world: int
    tp: int
    pp: int
    dp: int
    tp_groups: List[List[int]] = field(default_factory=list)
    pp_groups: List[List[int]] = field(default_factory=list)
    dp_groups: List[List[int]] = field(default_factory=list)
    mp_groups: List[List[int]] = field(default_factory=list)
    emb_groups: List[List[int]] = field(default_factory=list)

    def coords(self, rank):
        """(pp, dp, tp) coordinates of a global rank."""
        per_stage = self.dp * self.tp
        return rank // per_stage, (rank % per_stage) // self.tp, rank % self.tp

    def rank_of(self, pp, dp, tp):
        return pp * self.dp * self.tp + dp * self.tp + tp


def grid_layout(world: int, tp: int = 1, pp: int = 1) -> GridLayout:
    tp = min(tp, world)
    pp = min(pp, world)
    if world % (tp * pp):
        raise ValueError(f"world size {world} is not divisible by tp*pp = {tp * pp}")
    dp = world // (tp * pp)
    g = GridLayout(world, tp, pp, dp)
    per_stage = dp * tp
    for s in range(pp):
        for t in range(tp):
            g.dp_groups.append([s * per_stage + d * tp + t for d in range(dp)])
    for d in range(dp):
        g.mp_groups.append([grp[d] for grp in g.dp_groups])
    for i in range(world // tp):
        g.tp_groups.append(list(range(i * tp, (i + 1) * tp)))
    for i in range(per_stage):
        ranks = list(range(i, world, per_stage))
        g.pp_groups.append(ranks)
        g.emb_groups.append([ranks[0], ranks[-1]] if len(ranks) > 1 else list(ranks))
    return g


class ParallelGrid:
    """Holds the process groups of this rank.  A single instance is installed globally."""

    def __init__(self, tp=1, pp=1, backend=None, timeout_s=1800):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        self.layout = grid_layout(self.world, tp, pp)
        self.tp, self.pp, self.dp = self.layout.tp, self.layout.pp, self.layout.dp
        self.pp_rank, self.dp_rank, self.tp_rank = self.layout.coords(self.rank)
        self._timeout = datetime.timedelta(seconds=timeout_s)
        self.dp_group, self.dp_ranks = self._make(self.layout.dp_groups)
        self.mp_group, self.mp_ranks = self._make(self.layout.mp_groups)
        self.tp_group, self.tp_ranks = self._make(self.layout.tp_groups)
        self.pp_group, self.pp_ranks = self._make(self.layout.pp_groups)
        self.emb_group, self.emb_ranks = self._make(self.layout.emb_groups)
        # pipeline p2p: one group (one communicator, one stream) per direction, so activations flowing down and
        # gradients flowing up never queue behind each other, and a CPU group for the shape headers of dynamic
        # micro-batches (read on the host without touching the GPU)
        self.pp_fwd_group = self.pp_bwd_group = self.pp_host_group = None
        if self.pp > 1:
            self.pp_fwd_group, _ = self._make(self.layout.pp_groups)
            self.pp_bwd_group, _ = self._make(self.layout.pp_groups)
            self.pp_host_group, _ = self._make(self.layout.pp_groups, backend="gloo")
        self._gloo_world = None
        self.virtual_pp_rank = None
        self.virtual_pp_world = None

    def _make(self, tables, backend=None):
        mine, mine_ranks = None, None
        for ranks in tables:
            grp = dist.new_group(ranks, timeout=self._timeout, backend=backend)
            if self.rank in ranks:
                mine, mine_ranks = grp, list(ranks)
        return mine, mine_ranks

    # ---- stage helpers -------------------------------------------------------------
    def is_first_stage(self):
        return self.pp_rank == 0

    def is_last_stage(self):
        return self.pp_rank == self.pp - 1

    def next_stage_rank(self):
        return self.pp_ranks[(self.pp_rank + 1) % self.pp]

    def prev_stage_rank(self):
        return self.pp_ranks[(self.pp_rank - 1) % self.pp]

    def first_stage_rank(self):
        return self.pp_ranks[0]

    def last_stage_rank(self):
        return self.pp_ranks[-1]

    def tp_src_rank(self):
        """Global rank of tp index 0 in this rank's TP group."""
        return (self.rank // self.tp) * self.tp

    def gloo_world_group(self):
        """CPU side-channel for pickled objects and heartbeats (lazy)."""
        if self._gloo_world is None:
            if dist.get_backend() == "gloo":
                self._gloo_world = dist.group.WORLD
            else:
                self._gloo_world = dist.new_group(list(range(self.world)), backend="gloo")
        return self._gloo_world


_GRID: Optional[ParallelGrid] = None


class _Solo:
    """Grid stand-in for a single process without torch.distributed."""
    world = tp = pp = dp = 1
    rank = pp_rank = dp_rank = tp_rank = 0
    dp_group = mp_group = tp_group = pp_group = emb_group = None
    pp_fwd_group = pp_bwd_group = pp_host_group = None
    dp_ranks = mp_ranks = tp_ranks = pp_ranks = emb_ranks = [0]
    virtual_pp_rank = virtual_pp_world = None
    layout = grid_layout(1, 1, 1)

    def is_first_stage(self):
        return True

    def is_last_stage(self):
        return True

    def tp_src_rank(self):
        return 0

    def gloo_world_group(self):
        return None


_SOLO = _Solo()


def get_grid():
    return _GRID if _GRID is not None else _SOLO


def set_grid(g):
    global _GRID
    _GRID = g


def destroy_model_parallel():
    set_grid(None)


def initialize_model_parallel(tp=1, pp=1, virtual_pp=None, timeout_s=1800) -> ParallelGrid:
    g = ParallelGrid(tp, pp, timeout_s=timeout_s)
    if virtual_pp is not None:
        g.virtual_pp_rank, g.virtual_pp_world = 0, virtual_pp
    set_grid(g)
    return g


def model_parallel_is_initialized():
    return _GRID is not None


# ---- launcher bootstrap (dist_helper.py:408-516) ------------------------------------------
def _expand_slurm_nodelist(nodelist: str) -> str:
    """First host of a SLURM_NODELIST such as ``node[003-004,9],other1``."""
    head = nodelist.split(",")[0] if "[" not in nodelist.split(",")[0] else nodelist
    if "[" not in head:
        return head
    prefix, rest = head.split("[", 1)
    first = rest.split("]")[0].split(",")[0].split("-")[0]
    return prefix + first


def get_distributed_info(launcher="torch", port=13333):
    """Return (rank, world_size, local_rank) and export MASTER_* for the chosen launcher."""
    env = os.environ
    if launcher == "slurm" and "SLURM_PROCID" in env:
        rank, world = int(env["SLURM_PROCID"]), int(env["SLURM_NTASKS"])
        local = int(env.get("SLURM_LOCALID", 0))
        env.setdefault("MASTER_ADDR", _expand_slurm_nodelist(env.get("SLURM_NODELIST", "127.0.0.1")))
        env.setdefault("MASTER_PORT", str(port))
    elif launcher == "mpi" and "OMPI_COMM_WORLD_RANK" in env:
        rank, world = int(env["OMPI_COMM_WORLD_RANK"]), int(env["OMPI_COMM_WORLD_SIZE"])
        local = int(env.get("OMPI_COMM_WORLD_LOCAL_RANK", 0))
        env.setdefault("MASTER_ADDR", "127.0.0.1")
        env.setdefault("MASTER_PORT", str(port))
    else:
        rank, world = int(env.get("RANK", 0)), int(env.get("WORLD_SIZE", 1))
        local = int(env.get("LOCAL_RANK", 0))
        env.setdefault("MASTER_ADDR", "127.0.0.1")
        env.setdefault("MASTER_PORT", str(port))
    env["RANK"], env["WORLD_SIZE"], env["LOCAL_RANK"] = str(rank), str(world), str(local)
    return rank, world, local


def initialize_distributed(tp=1, pp=1, backend="nccl", launcher="torch", port=13333, timeout_s=1800):
    """Join the job (one process per GPU) and build the grid."""
    rank, world, local = get_distributed_info(launcher, port)
    if backend == "nccl" and not torch.cuda.is_available():
        backend = "gloo"
    if torch.cuda.is_available():
        ndev = torch.cuda.device_count()
        torch.cuda.set_device(local % ndev if ndev else 0)
    if not dist.is_initialized():
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return initialize_model_parallel(min(tp, world), min(pp, world), timeout_s=timeout_s)


# ---- module-level getters with the reference's names ----------------------------------------
def get_tensor_model_parallel_group(): return get_grid().tp_group
def get_pipeline_model_parallel_group(): return get_grid().pp_group
def get_data_parallel_group(): return get_grid().dp_group
def get_model_parallel_group(): return get_grid().mp_group
def get_embedding_group(): return get_grid().emb_group
def get_tensor_model_parallel_world_size(): return get_grid().tp
def get_pipeline_model_parallel_world_size(): return get_grid().pp
def get_data_parallel_world_size(): return get_grid().dp
def get_tensor_model_parallel_rank(): return get_grid().tp_rank
def get_pipeline_model_parallel_rank(): return get_grid().pp_rank
def get_data_parallel_rank(): return get_grid().dp_rank
def get_tensor_model_parallel_src_rank(): return get_grid().tp_src_rank()
def is_pipeline_first_stage(ignore_virtual=False): return get_grid().is_first_stage()
def is_pipeline_last_stage(ignore_virtual=False): return get_grid().is_last_stage()
