"""Process-group bootstrap and per-stage shard / replicate groups.

One process per GPU (or per CPU rank with gloo), identity from RANK / LOCAL_RANK /
WORLD_SIZE as set by torchrun — the reference reads the same variables
(utils/comm.py:42-110).  `StageGroups.create_all` creates the shard and replicate groups
of *every* stage on *every* rank in one fixed order, because `torch.distributed.new_group`
is collective over the world (reference zorse_utils/pipeline.py:58-63,
utils/comm.py:172-229); groups with identical membership are created once and shared.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.distributed as dist


def env_rank() -> int:
    return int(os.environ.get("RANK", "0"))


def env_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def env_world_size() -> int:
    return int(os.environ.get("WORLD_SIZE", "1"))


def dist_init(backend: Optional[str] = None, timeout_s: float = 300.0) -> torch.device:
    """Initialises torch.distributed (nccl on CUDA, gloo otherwise) and returns this rank's device.
    With WORLD_SIZE unset or 1 and no MASTER_ADDR the process runs standalone (no group)."""
    use_cuda = torch.cuda.is_available() and backend != "gloo"
    if use_cuda:
        torch.cuda.set_device(env_local_rank())
        device = torch.device("cuda", env_local_rank())
    else:
        device = torch.device("cpu")
    if dist.is_initialized():
        return device
    if env_world_size() == 1 and "MASTER_ADDR" not in os.environ:
        return device
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    be = backend or ("nccl" if use_cuda else "gloo")
    kw = {}
    if be == "nccl":
        kw["device_id"] = device
    dist.init_process_group(be, rank=env_rank(), world_size=env_world_size(),
                            timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return device


def is_dist() -> bool:
    return dist.is_available() and dist.is_initialized()


def world_size() -> int:
    return dist.get_world_size() if is_dist() else 1


def rank() -> int:
    return dist.get_rank() if is_dist() else 0


_gloo_world = None


def gloo_world_group(timeout_s: float = 300.0):
    """Host-side control group (barriers, metrics, heartbeats); the world group itself when
    the default backend already is gloo."""
    global _gloo_world
    if not is_dist():
        return None
    if dist.get_backend() == "gloo":
        return dist.group.WORLD
    if _gloo_world is None:
        _gloo_world = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))
    return _gloo_world


@dataclass
class Group:
    """A set of ranks with its torch process group (None when the set is a single rank or
    this process is not a member)."""
    ranks: tuple[int, ...]
    pg: object = None

    @property
    def size(self) -> int:
        return len(self.ranks)

    def index_of(self, r: int) -> int:
        return self.ranks.index(r)


class GroupCache:
    def __init__(self, timeout_s: float = 1800.0):
        self._cache: dict[tuple[int, ...], Group] = {}
        self.timeout_s = timeout_s

    def get(self, ranks: Sequence[int]) -> Group:
        key = tuple(ranks)
        if key not in self._cache:
            pg = None
            if len(key) > 1 and is_dist():
                pg = dist.new_group(ranks=list(key), timeout=datetime.timedelta(seconds=self.timeout_s))
            self._cache[key] = Group(key, pg)
        return self._cache[key]


@dataclass
class StageGroups:
    shard: Group
    replicate: Group
    tp: Optional[Group] = None   # the tensor-parallel group of this rank's lane (None when tp = 1)

    @staticmethod
    def create_all(stages, my_rank: int, cache: Optional[GroupCache] = None, tp: int = 1) -> dict[int, "StageGroups"]:
        """Creates every stage's groups on every rank (same order everywhere) and returns, per
        stage id this rank belongs to, its own shard / replicate groups.  With tensor parallelism
        the stage configs name lanes; process `l * tp + t` holds slice t of lane l, its shard and
        replicate groups connect the processes with the same t, its tensor-parallel group the tp
        processes of the lane.  `my_rank` and the ranks of the returned groups are process ranks."""
        cache = cache or GroupCache()
        mine: dict[int, StageGroups] = {}
        tp_group = None
        if tp > 1:
            lanes = sorted({r for st in stages for r in st.gpu_ranks})
            for lane in lanes:
                g = cache.get(tuple(lane * tp + i for i in range(tp)))
                if my_rank in g.ranks:
                    tp_group = g
        for t in range(tp):
            for st in stages:
                phys = lambda ranks: tuple(r * tp + t for r in ranks)
                shard_groups = [cache.get(phys(g)) for g in st.zero_config]
                width = len(st.zero_config[0])
                rep_groups = [cache.get(phys(tuple(g[j] for g in st.zero_config))) for j in range(width)]
                if my_rank % tp == t and my_rank // tp in st.gpu_ranks:
                    sg = next(g for g in shard_groups if my_rank in g.ranks)
                    rg = next(g for g in rep_groups if my_rank in g.ranks)
                    mine[st.stage_id] = StageGroups(sg, rg, tp_group)
        return mine
