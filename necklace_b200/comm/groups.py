"""Process-group registry and topology math for every trainer mode.

``init_nccl_groups_map(tmode, cfg)`` computes, for a trainer-mode string such as
``"dp+pp+mp"`` and the sizes in ``cfg``, which ranks form each data- / pipeline- /
tensor- / ZeRO-parallel group, and records the groups this rank belongs to.  The
nesting rule is the reference's (necklace/cuda/ncclgrp.py:584-767): kinds are
taken in the order they appear in the mode string, the first is outermost
(largest stride) and the last is innermost (contiguous ranks).  Unlike the
reference's hand-written 2-, 3- and 4-way cases this is one formula for any
number of kinds.  Function names match the reference module so user scripts port
unchanged (getters at ncclgrp.py:288-382).

Group objects here are pure descriptions (``GroupInfo``); communicators are
attached later with ``attach_comm`` by whichever backend the worker uses
(peer-memory ``PeerGroup``, ``TorchGroup``).
"""
from __future__ import annotations

from functools import reduce

KINDS = ("dp", "pp", "mp", "zr")

# Modes of the reference's tnmode list (necklace/trainer/tnmode.py:3-20).
SUPPORTED_MODES = ("no", "dp", "pp", "mp", "zr", "dp+pp", "dp+mp", "dp+pp+mp", "dp+zr", "zr+mp",
                   "dp+zr+mp")
UNSUPPORTED_MODES = ("pp+mp", "zr+pp", "zr+pp+mp", "dp+zr+pp", "dp+zr+pp+mp")


class GroupInfo:
    """One process group as seen from this rank.

    ``pg_ranks``: sorted global ranks; ``pg_rank``: my global rank;
    ``rank``: my index inside the group; ``ranks``: ``range(world_size)``.
    """

    def __init__(self, pg_rank: int, pg_ranks: list[int], kind: str = "main"):
        self.kind = kind
        self.pg_rank = pg_rank
        self.pg_ranks = sorted(pg_ranks)
        self.world_size = len(self.pg_ranks)
        self.ranks = list(range(self.world_size))
        self.rank = self.pg_ranks.index(pg_rank) if pg_rank in self.pg_ranks else -1
        self.comm = None  # backend communicator (PeerGroup / TorchGroup), attached later

    def to_cfg_dict(self) -> dict:
        return {"pg_rank": self.pg_rank, "pg_ranks": list(self.pg_ranks), "rank": self.rank,
                "ranks": list(self.ranks), "world_size": self.world_size}

    def attach_comm(self, comm) -> None:
        self.comm = comm

    def __repr__(self):
        return f"GroupInfo({self.kind}, rank {self.rank}/{self.world_size}, {self.pg_ranks})"


# the reference's name of the group object (necklace/cuda/ncclgrp.py:24-60)
NcclProcessGroup = GroupInfo


class _State:
    def __init__(self):
        self.reset()

    def reset(self):
        self.inited = False
        self.tmode = None
        self.main: GroupInfo | None = None
        self.main_world_size = None
        self.main_rank = None
        self.mine: dict[str, GroupInfo] = {}      # "<kind>_group" -> my group
        self.all: dict[str, list[list[int]]] = {}  # "<kind>_group" -> every group's ranks
        self.sizes: dict[str, int] = {}


_S = _State()


def ensure_divisibility(numerator: int, denominator: int) -> None:
    assert numerator % denominator == 0, f"{numerator} is not divisible by {denominator}"


def divide(numerator: int, denominator: int) -> int:
    ensure_divisibility(numerator, denominator)
    return numerator // denominator


def parse_tmode(tmode: str) -> list[str]:
    tmode = (tmode or "no").strip()
    if tmode == "no":
        return []
    kinds = tmode.split("+")
    for k in kinds:
        if k not in KINDS:
            raise ValueError(f"unknown parallelism kind {k!r} in trainer mode {tmode!r}")
    if len(set(kinds)) != len(kinds):
        raise ValueError(f"repeated kind in trainer mode {tmode!r}")
    return kinds


def calc_groups(world_size: int, kinds: list[str], sizes: dict[str, int]) -> dict[str, list]:
    """All groups of every kind.  ``kinds[0]`` is outermost.  Rank r has coordinates
    (c_0, ..., c_{k-1}) with r = sum c_i * stride_i, stride_i = prod(sizes[kinds[j]], j > i);
    a group of kind i holds the ranks that differ only in c_i."""
    if not kinds:
        return {}
    if len(kinds) == 1:
        return {kinds[0] + "_group": [list(range(world_size))]}
    szs = [int(sizes.get(k) or 0) for k in kinds]
    known = reduce(lambda a, b: a * b, [s for s in szs if s > 0], 1)
    if szs.count(0) == 1:
        szs[szs.index(0)] = divide(world_size, known)
    if any(s <= 0 for s in szs):
        raise ValueError(f"sizes for {kinds} are under-specified: {sizes}")
    if reduce(lambda a, b: a * b, szs, 1) != world_size:
        raise ValueError(f"sizes {dict(zip(kinds, szs))} do not multiply to world size "
                         f"{world_size}")
    strides = [reduce(lambda a, b: a * b, szs[i + 1:], 1) for i in range(len(szs))]
    out = {}
    for i, k in enumerate(kinds):
        groups = {}
        for r in range(world_size):
            c_i = (r // strides[i]) % szs[i]
            base = r - c_i * strides[i]
            groups.setdefault(base, []).append(r)
        out[k + "_group"] = [sorted(v) for _, v in sorted(groups.items())]
    return out


# reference-named helpers for the fixed-arity cases (necklace/cuda/ncclgrp.py:672-767)
def calc_pgs_p2(world_size, aa_size, bb_size):
    g = calc_groups(world_size, ["dp", "mp"], {"dp": aa_size, "mp": bb_size})
    return g["dp_group"], g["mp_group"]


def calc_pgs_p3(world_size, aa_size, bb_size, cc_size):
    g = calc_groups(world_size, ["dp", "pp", "mp"], {"dp": aa_size, "pp": bb_size, "mp": cc_size})
    return g["dp_group"], g["pp_group"], g["mp_group"]


def calc_pgs_p4(world_size, aa_size, bb_size, cc_size, dd_size):
    g = calc_groups(world_size, ["dp", "zr", "pp", "mp"],
                    {"dp": aa_size, "zr": bb_size, "pp": cc_size, "mp": dd_size})
    return g["dp_group"], g["zr_group"], g["pp_group"], g["mp_group"]


def build_nccl_pgs_map(tmode: str, cfg: dict | None = None):
    cfg = cfg or {}
    world_size, my_rank = cfg.get("world_size"), cfg.get("my_rank")
    if world_size is None or my_rank is None:
        raise ValueError(f"cannot build the group map: ({tmode}) [{cfg}]")
    if world_size < 1:
        raise ValueError(f"world_size ({world_size}) should be >= 1")
    kinds = parse_tmode(tmode)
    sizes = {k: cfg.get(k + "_size") for k in KINDS}
    pgs = calc_groups(world_size, kinds, sizes)
    pgs_sz = {k: len(v[0]) for k, v in pgs.items()}
    return pgs, pgs_sz


def init_nccl_group_main(world_size: int, my_rank: int) -> GroupInfo:
    _S.main = GroupInfo(my_rank, list(range(world_size)), "main")
    _S.main_world_size, _S.main_rank = world_size, my_rank
    return _S.main


def init_nccl_pgs_map(tmode: str, cfg: dict | None = None) -> None:
    cfg = cfg or {}
    world_size, my_rank = cfg.get("world_size"), cfg.get("my_rank")
    is_worker = cfg.get("is_worker", True)
    pgs, pgs_sz = build_nccl_pgs_map(tmode, cfg)
    _S.tmode, _S.all, _S.sizes = tmode, pgs, pgs_sz
    init_nccl_group_main(world_size, my_rank)
    _S.mine = {}
    if is_worker:
        for key, groups in pgs.items():
            for ranks in groups:
                if my_rank in ranks:
                    _S.mine[key] = GroupInfo(my_rank, ranks, key[:2])


def init_nccl_groups_map(tmode: str, cfg: dict | None = None, verbose: bool = False) -> None:
    """Idempotent (the reference guards with a module flag, ncclgrp.py:388-397)."""
    if not _S.inited:
        init_nccl_pgs_map(tmode, cfg)
        if verbose:
            print("NCCL_GROUPS_MAP", {k: v.to_cfg_dict() for k, v in _S.mine.items()})
            print("NCCL_GROUPS_GRP_MAP", _S.all)
    _S.inited = True


def reset_nccl_groups_map() -> None:
    """Forget everything (tests; re-initialisation after an elastic restart)."""
    _S.reset()


def get_nccl_groups_map() -> dict:
    return _S.mine


def get_nccl_groups_map_cfg_dict() -> dict:
    return {k: v.to_cfg_dict() for k, v in _S.mine.items()}


def get_nccl_groups_map_grp_dict() -> dict:
    return _S.all


def get_nccl_group_main_grp_list() -> list[int]:
    return list(range(_S.main_world_size or 0))


def get_nccl_group_main(*a, **k):
    return _S.main


def get_nccl_group_main_world_size(*a, **k):
    return _S.main_world_size


def get_nccl_group_main_rank(*a, **k):
    return _S.main_rank


# -- the reference's builder-level entry points (necklace/cuda/ncclgrp.py:62-121, :429-500): a
# script that assembles its groups by hand instead of from a trainer mode uses these ----------
def build_pg_cfg(pg_rank, pg_ranks):
    return {"pg_rank": pg_rank, "pg_ranks": list(pg_ranks)}


def make_pg_by_nk(nk, comm_i, pg_rank, pg_ranks):
    """A group object for ``pg_ranks`` as seen from global rank ``pg_rank``.  ``nk`` (a
    communicator to attach, may be ``None``) and ``comm_i`` keep the reference's positions; the
    communicator can also be attached later with ``attach_comm``."""
    g = GroupInfo(pg_rank, list(pg_ranks))
    if nk is not None:
        g.attach_comm(nk)
    return g


def make_pg_by_nc(nc, pg_rank, pg_ranks):
    return make_pg_by_nk(nc, None, pg_rank, pg_ranks)


def set_nccl_group_main_world_size(world_size):
    _S.main_world_size = world_size


def set_nccl_group_main_rank(rank):
    _S.main_rank = rank


def set_nccl_group_main_by_nc(nc, world_size):
    """The main group of ``world_size`` ranks around an existing communicator ``nc`` (its
    ``rank`` attribute is this process's global rank)."""
    rank = int(getattr(nc, "rank", _S.main_rank or 0))
    _S.main = make_pg_by_nk(nc, None, rank, list(range(world_size)))
    _S.main.kind = "main"
    _S.main_world_size, _S.main_rank = world_size, rank
    return _S.main


def get_nccl_main_nk(*a, **k):
    """The communicator of the main group (``None`` before bring-up)."""
    return getattr(_S.main, "comm", None)


def set_nccl_groups_map(pg_map):
    _S.mine = dict(pg_map)


def init_nccl_group_pg(pg, group, ranks):
    """Register ``group`` as this rank's group of kind ``pg`` (``'dp_group'``, ...)."""
    assert pg not in _S.mine, f"{pg} is already initialized"
    group.kind = pg[:2]
    _S.mine[pg] = group


def init_nccl_group_pgs(world_size, my_rank, pgs_dl, pgs_sz=None, is_worker=True):
    """Groups from explicit rank lists: ``pgs_dl = {'dp_group': [[0, 2], [1, 3]], ...}``."""
    for pg, grp in pgs_dl.items():
        if is_worker:
            for ranks in grp:
                if my_rank in ranks:
                    init_nccl_group_pg(pg, make_pg_by_nk(None, None, my_rank, ranks), ranks)
        _S.all[pg] = [list(r) for r in grp]
        _S.sizes[pg] = len(grp[0]) if grp else 0


def _get(kind):
    return _S.mine.get(kind + "_group")


def get_nccl_group_dp(*a, **k):
    return _get("dp")


def get_nccl_group_mp(*a, **k):
    return _get("mp")


def get_nccl_group_pp(*a, **k):
    return _get("pp")


def get_nccl_group_zr(*a, **k):
    return _get("zr")


def get_nccl_group_dp_or_main(*a, **k):
    return _get("dp") or _S.main


def get_nccl_group_mp_or_main(*a, **k):
    return _get("mp") or _S.main


def get_nccl_group_pp_or_main(*a, **k):
    return _get("pp") or _S.main


def get_nccl_group_zr_or_main(*a, **k):
    return _get("zr") or _S.main


def get_rank(group=None) -> int:
    group = group or _S.main
    if group is None:
        return _S.main_rank
    return group.rank


def get_world_size(group=None) -> int:
    group = group or _S.main
    if group is None:
        return _S.main_world_size
    return group.world_size


def del_nccl_groups_map_comms() -> None:
    for g in list(_S.mine.values()) + ([_S.main] if _S.main else []):
        g.comm = None
