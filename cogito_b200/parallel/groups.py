"""Rank arithmetic and process groups of the DP x TP x PP layout.

The mapping is the reference's (src/pipeline/pipeline.c:150-152):
``tp_rank = r % tp``, ``pp_rank = (r / tp) % pp``, ``dp_rank = r / (tp * pp)``, with
group colours tp: ``dp*pp + pp_rank``, pp: ``dp*tp + tp_rank``, dp: ``pp_rank*tp + tp_rank``
(:160,165,170).  The reference stops at the arithmetic (its communicator split is
commented out); here the groups are real ``torch.distributed`` groups (NCCL on GPUs,
gloo on CPU ranks).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch.distributed as dist


@dataclass
class Coords:
    rank: int
    dp: int
    tp: int
    pp: int
    dp_rank: int = 0
    tp_rank: int = 0
    pp_rank: int = 0

    def __post_init__(self):
        if self.dp * self.tp * self.pp <= 0:
            raise ValueError("dp, tp, pp must be positive")
        self.tp_rank = self.rank % self.tp
        self.pp_rank = (self.rank // self.tp) % self.pp
        self.dp_rank = self.rank // (self.tp * self.pp)

    @property
    def world(self) -> int:
        return self.dp * self.tp * self.pp

    def tp_color(self) -> int:
        return self.dp_rank * self.pp + self.pp_rank

    def pp_color(self) -> int:
        return self.dp_rank * self.tp + self.tp_rank

    def dp_color(self) -> int:
        return self.pp_rank * self.tp + self.tp_rank


def rank_of(dp_rank: int, pp_rank: int, tp_rank: int, tp: int, pp: int) -> int:
    return (dp_rank * pp + pp_rank) * tp + tp_rank


def group_ranks(world: int, dp: int, tp: int, pp: int):
    """The rank lists of every tp / pp / dp group, keyed by colour."""
    if dp * tp * pp != world:
        raise ValueError(f"dp*tp*pp = {dp * tp * pp} does not match world size {world}")
    tp_groups, pp_groups, dp_groups = {}, {}, {}
    for r in range(world):
        c = Coords(r, dp, tp, pp)
        tp_groups.setdefault(c.tp_color(), []).append(r)
        pp_groups.setdefault(c.pp_color(), []).append(r)
        dp_groups.setdefault(c.dp_color(), []).append(r)
    return tp_groups, pp_groups, dp_groups


@dataclass
class ParallelContext:
    """Coordinates of this rank plus its three process groups."""
    coords: Coords
    tp_group: object = None
    pp_group: object = None
    dp_group: object = None
    mp_group: object = None          # all ranks of one model replica (same dp rank)
    tp_ranks: list = field(default_factory=list)
    pp_ranks: list = field(default_factory=list)
    dp_ranks: list = field(default_factory=list)
    mp_ranks: list = field(default_factory=list)
    # one two-rank group per pipeline neighbour and direction: 'recv_fwd' (from the previous stage),
    # 'send_fwd' (to the next), 'recv_bwd' (from the next), 'send_bwd' (to the previous).  Each carries
    # the transfers of one direction between one pair of stages, in micro-batch order, on its own
    # communicator, so that a receive posted early never sits in front of a send to the other neighbour.
    pipeline_links: dict = field(default_factory=dict)

    @property
    def prev_stage(self) -> int | None:
        c = self.coords
        return None if c.pp_rank == 0 else rank_of(c.dp_rank, c.pp_rank - 1, c.tp_rank, c.tp, c.pp)

    @property
    def next_stage(self) -> int | None:
        c = self.coords
        return None if c.pp_rank == c.pp - 1 else rank_of(c.dp_rank, c.pp_rank + 1, c.tp_rank, c.tp, c.pp)


def init_parallel(dp: int = 1, tp: int = 1, pp: int = 1, pipeline_links: bool = True) -> ParallelContext:
    """Create the tp / pp / dp groups (collective: every rank of the world calls it), and with
    ``pipeline_links`` the per-neighbour, per-direction groups of the pipeline transfers."""
    import os
    if pp > 1:
        # point-to-point kernels of the pipeline run beside compute kernels: keep them to a few CTAs
        # (the executor leaves that many SMs free); must be set before the communicators exist
        os.environ.setdefault("NCCL_MAX_P2P_NCHANNELS", "2")
    if not dist.is_initialized():
        if dp * tp * pp != 1:
            raise RuntimeError("torch.distributed is not initialised")
        return ParallelContext(Coords(0, 1, 1, 1), tp_ranks=[0], pp_ranks=[0], dp_ranks=[0])
    world, rank = dist.get_world_size(), dist.get_rank()
    tpg, ppg, dpg = group_ranks(world, dp, tp, pp)
    ctx = ParallelContext(Coords(rank, dp, tp, pp))
    for groups, attr, rattr in ((tpg, "tp_group", "tp_ranks"), (ppg, "pp_group", "pp_ranks"),
                                (dpg, "dp_group", "dp_ranks")):
        for colour in sorted(groups):
            ranks = groups[colour]
            g = dist.new_group(ranks)          # every rank creates every group, in the same order
            if rank in ranks:
                setattr(ctx, attr, g)
                setattr(ctx, rattr, ranks)
    for d in range(dp):
        ranks = [r for r in range(world) if Coords(r, dp, tp, pp).dp_rank == d]
        g = dist.new_group(ranks)
        if rank in ranks:
            ctx.mp_group, ctx.mp_ranks = g, ranks
    if pp > 1 and pipeline_links:
        for colour in sorted(ppg):
            ranks = ppg[colour]                     # the stages of one pipeline, first to last
            for a, b in zip(ranks[:-1], ranks[1:]):
                fwd, bwd = dist.new_group([a, b]), dist.new_group([a, b])
                if rank == a:
                    ctx.pipeline_links["send_fwd"], ctx.pipeline_links["recv_bwd"] = fwd, bwd
                if rank == b:
                    ctx.pipeline_links["recv_fwd"], ctx.pipeline_links["send_bwd"] = fwd, bwd
    return ctx
