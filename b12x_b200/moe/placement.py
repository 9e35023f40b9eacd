"""Placement of replicated experts for expert parallelism under skewed routing.

With experts block-partitioned over the ranks, the rank that owns a hot expert sets the step time
(a Zipf(1.2) load over eight experts on eight ranks leaves the average rank at a third of the
hottest one).  Each rank therefore keeps a few spare expert slots; hot experts are copied into the
spare slots of cold ranks, and the routes of such an expert are spread over its holders in
sixteenths.  Every holder computes the same bytes for a route, so the layer's output does not depend
on the placement.  The reference library has no counterpart (its ``ep_moe`` replicates the INPUT and
leaves the sum to the caller, ``b12x/moe/ep_moe/_impl.py:1-14``).

This module is host-side arithmetic only (no torch, no CUDA): the same plan must come out on every
rank from the same loads."""

from __future__ import annotations

from dataclasses import dataclass

PATTERN = 16          # routes of an expert are dealt to its holders by (flat route index) % PATTERN


@dataclass(frozen=True)
class ReplicaPlan:
    """``holders[e]`` = ((rank, local slot, sixteenths), ...) with the owner first; ``extra[r]`` = the
    global ids of the experts copied into rank r's spare slots, in slot order (local id = experts per
    rank + position)."""

    world: int
    experts_per_rank: int
    slots_per_rank: int
    holders: tuple[tuple[tuple[int, int, int], ...], ...]
    extra: tuple[tuple[int, ...], ...]

    def pattern_tables(self) -> tuple[list[int], list[int]]:
        """Flat ``[E * 16]`` tables of the destination rank and the local expert id per pattern entry."""
        ranks: list[int] = []
        local: list[int] = []
        for hs in self.holders:
            row_r: list[int] = []
            row_l: list[int] = []
            for rank, slot, share in hs:
                row_r += [rank] * share
                row_l += [slot] * share
            assert len(row_r) == PATTERN
            # interleave the holders over the sixteen entries so that short runs of routes spread too
            order = sorted(range(PATTERN), key=lambda i: ((i * 7) % PATTERN))
            ranks += [row_r[i] for i in order]
            local += [row_l[i] for i in order]
        return ranks, local

    def rank_loads(self, loads: list[float]) -> list[float]:
        out = [0.0] * self.world
        for e, hs in enumerate(self.holders):
            for rank, _slot, share in hs:
                out[rank] += loads[e] * share / PATTERN
        return out


def _sixteenths(shares: list[float]) -> list[int]:
    """Largest-remainder rounding of fractions (sum 1) to sixteenths; every positive share keeps >= 1."""
    raw = [s * PATTERN for s in shares]
    out = [max(int(r), 1 if r > 0 else 0) for r in raw]
    while sum(out) > PATTERN:
        i = max(range(len(out)), key=lambda j: (out[j] - raw[j], out[j]))
        out[i] -= 1
    while sum(out) < PATTERN:
        i = max(range(len(out)), key=lambda j: raw[j] - out[j])
        out[i] += 1
    return out


def plan_expert_replicas(loads: list[float], world: int, slots_per_rank: int) -> ReplicaPlan:
    """Greedy water-filling: while the hottest rank is above the mean, move part of its largest
    expert share to the coldest rank that has a spare slot (or already holds that expert).

    ``loads[e]`` = fraction of all routes that go to expert e (any non-negative numbers; they are
    normalised).  Expert e is owned by rank ``e // (E / world)``."""
    num = len(loads)
    if world < 1 or num % world:
        raise ValueError("experts must divide evenly over the ranks")
    if slots_per_rank < 0:
        raise ValueError("slots_per_rank must be >= 0")
    per = num // world
    total = float(sum(loads))
    frac = [(x / total if total > 0 else 1.0 / num) for x in loads]
    # share[e] = {rank: fraction of ALL routes that go to expert e on that rank}
    share: list[dict[int, float]] = [{e // per: frac[e]} for e in range(num)]
    extra: list[list[int]] = [[] for _ in range(world)]
    rank_load = [sum(frac[r * per:(r + 1) * per]) for r in range(world)]
    target = 1.0 / world
    for _ in range(4 * world * max(slots_per_rank, 1)):
        hot = max(range(world), key=lambda r: (rank_load[r], -r))
        if rank_load[hot] <= target * 1.02:
            break
        # the largest share on the hot rank
        e = max((x for x in range(num) if hot in share[x]), key=lambda x: (share[x][hot], -x))
        cands = [r for r in range(world) if r != hot and rank_load[r] < target
                 and (r in share[e] or len(extra[r]) < slots_per_rank)]
        if not cands:
            break
        cold = min(cands, key=lambda r: (rank_load[r], r))
        move = min(rank_load[hot] - target, target - rank_load[cold], share[e][hot] * 15.0 / 16.0)
        if move <= 1e-9:
            break
        if cold not in share[e]:
            extra[cold].append(e)
        share[e][cold] = share[e].get(cold, 0.0) + move
        share[e][hot] -= move
        rank_load[hot] -= move
        rank_load[cold] += move
    holders = []
    for e in range(num):
        owner = e // per
        ranks = [owner] + sorted(r for r in share[e] if r != owner)
        sixteenths = _sixteenths([share[e][r] / frac[e] if frac[e] > 0 else (1.0 if r == owner else 0.0) for r in ranks])
        hs = []
        for r, q in zip(ranks, sixteenths):
            if q == 0:
                continue
            slot = (e - owner * per) if r == owner else per + extra[r].index(e)
            hs.append((r, slot, q))
        if not hs or hs[0][0] != owner:
            # the owner always keeps a share (its weights are there anyway)
            hs = [(owner, e - owner * per, 0)] + hs
            give = max(range(1, len(hs)), key=lambda i: hs[i][2])
            hs[0] = (owner, hs[0][1], 1)
            hs[give] = (hs[give][0], hs[give][1], hs[give][2] - 1)
        holders.append(tuple(h for h in hs if h[2] > 0))
    # a spare slot whose expert lost its last sixteenth to rounding stays allocated (weights are
    # copied into it) but receives no routes
    return ReplicaPlan(world, per, slots_per_rank, tuple(holders), tuple(tuple(x) for x in extra))
