"""Rank-group enumeration for a mixed TP/CP/DP/PP layout.

A global rank is a mixed-radix number whose digits are the coordinates along
the dimensions listed in ``order`` (first = fastest varying).  A group for a
token such as ``"tp"`` or ``"dp-cp"`` is the set of ranks that agree on every
digit *not* named by the token.  The resulting tables equal the reference's
(nano_megatron/parallel/rank_generator.py:4-105): world 8 with tp2 dp2 pp2
gives tp ``[[0,1],[2,3],...]``, dp ``[[0,2],[1,3],...]``, pp ``[[0,4],[1,5],...]``.
"""
from __future__ import annotations

import itertools


def prefix_product(values: list[int], init: int = 1) -> list[int]:
    """``[init, init*v0, init*v0*v1, ...]``: the stride table of a mixed-radix rank layout
    (same helper as nano_megatron/parallel/rank_generator.py:4-10)."""
    out = [init]
    for v in values:
        out.append(out[-1] * v)
    return out


def _strides(sizes: list[int]) -> list[int]:
    out, acc = [], 1
    for s in sizes:
        out.append(acc)
        acc *= s
    return out


def generate_masked_orthogonal_rank_groups(world_size: int, parallel_size: list[int], mask: list[bool]) -> list[list[int]]:
    """Groups vary the masked dimensions and hold the unmasked ones fixed.

    Groups are listed in increasing order of their fixed coordinates (first
    unmasked dimension fastest); members in increasing order of their masked
    coordinates (first masked dimension fastest).
    """
    stride = _strides(parallel_size)
    inner = [(s, d) for s, d, m in zip(parallel_size, stride, mask) if m]
    outer = [(s, d) for s, d, m in zip(parallel_size, stride, mask) if not m]

    def offsets(dims: list[tuple[int, int]]) -> list[int]:
        # itertools.product varies the LAST factor fastest; reverse so that the
        # first dimension is the fastest one.
        ranges = [range(size) for size, _ in reversed(dims)]
        res = []
        for combo in itertools.product(*ranges):
            res.append(sum(c * d for c, (_, d) in zip(combo, reversed(dims))))
        return res

    member_offsets = offsets(inner)
    groups = [[base + off for off in member_offsets] for base in offsets(outer)]
    assert sum(len(g) for g in groups) == world_size
    return groups


class RankGenerator:
    def __init__(self, tp: int, dp: int, pp: int, cp: int = 1, order: str = "tp-cp-dp-pp") -> None:
        if min(tp, dp, pp, cp) < 1:
            raise ValueError("all parallel sizes must be >= 1")
        self.tp, self.dp, self.pp, self.cp = tp, dp, pp, cp
        self.world_size = tp * dp * pp * cp
        self.name_to_size = {"tp": tp, "pp": pp, "dp": dp, "cp": cp}
        names = order.lower().split("-")
        for name, size in self.name_to_size.items():
            if name not in names:
                if size != 1:
                    raise RuntimeError(f"size of ({name}) is ({size}), but order ({order.lower()}) omits it")
                names.append(name)
        self.order = "-".join(names)
        self.ordered_names = names
        self.ordered_size = [self.name_to_size[n] for n in names]

    def get_mask(self, token: str) -> list[bool]:
        wanted = set(token.split("-"))
        unknown = wanted - set(self.ordered_names)
        if unknown:
            raise ValueError(f"unknown parallel dimension(s): {sorted(unknown)}")
        return [n in wanted for n in self.ordered_names]

    def get_ranks(self, token: str) -> list[list[int]]:
        return generate_masked_orthogonal_rank_groups(self.world_size, self.ordered_size, self.get_mask(token))

    def decode(self, global_rank: int) -> dict[str, int]:
        if not 0 <= global_rank < self.world_size:
            raise ValueError(f"rank {global_rank} out of range [0, {self.world_size})")
        coords, rest = {}, global_rank
        for name, size in zip(self.ordered_names, self.ordered_size):
            coords[name] = rest % size
            rest //= size
        return coords

    def encode(self, ranks: dict[str, int]) -> int:
        return sum(ranks[n] * d for n, d in zip(self.ordered_names, _strides(self.ordered_size)))
