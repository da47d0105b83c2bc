"""Partitioning of the path's independent units across GPUs (one process per GPU).

Every operation of this library works on independent units -- (image, group) slabs for
GroupNorm, rows for LayerNorm and GEGLU, tokens for the embedding, elements for the
activations -- so N GPUs need no exchange step: each rank takes a contiguous range of units
and never talks to its peers on the data path.  The reference is single-device
(native-lib.cpp:41-50: one cl_device_id, one queue); this module is the added multi-GPU layer.
"""
from __future__ import annotations

from dataclasses import dataclass


def partition(units: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced range [lo, hi) of `units` for `rank` of `world`."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if units < 0:
        raise ValueError("units must be >= 0")
    base, rem = divmod(units, world)
    lo = rank * base + min(rank, rem)
    hi = lo + base + (1 if rank < rem else 0)
    return lo, hi


def partition_alive(units: int, alive: list[int], rank: int) -> tuple[int, int]:
    """Same, over the ranks still taking work.  A rank not in `alive` gets an empty range; the
    others split everything, so a device marked unavailable by the host costs no units."""
    ranks = sorted(set(alive))
    if not ranks:
        raise ValueError("no rank alive")
    if rank not in ranks:
        return 0, 0
    return partition(units, len(ranks), ranks.index(rank))


@dataclass(frozen=True)
class GroupNormPiece:
    """A run of whole groups of one image: groups [g0, g0 + ng) of image `image`."""
    image: int
    g0: int
    ng: int


def groupnorm_pieces(batch: int, num_groups: int, world: int, rank: int) -> list[GroupNormPiece]:
    """This rank's share of a [batch, C, H, W] GroupNorm, as runs of groups within images.

    Whole images when batch >= world divides evenly; otherwise the batch * num_groups slabs are
    split, and a rank's range may start and end inside an image.  Each piece is one kernel
    call on a sub-tensor (channels [g0*cpg, (g0+ng)*cpg) of one image, or several whole images
    merged by `merge_whole_images`)."""
    lo, hi = partition(batch * num_groups, world, rank)
    pieces: list[GroupNormPiece] = []
    s = lo
    while s < hi:
        image, g0 = divmod(s, num_groups)
        ng = min(num_groups - g0, hi - s)
        pieces.append(GroupNormPiece(image, g0, ng))
        s += ng
    return pieces


def merge_whole_images(pieces: list[GroupNormPiece], num_groups: int) -> list[tuple[int, int, int, int]]:
    """Fuse consecutive whole-image pieces into (first_image, n_images, g0, ng) calls."""
    calls: list[tuple[int, int, int, int]] = []
    for p in pieces:
        whole = p.g0 == 0 and p.ng == num_groups
        if whole and calls and calls[-1][2] == 0 and calls[-1][3] == num_groups \
                and calls[-1][0] + calls[-1][1] == p.image:
            first, n, g0, ng = calls[-1]
            calls[-1] = (first, n + 1, g0, ng)
        else:
            calls.append((p.image, 1, p.g0, p.ng))
    return calls
