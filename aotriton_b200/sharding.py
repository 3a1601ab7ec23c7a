"""Batch x head partitioning of one attention problem over the GPUs of a node.

Every (batch element, kv head) pair -- with the group of q heads that shares the kv head -- is an
independent unit in forward and backward: dK/dV reduce only over the q heads of their own kv head
(ROCm/aotriton modules/flash/kernel/bwd_kernel_dk_dv.py:285).  The units are flattened, dealt out
in contiguous ranges, and each rank runs the ordinary operator on views of its range.  No
collective is needed on the data path; gathers are for verification only.

Dropout stays bit-identical to the unsharded run: the Philox counter of element (z, h, m, n) is
  base + ((z * Hq_total + h) * Max_seqlen_q + m) * stride + n // 4
so a shard that starts at batch b0 adds b0 * Hq_total * Max_seqlen_q * stride to the host-side
offset, and passes its first q head and Hq_total to the kernels (philox_head_offset /
philox_num_head_q of the C-ABI).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Segment:
    """Units [hk_lo, hk_hi) of batch element b (dense) -- or of all sequences (varlen, b = None)."""
    b: int | None
    hk_lo: int
    hk_hi: int


def unit_range(num_units: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced: the first (num_units % world) ranks get one extra unit."""
    base, extra = divmod(num_units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def partition_dense(batch: int, num_head_k: int, world: int, rank: int) -> list[Segment]:
    """Segments (one per touched batch element) covering this rank's units of a dense problem."""
    lo, hi = unit_range(batch * num_head_k, world, rank)
    segs = []
    u = lo
    while u < hi:
        b, h = divmod(u, num_head_k)
        h_end = min(num_head_k, h + (hi - u))
        segs.append(Segment(b, h, h_end))
        u += h_end - h
    return segs


def partition_varlen(num_head_k: int, world: int, rank: int) -> list[Segment]:
    """Varlen problems are split over kv heads only, so that every rank sees every sequence."""
    lo, hi = unit_range(num_head_k, world, rank)
    return [Segment(None, lo, hi)] if hi > lo else []


def philox_adjustment(seg: Segment, group: int, num_head_q: int, max_seqlen_q: int, max_seqlen_k: int) -> dict:
    """Extra C-ABI problem fields that keep a segment's dropout mask equal to the unsharded one."""
    stride = (max_seqlen_k + 3) // 4
    b0 = seg.b or 0
    return dict(philox_offset2_add=b0 * num_head_q * max_seqlen_q * stride,
                philox_head_offset=seg.hk_lo * group, philox_num_head_q=num_head_q)


def slice_dense(seg: Segment, group: int, q_like, kv_like=None):
    """Views of (B, H, S, D) tensors for a segment: q-like tensors take heads [hk_lo*G, hk_hi*G)."""
    b = seg.b
    out = q_like[b:b + 1, seg.hk_lo * group:seg.hk_hi * group]
    if kv_like is None:
        return out
    return out, kv_like[b:b + 1, seg.hk_lo:seg.hk_hi]


def slice_lse_dense(seg: Segment, group: int, lse, num_head_q: int):
    """Rows of the (B*Hq, Sq) logsumexp / delta matrix that belong to a segment."""
    r0 = seg.b * num_head_q + seg.hk_lo * group
    return lse[r0:r0 + (seg.hk_hi - seg.hk_lo) * group]
