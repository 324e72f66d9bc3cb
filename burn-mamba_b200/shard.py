"""(batch x head) sharding of the SSD across the GPUs of one box.

Every (batch row, head) pair is an independent SSD problem (state [p, r], one decay scalar per head;
B/C shared inside a group), so the path shards with no exchange inside the scan.  The partitioner hands
each rank a contiguous range of flattened (b, h) units, whole batch rows first; heads of one row are
split only when there are more ranks than rows.  The one collective this path can need is the
all-gather of y along the head axis when a row's heads live on several ranks (the gated norm that
follows the SSD in the block reduces over all of d_inner, src/mamba2/mamba2.rs:776).  Decode steps are
never sharded.
"""
from dataclasses import dataclass


@dataclass(frozen=True)
class UnitRange:
    """Units [start, stop) of the flattened (batch, head) index u = b * nheads + h owned by one rank."""
    start: int
    stop: int
    nheads: int

    @property
    def count(self):
        return self.stop - self.start

    def slices(self):
        """[(b, h_lo, h_hi)]: per batch row the head interval this rank owns."""
        out = []
        u = self.start
        while u < self.stop:
            b, h = divmod(u, self.nheads)
            h_hi = min(self.nheads, h + (self.stop - u))
            out.append((b, h, h_hi))
            u += h_hi - h
        return out

    @property
    def splits_heads(self):
        return any(h_lo != 0 or h_hi != self.nheads for _, h_lo, h_hi in self.slices())


def partition_units(batch, nheads, ngroups, world):
    """Contiguous, balanced unit ranges for `world` ranks.  Cut points fall on batch-row boundaries when
    world <= batch and divides it, otherwise on group boundaries of the head axis (a rank never owns a
    fraction of a B/C group, so its B/C slice stays a plain slice)."""
    if batch <= 0 or nheads <= 0 or world <= 0 or ngroups <= 0 or nheads % ngroups:
        raise ValueError("batch, nheads, world must be positive and nheads divisible by ngroups")
    hpg = nheads // ngroups
    blocks = batch * ngroups           # indivisible blocks of hpg heads
    cuts = [round(i * blocks / world) for i in range(world + 1)]
    return [UnitRange(cuts[i] * hpg, cuts[i + 1] * hpg, nheads) for i in range(world)]


def ssd2_fwd_sharded(fwd, x, dt, a, b, c, d, h0, chunk_len, rank, world, group=None, gather=True):
    """Runs `fwd` (an ssd2_fwd-compatible callable) on this rank's units and, when `gather`, all-gathers
    y and the final state so that every rank holds the full result (what the block's gated norm needs).
    Inputs are the full tensors (each rank slices its own part; B/C are sliced by group).
    Returns (y, h_final) full-size, or this rank's [(b, h_lo, h_hi, y_part, h_part)] list when not gathering."""
    import torch
    import torch.distributed as dist

    bsz, s, h, p = x.shape
    g = b.shape[2]
    hpg = h // g
    mine = partition_units(bsz, h, g, world)[rank]
    parts = []
    for bi, h_lo, h_hi in mine.slices():
        g_lo, g_hi = h_lo // hpg, -(-h_hi // hpg)
        y_p, hf_p = fwd(x[bi:bi + 1, :, h_lo:h_hi].contiguous(), dt[bi:bi + 1, :, h_lo:h_hi].contiguous(),
                        a[h_lo:h_hi].contiguous(), b[bi:bi + 1, :, g_lo:g_hi].contiguous(),
                        c[bi:bi + 1, :, g_lo:g_hi].contiguous(), None if d is None else d[h_lo:h_hi].contiguous(),
                        None if h0 is None else h0[bi:bi + 1, h_lo:h_hi].contiguous(), chunk_len)
        parts.append((bi, h_lo, h_hi, y_p, hf_p))
    if not gather:
        return parts
    r = b.shape[3]
    y = torch.zeros_like(x)
    hf = torch.zeros((bsz, h, p, r), dtype=torch.float32, device=x.device)
    for bi, h_lo, h_hi, y_p, hf_p in parts:
        y[bi:bi + 1, :, h_lo:h_hi] = y_p
        hf[bi:bi + 1, h_lo:h_hi] = hf_p
    if world > 1:
        # units are disjoint across ranks, so a sum over ranks is the gather (one collective per tensor)
        dist.all_reduce(y, group=group)
        dist.all_reduce(hf, group=group)
    return y, hf
