"""(batch x head) sharding of the SSD across the GPUs of one box.

Every (batch row, head) pair is an independent SSD problem (state [p, r], one decay scalar per head;
B/C shared inside a group), so the path shards with no exchange inside the scan.  The partitioner hands
each rank a contiguous range of flattened (b, h) units, whole batch rows first; heads of one row are
split only when there are more ranks than rows.  The one collective this path can need is the
all-gather of y along the head axis when a row's heads live on several ranks (the gated norm that
follows the SSD in the block reduces over all of d_inner, src/mamba2/mamba2.rs:776).  Ranks that own
whole rows exchange nothing.  Decode steps are never sharded.

A single long sequence can also be cut along time (`ssd2_fwd_sequence_parallel`): the recurrence over a slice is
an affine map of the entering state, h_out = decay * h_in + h_from_zero with decay = exp(A * sum(dt)) per
(row, head), so every rank first runs its slice from a zero state, the ranks all-gather those two small tensors,
each folds the maps of the ranks before it into its true entering state and runs its slice a second time from
that state.  Two passes on every rank but the first (which therefore takes a slice twice as long,
`sequence_cuts`): the exchange is [b, h, p, r] float32 per rank, independent of the sequence length.
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

    def calls(self):
        """[(b_lo, b_hi, h_lo, h_hi)]: the rank's units as the fewest rectangular library calls -- runs of
        whole rows become one call of batch b_hi - b_lo, partial rows one call each."""
        out = []
        for b, h_lo, h_hi in self.slices():
            whole = h_lo == 0 and h_hi == self.nheads
            if whole and out and out[-1][2] == 0 and out[-1][3] == self.nheads and out[-1][1] == b:
                out[-1] = (out[-1][0], b + 1, 0, self.nheads)
            else:
                out.append((b, b + 1, h_lo, h_hi))
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


def partition_heads(batch, nheads, world):
    """Unit ranges that may cut inside a B/C group (every head of a group reads the same B/C, so a rank that
    owns part of a group simply reads that group too).  Used when there are more ranks than
    batch x groups blocks, e.g. one group per row and more GPUs than rows."""
    if batch <= 0 or nheads <= 0 or world <= 0:
        raise ValueError("batch, nheads, world must be positive")
    units = batch * nheads
    cuts = [round(i * units / world) for i in range(world + 1)]
    return [UnitRange(cuts[i], cuts[i + 1], nheads) for i in range(world)]


def row_owners(parts):
    """{row: [(rank, h_lo, h_hi), ...]} for the rows whose heads are spread over more than one rank."""
    owners = {}
    for rank, pr in enumerate(parts):
        for b, h_lo, h_hi in pr.slices():
            owners.setdefault(b, []).append((rank, h_lo, h_hi))
    return {b: v for b, v in owners.items() if len(v) > 1}


def ssd2_fwd_local(fwd, x, dt, a, b, c, d, h0, chunk_len, mine):
    """Runs `fwd` (an ssd2_fwd-compatible callable) on one rank's units: one call per rectangle of
    UnitRange.calls().  Inputs are full tensors or any tensors indexable the same way; B/C are sliced by group.
    Returns [(b_lo, b_hi, h_lo, h_hi, y_part, h_part)]."""
    h = x.shape[2]
    g = b.shape[2]
    hpg = h // g
    parts = []
    for b_lo, b_hi, h_lo, h_hi in mine.calls():
        # a head range that starts or ends inside a B/C group is cut at the group boundaries: every piece then
        # lies inside one group (the call sees that group as its only one) or covers whole groups
        cuts = sorted({h_lo, h_hi, min(h_hi, -(-h_lo // hpg) * hpg), max(h_lo, (h_hi // hpg) * hpg)})
        ys, hs = [], []
        for lo, hi in zip(cuts[:-1], cuts[1:]):
            g_lo, g_hi = lo // hpg, -(-hi // hpg)
            heads = slice(lo, hi)
            y_p, hf_p = fwd(x[b_lo:b_hi, :, heads].contiguous(), dt[b_lo:b_hi, :, heads].contiguous(),
                            a[heads].clone(), b[b_lo:b_hi, :, g_lo:g_hi].contiguous(),
                            c[b_lo:b_hi, :, g_lo:g_hi].contiguous(), None if d is None else d[heads].clone(),
                            None if h0 is None else h0[b_lo:b_hi, heads].contiguous(), chunk_len)
            ys.append(y_p)
            hs.append(hf_p)
        if len(ys) > 1:
            import torch
            ys, hs = [torch.cat(ys, dim=2)], [torch.cat(hs, dim=1)]
        parts.append((b_lo, b_hi, h_lo, h_hi, ys[0], hs[0]))
    return parts


_group_cache = {}


def _subgroup(ranks, world):
    """Process group of `ranks` (every rank of the world must call this with the same sequence of rank sets)."""
    import torch.distributed as dist
    if len(ranks) == world:
        return None
    key = tuple(ranks)
    if key not in _group_cache:
        _group_cache[key] = dist.new_group(list(ranks))
    return _group_cache[key]


def gather_heads(parts, parts_of_all, rank, world, nheads):
    """All-gather along the head axis for the rows whose heads are split: every rank that owns a piece of such
    a row ends up with the row's full y [1, s, H, p] and final state [1, H, p, r].  One all_gather per tensor and
    split row, inside the sub-group of the ranks that share the row; pieces of unequal width are padded to
    the widest.  Rows owned whole by one rank are returned as they are.  -> {row: (y_full, h_full)}."""
    import torch
    import torch.distributed as dist

    split = row_owners(parts_of_all)
    out = {}
    for b_lo, b_hi, h_lo, h_hi, y_p, hf_p in parts:
        if h_lo == 0 and h_hi == nheads:
            for i, row in enumerate(range(b_lo, b_hi)):
                out[row] = (y_p[i:i + 1], hf_p[i:i + 1])
    # every rank walks the split rows in the same order so that group creation and collectives line up
    for row in sorted(split):
        owners = split[row]
        ranks = [r for r, _, _ in owners]
        group = _subgroup(ranks, world) if world > 1 else None
        if rank not in ranks:
            continue
        mine = next(p for p in parts if p[0] == row and not (p[2] == 0 and p[3] == nheads))
        _, _, h_lo, h_hi, y_p, hf_p = mine
        width = max(hi - lo for _, lo, hi in owners)
        pad = lambda t, dim: t if t.shape[dim] == width else torch.cat(
            [t, t.new_zeros(t.shape[:dim] + (width - t.shape[dim],) + t.shape[dim + 1:])], dim=dim)
        ys, hs = pad(y_p, 2).contiguous(), pad(hf_p, 1).contiguous()
        y_all = ys.new_empty((len(ranks),) + tuple(ys.shape))
        h_all = hs.new_empty((len(ranks),) + tuple(hs.shape))
        if world > 1:
            try:
                dist.all_gather_into_tensor(y_all, ys, group=group)
                dist.all_gather_into_tensor(h_all, hs, group=group)
            except (RuntimeError, NotImplementedError):   # back ends without the flat form
                yl, hl = list(y_all.unbind(0)), list(h_all.unbind(0))
                dist.all_gather(yl, ys, group=group)
                dist.all_gather(hl, hs, group=group)
                y_all, h_all = torch.stack(yl), torch.stack(hl)
        else:
            y_all[0], h_all[0] = ys, hs
        y_full = torch.cat([y_all[i][:, :, :hi - lo] for i, (_, lo, hi) in enumerate(owners)], dim=2)
        h_full = torch.cat([h_all[i][:, :hi - lo] for i, (_, lo, hi) in enumerate(owners)], dim=1)
        out[row] = (y_full, h_full)
    return out


def ssd2_fwd_sharded(fwd, x, dt, a, b, c, d, h0, chunk_len, rank, world, gather=True, by_heads=False):
    """This rank's share of one SSD problem: runs `fwd` on the rank's units and, when `gather`, completes the
    rows whose heads are split with an all-gather along heads.  Returns {row: (y [1,s,H,p], h_final [1,H,p,r])}
    for the rows this rank holds in full afterwards (its own whole rows plus the split rows it shares), or the
    raw parts list when not gathering."""
    bsz, _, h, _ = x.shape
    parts_of_all = partition_heads(bsz, h, world) if by_heads else partition_units(bsz, h, b.shape[2], world)
    parts = ssd2_fwd_local(fwd, x, dt, a, b, c, d, h0, chunk_len, parts_of_all[rank])
    if not gather:
        return parts
    return gather_heads(parts, parts_of_all, rank, world, h)


def sequence_cuts(seqlen, world, align):
    """[(start, stop)] of the `world` time slices of one sequence.  Rank 0 runs its slice once, every other rank
    twice, so rank 0 gets two shares and the others one each (all ranks then do 2 / (world + 1) of the sequence's
    work); cut points are multiples of `align` (the chunk length, so that slices start on tile boundaries)."""
    if seqlen <= 0 or world <= 0 or align <= 0:
        raise ValueError("seqlen, world, align must be positive")
    blocks = -(-seqlen // align)
    cuts = [0] + [min(blocks, round((i + 1) * blocks / (world + 1))) for i in range(1, world)] + [blocks]
    for i in range(1, len(cuts)):
        cuts[i] = max(cuts[i], cuts[i - 1])
    return [(min(cuts[i] * align, seqlen), min(cuts[i + 1] * align, seqlen)) for i in range(world)]


def entering_state(h_locs, decays, rank):
    """State entering slice `rank` of a sequence cut along time.  h_locs[k] [b, h, p, r]: the state slice k reaches
    from its own start (slice 0 from the sequence's initial state, the others from zero); decays[k] [b, h]:
    exp(A * sum of dt over slice k).  Folds the affine maps of slices 0 .. rank - 1 in order; for rank 0 returns None
    (the caller's own initial state applies).  rank = len(h_locs) gives the state after the whole sequence."""
    if rank == 0:
        return None
    h = h_locs[0]
    for k in range(1, rank):
        h = h_locs[k] + h * decays[k][:, :, None, None]
    return h


def slice_decay(dt, a):
    """exp(A[h] * sum_t dt[b, t, h]) of one slice, float32 [b, h]; dt must be the step sizes the scan uses (after any
    softplus / clamp)."""
    import torch
    return torch.exp(a.float()[None, :] * dt.float().sum(dim=1))


def ssd2_fwd_sequence_parallel(fwd, x, dt, a, b, c, d, h0, chunk_len, rank, world, group=None):
    """One SSD problem whose sequence is cut into `world` consecutive slices, this rank holding slice `rank`
    (x [b, s_loc, h, p], dt [b, s_loc, h] as used by the scan, B / C [b, s_loc, g, r]).  `fwd` is an
    ssd2_fwd-compatible callable; h0 is the initial state of the whole sequence (read by rank 0 only).
    Returns (y of this slice, final state of the whole sequence).  One all-gather of the slice end states and decays;
    every rank but the first runs its slice twice."""
    import torch
    import torch.distributed as dist

    y, h_loc = fwd(x, dt, a, b, c, d, h0 if rank == 0 else None, chunk_len)
    dec = slice_decay(dt, a)
    if world == 1:
        return y, h_loc
    h_loc = h_loc.float().contiguous()
    h_all = h_loc.new_empty((world,) + tuple(h_loc.shape))
    d_all = dec.new_empty((world,) + tuple(dec.shape))
    try:
        dist.all_gather_into_tensor(h_all, h_loc, group=group)
        dist.all_gather_into_tensor(d_all, dec.contiguous(), group=group)
    except (RuntimeError, NotImplementedError):   # back ends without the flat form
        hl, dl = list(h_all.unbind(0)), list(d_all.unbind(0))
        dist.all_gather(hl, h_loc, group=group)
        dist.all_gather(dl, dec.contiguous(), group=group)
        h_all, d_all = torch.stack(hl), torch.stack(dl)
    # one fold over the ranks gives this rank's entering state (after the maps of the ranks before it; the second pass
    # is launched as soon as it is known) and the state after the whole sequence
    h = h_all[0]
    for k in range(1, world):
        if k == rank:
            y, _ = fwd(x, dt, a, b, c, d, h.contiguous(), chunk_len)
        h = torch.addcmul(h_all[k], h, d_all[k][:, :, None, None])
    return y, h
