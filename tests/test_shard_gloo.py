"""CPU tests of the multi-GPU host logic: the (batch x head) partitioner and the world_size-2 gather,
run as two gloo ranks.  The per-rank compute is injected (the numpy oracle stands in for the CUDA call,
which needs a GPU), so only the sharding, slicing and collective plumbing are under test here."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _shard():
    import __graft_entry__ as ge
    ge.load_package()
    import importlib
    return importlib.import_module("burn_mamba_b200.shard")


@pytest.mark.parametrize("batch,nheads,ngroups,world", [(8, 80, 1, 1), (8, 80, 1, 2), (8, 80, 1, 4), (8, 80, 1, 8),
                                                        (1, 80, 1, 8), (2, 8, 2, 8), (3, 6, 3, 4), (2, 4, 4, 3)])
def test_partition_covers_every_unit_once_and_is_balanced(batch, nheads, ngroups, world):
    shard = _shard()
    parts = shard.partition_units(batch, nheads, ngroups, world)
    seen = np.zeros(batch * nheads, int)
    for pr in parts:
        seen[pr.start:pr.stop] += 1
        for b, h_lo, h_hi in pr.slices():
            assert 0 <= h_lo < h_hi <= nheads and h_lo % (nheads // ngroups) == 0 and h_hi % (nheads // ngroups) == 0
    assert np.all(seen == 1)
    counts = [pr.count for pr in parts]
    assert max(counts) - min(counts) <= nheads // ngroups
    if world <= batch and batch % world == 0:
        assert not any(pr.splits_heads for pr in parts)   # whole batch rows: no collective needed


def _oracle_fwd(x, dt, a, b, c, d, h0, chunk_len):
    from oracle import mamba2
    n = lambda t: None if t is None else t.numpy()
    h0n = np.zeros((x.shape[0], x.shape[2], x.shape[3], b.shape[3]), np.float32) if h0 is None else h0.numpy()
    y, hf = mamba2.ssd_serial(n(x), n(dt), n(a), n(b), n(c), n(d), h0n, chunk_len)
    return torch.from_numpy(y), torch.from_numpy(hf)


def _worker(rank, world, port, cfg, by_heads, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shard = _shard()
        t = {k: torch.from_numpy(v) for k, v in cfg.items()}
        rows = shard.ssd2_fwd_sharded(_oracle_fwd, t["x"], t["dt"], t["a"], t["b"], t["c"], t["d"], t["h0"], 16,
                                      rank, world, by_heads=by_heads)
        q.put((rank, {r: (y.numpy(), hf.numpy()) for r, (y, hf) in rows.items()}))
    finally:
        dist.destroy_process_group()


# whole rows per rank (no collective) / heads split at a group boundary / heads split inside the only group
@pytest.mark.parametrize("batch,nheads,ngroups,by_heads", [(2, 4, 1, False), (1, 4, 2, False), (1, 4, 1, True),
                                                           (3, 4, 2, True)])
def test_two_rank_shards_equal_the_single_rank_result(batch, nheads, ngroups, by_heads):
    from oracle import inputs, mamba2
    shard = _shard()
    cfg = inputs.ssd2_prefill(seed=21, batch=batch, seqlen=40, nheads=nheads, headdim=8, state_rank=8, ngroups=ngroups,
                              h0_std=0.1)
    cfg = {k: cfg[k] for k in ("x", "dt", "a", "b", "c", "d", "h0")}
    want_y, want_h = mamba2.ssd_serial(cfg["x"], cfg["dt"], cfg["a"], cfg["b"], cfg["c"], cfg["d"], cfg["h0"], 16)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, cfg, by_heads, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    parts = shard.partition_heads(batch, nheads, 2) if by_heads else shard.partition_units(batch, nheads, ngroups, 2)
    split = shard.row_owners(parts)
    held = {}
    for rank, rows in results.items():
        for row, (y, hf) in rows.items():   # whatever a rank holds is a full, correct row
            assert y.shape[2] == nheads
            assert np.max(np.abs(y[0] - want_y[row])) < 1e-5 and np.max(np.abs(hf[0] - want_h[row])) < 1e-5
            held.setdefault(row, set()).add(rank)
    assert set(held) == set(range(batch))          # every row is held by someone
    for row, owners in split.items():              # split rows end up on every rank that owns a piece
        assert held[row] == {r for r, _, _ in owners}
    for row in set(range(batch)) - set(split):     # whole rows stay where they were computed: no exchange
        assert len(held[row]) == 1


def test_calls_merge_whole_rows_into_one_library_call():
    shard = _shard()
    parts = shard.partition_units(8, 80, 1, 2)
    assert parts[0].calls() == [(0, 4, 0, 80)] and parts[1].calls() == [(4, 8, 0, 80)]
    parts = shard.partition_heads(4, 80, 8)
    assert parts[0].calls() == [(0, 1, 0, 40)] and parts[1].calls() == [(0, 1, 40, 80)]
    ur = shard.UnitRange(40, 280, 80)   # half a row, two whole rows, half a row
    assert ur.calls() == [(0, 1, 40, 80), (1, 3, 0, 80), (3, 4, 0, 40)]


def _seq_worker(rank, world, port, cfg, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shard = _shard()
        t = {k: torch.from_numpy(v) for k, v in cfg.items()}
        cut = slice(*shard.sequence_cuts(t["x"].shape[1], world, 16)[rank])
        y, hf = shard.ssd2_fwd_sequence_parallel(_oracle_fwd, t["x"][:, cut].contiguous(), t["dt"][:, cut].contiguous(),
                                                 t["a"], t["b"][:, cut].contiguous(), t["c"][:, cut].contiguous(),
                                                 t["d"], t["h0"], 16, rank, world)
        q.put((rank, y.numpy(), hf.numpy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_cut_along_time_equals_the_whole_sequence(world):
    """Slices of one sequence on `world` gloo ranks: zero-state pass, all-gather of the slice maps, fold, second
    pass from the true entering state; y of every slice and the final state equal the single call."""
    from oracle import inputs, mamba2
    cfg = inputs.ssd2_prefill(seed=33, batch=2, seqlen=32 * world, nheads=4, headdim=8, state_rank=8, ngroups=2, h0_std=0.2)
    cfg = {k: cfg[k] for k in ("x", "dt", "a", "b", "c", "d", "h0")}
    want_y, want_h = mamba2.ssd_serial(cfg["x"], cfg["dt"], cfg["a"], cfg["b"], cfg["c"], cfg["d"], cfg["h0"], 16)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() % 2000) + world
    procs = [ctx.Process(target=_seq_worker, args=(r, world, port, cfg, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted((q.get(timeout=120) for _ in range(world)), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    y = np.concatenate([g[1] for g in got], axis=1)
    assert np.max(np.abs(y - want_y)) < 1e-5
    for _, _, hf in got:                      # every rank ends with the state after the whole sequence
        assert np.max(np.abs(hf - want_h)) < 1e-5


def test_entering_state_folds_the_slice_maps_in_order():
    shard = _shard()
    rng = np.random.default_rng(0)
    h = [torch.from_numpy(rng.standard_normal((2, 3, 4, 5)).astype(np.float32)) for _ in range(3)]
    dcy = [torch.from_numpy(rng.uniform(0.1, 1.0, (2, 3)).astype(np.float32)) for _ in range(3)]
    assert shard.entering_state(h, dcy, 0) is None
    assert torch.equal(shard.entering_state(h, dcy, 1), h[0])
    want = (h[0] * dcy[1][:, :, None, None] + h[1]) * dcy[2][:, :, None, None] + h[2]
    assert torch.allclose(shard.entering_state(h, dcy, 3), want)


@pytest.mark.parametrize("seqlen,world,align", [(4096, 2, 256), (131072, 8, 256), (1000, 3, 128), (256, 4, 256), (96, 3, 16)])
def test_sequence_cuts_cover_the_sequence_on_aligned_points_with_a_double_first_slice(seqlen, world, align):
    shard = _shard()
    cuts = shard.sequence_cuts(seqlen, world, align)
    assert len(cuts) == world and cuts[0][0] == 0 and cuts[-1][1] == seqlen
    for (a0, a1), (b0, b1) in zip(cuts[:-1], cuts[1:]):
        assert a1 == b0 and a0 <= a1 and a1 % align == 0
    if seqlen >= 4 * world * align:
        lens = [b - a for a, b in cuts]
        assert abs(lens[0] - 2 * lens[1]) <= 2 * align and max(lens[1:]) - min(lens[1:]) <= align
