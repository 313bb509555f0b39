"""Host-side multi-rank logic on CPU: contiguous walker shards and the energy-moment
all-reduce, with a world_size-2 gloo group."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hamiltonzero_b200 import sharding


def test_shard_bounds_cover_the_batch_without_overlap():
    for n in (0, 1, 7, 16, 16384, 16385):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_bounds(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and a <= b and c <= d
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_bounds(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, energies, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = sharding.shard(torch.from_numpy(energies), rank, world)
        stats = sharding.reduce_moments(sharding.local_moments(mine))
        c = sharding.centred(mine, stats)
        out[rank] = (stats["mean"], stats["variance"], stats["count"], complex(c.sum()))
    finally:
        dist.destroy_process_group()


def test_moment_allreduce_world_size_2_gloo():
    rng = np.random.default_rng(0)
    e = (rng.standard_normal(101) + 1j * rng.standard_normal(101)).astype(np.complex64)
    e[17] = np.nan            # a failed sample is skipped on whichever rank holds it
    manager = mp.Manager()
    out = manager.dict()
    port = _free_port()
    mp.spawn(_worker, args=(2, port, e, out), nprocs=2, join=True)
    good = e[np.isfinite(e.real)].astype(np.complex128)
    for rank in (0, 1):
        mean, var, count, _ = out[rank]
        assert count == 100
        assert abs(mean - good.mean()) < 1e-6
        assert abs(var - (np.abs(good) ** 2).mean() + abs(good.mean()) ** 2) < 1e-5
    assert out[0][0] == out[1][0]           # every rank holds the same global mean


def test_single_process_moments_need_no_group():
    e = torch.tensor([1 + 1j, 3 - 1j], dtype=torch.complex64)
    stats = sharding.reduce_moments(sharding.local_moments(e))
    assert stats["mean"] == 2 + 0j and stats["count"] == 2 and abs(stats["variance"] - 2.0) < 1e-12


def _grad_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = {"merge_V": torch.full((3, 2), float(rank + 1)),
             "merge_h": [torch.full((2,), 10.0 * (rank + 1)), torch.full((1,), 100.0 * (rank + 1))]}
        f = {"merge_V_in": torch.eye(2) * (rank + 1)}
        n = sharding.reduce_gradients(g, f, None)
        out[rank] = (n, g["merge_V"].tolist(), [h.tolist() for h in g["merge_h"]],
                     f["merge_V_in"].tolist())
    finally:
        dist.destroy_process_group()


def test_gradient_and_factor_allreduce_world_size_2_gloo():
    manager = mp.Manager()
    out = manager.dict()
    mp.spawn(_grad_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    for rank in (0, 1):
        n, mv, mh, fin = out[rank]
        assert n == 6 + 3 + 4
        assert mv == [[3.0, 3.0]] * 3
        assert mh == [[30.0, 30.0], [300.0]]
        assert fin == [[3.0, 0.0], [0.0, 3.0]]


def _fake_counters(state, seed):
    """Counters as a sampler call would leave them (no GPU needed for the adaptation itself)."""
    g = torch.Generator().manual_seed(seed)
    B, R = state.q.shape[:2]
    state.n_local, state.n_haar = 40, 10
    state.n_local_accept = torch.randint(0, 41, (B, R), generator=g).float()
    state.n_haar_accept = torch.randint(0, 11, (B, R), generator=g).float()
    state.n_swap = torch.full((B, R - 1), 20, dtype=torch.int32)
    state.n_swap_accept = torch.randint(0, 21, (B, R - 1), generator=g).float()
    return state


def _adapt_worker(rank, world, port, out):
    from hamiltonzero_b200 import mcmc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sizes = (5, 3)                       # ragged shards
        st = _fake_counters(mcmc.init_batched_state(1, np.ones(6), sizes[rank], 6, device="cpu"),
                            100 + rank)
        pooled = mcmc.all_reduce_counters(st)
        new = mcmc.adapt_batched(st)
        out[rank] = (pooled.tolist(), new.sigma.tolist(), new.m.tolist(), new.beta.tolist(),
                     float(new.n_local_accept.abs().sum()), int(new.n_swap.sum()))
    finally:
        dist.destroy_process_group()


def test_sharded_adaptation_pools_counters_over_ranks_gloo():
    """Two ranks with ragged walker shards adapt to the same widths, Haar counts and ladder, and
    these equal what one process holding all eight walkers computes."""
    from dataclasses import replace
    from hamiltonzero_b200 import mcmc
    manager = mp.Manager()
    out = manager.dict()
    mp.spawn(_adapt_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    parts = [_fake_counters(mcmc.init_batched_state(1, np.ones(6), b, 6, device="cpu"), 100 + r)
             for r, b in enumerate((5, 3))]
    whole = replace(parts[0], q=torch.cat([p.q for p in parts]),
                    n_local_accept=torch.cat([p.n_local_accept for p in parts]),
                    n_haar_accept=torch.cat([p.n_haar_accept for p in parts]),
                    n_swap=torch.cat([p.n_swap for p in parts]),
                    n_swap_accept=torch.cat([p.n_swap_accept for p in parts]))
    ref = mcmc.adapt_batched(whole)
    assert out[0][:4] == out[1][:4]
    pooled = np.asarray(out[0][0])
    assert pooled[4, 0] == 8 and pooled[3, 0] == 160
    np.testing.assert_array_equal(pooled, mcmc.pooled_counters(whole).numpy())
    assert out[0][1] == ref.sigma.tolist() and out[0][2] == ref.m.tolist()
    np.testing.assert_allclose(out[0][3], ref.beta.tolist(), rtol=0, atol=0)
    assert out[0][4] == 0.0 and out[0][5] == 0
