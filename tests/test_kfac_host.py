"""Host side of the KFAC step (moving averages, pi-adjusted damping, Cholesky inverses, the
centring and cotangents of the fine-tune loss) against the float64 restatement in oracle/kfac.py
and against dense Kronecker products; a world_size-2 gloo run for the sums that cross ranks."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hamiltonzero_b200 import finetune, kfac
from oracle import kfac as K


def _spd(rng, n, rank=None):
    x = rng.standard_normal((rank or 3 * n, n))
    return x.T @ x / x.shape[0]


def test_moving_average_follows_the_accumulator_rule():
    rng = np.random.default_rng(0)
    avg = kfac.WeightedMovingAverage(torch.zeros(3, 3, dtype=torch.float64))
    v, w = np.zeros((3, 3)), 0.0
    for step in range(5):
        new = _spd(rng, 3)
        avg.update(torch.from_numpy(new), 0.95, 1.0 if step != 2 else -0.5)
        v, w = K.ema_update(v, w, new, 0.95, 1.0 if step != 2 else -0.5)
        np.testing.assert_allclose(avg.value.numpy(), v, rtol=1e-14, atol=1e-15)
        assert abs(avg.weight - w) < 1e-14


def test_pi_adjusted_damping_and_cholesky_inverse_match_the_dense_kronecker_solve():
    rng = np.random.default_rng(1)
    a, g = _spd(rng, 5), 40.0 * _spd(rng, 4)
    block = kfac.DenseBlock(5, 4)
    x = rng.standard_normal((60, 5)); dy = rng.standard_normal((60, 4))
    mask = (rng.random(60) < 0.7)
    s_in, s_out, rep = K.dense_block_statistics(x, dy, mask, logical_batch=12, batch_size=12)
    m = mask[:, None].astype(np.float64)
    block.update(torch.from_numpy((x * m).T @ (x * m)), torch.from_numpy((dy * m).T @ (dy * m)),
                 float(mask.sum()), logical_batch=12, batch_size=12, ema_old=0.95, ema_new=1.0)
    np.testing.assert_allclose(block.a.value.numpy(), s_in, rtol=1e-13)
    np.testing.assert_allclose(block.g.value.numpy(), s_out, rtol=1e-13)
    # repeats starts at one with unit weight (the reference's initial state)
    want_rep, _ = K.ema_update(1.0, 1.0, rep, 0.95, 1.0)
    assert abs(float(block.repeats.value) - want_rep) < 1e-14
    grad = rng.standard_normal((5, 4))
    block.update_inverse(damping=1e-3)
    got = block.precondition(torch.from_numpy(grad)).numpy()
    want = K.dense_block_precondition(s_in, s_out, want_rep, 1e-3, grad)
    np.testing.assert_allclose(got, want, rtol=1e-9, atol=1e-12)
    # the factored damping keeps the product of the average diagonals and adds the damping to it
    fa, fg = kfac.pi_adjusted_kronecker_factors(torch.from_numpy(a), torch.from_numpy(g), damping=0.1)
    na, ng = np.trace(a) / 5, np.trace(g) / 4
    assert abs(np.trace(fa.numpy()) / 5 * np.trace(fg.numpy()) / 4
               - (np.sqrt(na * ng) + np.sqrt(0.1)) ** 2) < 1e-12
    z = kfac.pi_adjusted_kronecker_factors(torch.zeros(3, 3, dtype=torch.float64),
                                           torch.from_numpy(g), damping=0.04)
    np.testing.assert_allclose(z[0].numpy(), 0.2 * np.eye(3)); np.testing.assert_allclose(z[1].numpy(), 0.2 * np.eye(4))


def test_two_kronecker_and_diagonal_blocks():
    rng = np.random.default_rng(2)
    block = kfac.TwoKroneckerBlock(6, 4)
    left, right = _spd(rng, 6), _spd(rng, 4)
    block.update(left, right, 2.5, ema_old=0.0, ema_new=1.0)        # history dropped
    np.testing.assert_allclose(block.left.value.numpy(), left, rtol=1e-14)
    assert abs(float(block.repeats.value) - 2.5) < 1e-14
    block.update_inverse(damping=1e-2)
    grad = rng.standard_normal((2, 3, 2, 2))                        # [G, d_j, d_k, d_l]
    got = block.precondition(torch.from_numpy(grad)).numpy()
    eps = 1e-6
    fl = left + max(eps, eps - np.trace(left) / 6) * np.eye(6)
    fr = right + max(eps, eps - np.trace(right) / 4) * np.eye(4)
    want = K.dense_block_precondition(fl, fr, 2.5, 1e-2, grad.reshape(6, 4)).reshape(grad.shape)
    np.testing.assert_allclose(got, want, rtol=1e-9, atol=1e-12)
    d = kfac.DiagonalBlock((3, 2))
    sq = rng.random((3, 2))
    d.update(torch.from_numpy(sq * 8), batch_size=8, ema_old=0.95, ema_new=1.0)
    g = rng.standard_normal((3, 2))
    np.testing.assert_allclose(d.precondition(torch.from_numpy(g), 0.5).numpy(), g / (sq + 0.5), rtol=1e-13)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _loss_worker(rank, world, port, energy, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lo, hi = (0, 5) if rank == 0 else (5, 8)
        e = torch.from_numpy(energy[:, lo:hi])
        ca, cp, loss = finetune.loss_cotangents(e)
        avg = kfac.WeightedMovingAverage(torch.full((2, 2), float(rank + 1), dtype=torch.float64), 1.0).sync()
        signs = finetune.make_fisher_signs(3, torch.zeros(1, hi - lo, 4, 4))
        out[rank] = (ca.numpy(), cp.numpy(), float(loss), avg.value.numpy(), signs.numpy())
    finally:
        dist.destroy_process_group()


def test_loss_cotangents_centre_over_all_ranks_gloo():
    rng = np.random.default_rng(5)
    energy = (rng.standard_normal((1, 8)) + 1j * rng.standard_normal((1, 8))).astype(np.complex64)
    out = mp.Manager().dict()
    mp.spawn(_loss_worker, args=(2, _free_port(), energy, out), nprocs=2, join=True)
    e = energy.astype(np.complex128)
    delta = e - e.mean(axis=1, keepdims=True)
    n_eff = (np.abs(delta) > 0).sum()
    ca = np.concatenate([out[0][0], out[1][0]], axis=1)
    cp = np.concatenate([out[0][1], out[1][1]], axis=1)
    np.testing.assert_allclose(ca, 2 * delta.real / n_eff, rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(cp, 2 * delta.imag / n_eff, rtol=1e-6, atol=1e-7)
    assert abs(out[0][2] - e.mean().real) < 1e-6 and out[0][2] == out[1][2]
    np.testing.assert_allclose(out[0][3], np.full((2, 2), 1.5))       # pmean of the factor
    for r in (0, 1):
        s = out[r][4]
        assert s.shape == (1, 5 if r == 0 else 3, 3) and set(np.unique(s)) <= {-1.0, 1.0}
    assert not np.array_equal(out[0][4][:, :3], out[1][4])            # shards draw their own signs


def test_single_process_centring_needs_no_group():
    e = torch.tensor([[1 + 1j, 3 - 1j, 2 + 0j]], dtype=torch.complex64)
    delta, mean = finetune.center_preprocessed_energy(e)
    assert complex(mean[0]) == 2 + 0j
    ca, cp, loss = finetune.loss_cotangents(e)
    np.testing.assert_allclose(ca.numpy(), [[-1.0, 1.0, 0.0]])      # 2 * Re dE / n_eff, n_eff = 2
    np.testing.assert_allclose(cp.numpy(), [[1.0, -1.0, 0.0]])
    assert float(loss) == 2.0
