"""Test infrastructure, not product code: float64 numpy restatement of the KFAC host step that
hamiltonzero_b200/kfac.py performs (moving averages, pi-adjusted damping, inverses), written
against dense Kronecker products so that the factored form can be checked against the matrix it
stands for. Follows src/kfac_jax/_src/utils/accumulators.py:66-94,
src/kfac_jax/_src/utils/math.py:631-745 and src/hamiltonzero/optim/blocks.py:1122-1204,318-324.
Parity unpinned: the reference's tests hold no golden vectors for these functions and JAX is not
installed where this was written; the restatement is anchored on the reference's formulas and on
the dense identity ``(kron(A', G'))^-1 vec = A'^-1 X G'^-1``."""
import numpy as np


def ema_update(value, weight, new_value, ema_old, ema_new):
    weight = ema_old * weight + max(ema_new, 0.0)
    eta_old = max(ema_new, 0.0) / weight
    eta_new = abs(ema_new) / weight
    return value * (1.0 - eta_old) + new_value * eta_new, weight


def pi_adjusted(factors, damping):
    k = len(factors)
    norms = np.array([np.trace(f) / f.shape[0] for f in factors])
    if norms.min() <= 0:
        return [damping ** (1.0 / k) * np.eye(f.shape[0]) for f in factors]
    c_k = np.exp(np.mean(np.log(norms)))
    d_hat = damping ** (1.0 / k) / c_k
    return [(f / n + d_hat * np.eye(f.shape[0])) * c_k for f, n in zip(factors, norms)]


def dense_block_precondition(a, g, repeats, damping, grad):
    """``(scale kron(A, G)_pi-damped)^-1 vec(grad)`` through the dense Kronecker matrix
    (row-major vec of ``grad [in, out]`` pairs with ``kron(A, G)``)."""
    scale = 1.0 / (repeats if repeats > 0 else 1.0)
    a_d, g_d = pi_adjusted([a, g], damping / scale)
    dense = scale * np.kron(a_d, g_d)
    return np.linalg.solve(dense, grad.reshape(-1)).reshape(grad.shape)


def dense_block_statistics(x, dy, mask, logical_batch, batch_size):
    """blocks.py:1179-1196 for rows already grouped: ``x [rows, in]``, ``dy [rows, out]``,
    ``mask [rows]``."""
    m = mask.astype(np.float64)[:, None]
    xm, dym = x * m, dy * m
    return xm.T @ xm / logical_batch, dym.T @ dym / batch_size, m.sum() / logical_batch
