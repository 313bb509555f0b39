"""Moving averages, damping and inverses of the curvature blocks that the reverse pass feeds
(the host side of the KFAC step; the second-moment sums come from ``hz_logpsi_vjp``).

Restated from the reference's blocks and the kfac_jax copy it vendors:
  * weighted moving average of a factor - src/kfac_jax/_src/utils/accumulators.py:66-94;
  * structural dense block: ``A = X^T X / logical_batch``, ``G = dY^T dY / batch_size``, the
    average repeat count and ``state_dependent_scale = 1 / repeats`` -
    src/hamiltonzero/optim/blocks.py:1122-1204;
  * diagonal block of a scale tag - blocks.py:1016-1110,1207-1286;
  * two-Kronecker block of the quadrilinear tag (left/right marginals with the repeat scale) -
    src/hamiltonzero/optim/spin_blocks.py:443-556;
  * pi-adjusted factored damping and Cholesky inverses -
    src/kfac_jax/_src/utils/math.py:631-745 (``set_use_cholesky_inversion(True)``,
    src/hamiltonzero/optim/production.py:231-232).
Everything is torch on whichever device holds the sums; the matrices are at most 1536 x 1536,
once per ``inverse_update_period`` steps, so this is library linear algebra, not a kernel."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class WeightedMovingAverage:
    value: torch.Tensor
    weight: float = 0.0

    def update(self, value: torch.Tensor, old_weight_multiplier: float, new_weight: float):
        """accumulators.py:66-88 (a negative ``new_weight`` adds without raising the weight)."""
        self.weight = old_weight_multiplier * self.weight + max(new_weight, 0.0)
        eta_old = max(new_weight, 0.0) / self.weight
        eta_new = abs(new_weight) / self.weight
        self.value = self.value * (1.0 - eta_old) + value.to(self.value.dtype) * eta_new
        return self

    def sync(self, group=None):
        """Mean over the ranks (``pmean``)."""
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            dist.all_reduce(self.value, op=dist.ReduceOp.SUM, group=group)
            self.value = self.value / dist.get_world_size(group)
        return self


def _avg_diag(f: torch.Tensor) -> torch.Tensor:
    return (torch.diagonal(f).sum() / f.shape[0]) if f.ndim == 2 else f.mean()


def pi_adjusted_kronecker_factors(*factors: torch.Tensor, damping: float):
    """Factors ``F_i'`` whose Kronecker product approximates ``kron(F_i) + damping I``
    (math.py:631-745): each factor is written ``n_i U_i`` with ``avg diag(U_i) = 1``; the
    geometric mean ``c`` of the ``n_i`` goes back into every factor and the damping is split
    evenly, ``F_i' = c (U_i + damping^(1/k) / c I)``. A vanishing factor gives
    ``damping^(1/k) I`` for all."""
    k = len(factors)
    norms = torch.stack([_avg_diag(f) for f in factors])
    if float(norms.min()) <= 0.0:
        c = float(damping) ** (1.0 / k)
        return tuple(c * (torch.eye(f.shape[0], dtype=f.dtype, device=f.device) if f.ndim == 2
                          else torch.ones_like(f)) for f in factors)
    c_k = torch.exp(torch.log(norms).mean())
    d_hat = float(damping) ** (1.0 / k) / c_k
    out = []
    for f, n in zip(factors, norms):
        u = f / n
        u = u + d_hat * torch.eye(f.shape[0], dtype=f.dtype, device=f.device) if f.ndim == 2 else u + d_hat
        out.append(u * c_k)
    return tuple(out)


def floor_matrix_avg_diag(m: torch.Tensor, eps: float) -> torch.Tensor:
    """Shift the diagonal so that its average is at least ``eps`` (blocks.py:318-324)."""
    shift = max(eps, eps - float(_avg_diag(m)))
    return m + shift * torch.eye(m.shape[-1], dtype=m.dtype, device=m.device)


def psd_inv_cholesky(m: torch.Tensor) -> torch.Tensor:
    """Inverse of a positive-definite matrix through its Cholesky factor, symmetrised."""
    chol = torch.linalg.cholesky(0.5 * (m + m.T))
    inv = torch.cholesky_inverse(chol)
    return 0.5 * (inv + inv.T)


@dataclass
class DenseBlock:
    """Kronecker-factored block of one dense tag, parameter ``W [in, out]``."""
    in_dim: int
    out_dim: int
    device: torch.device | str = "cpu"
    dtype: torch.dtype = torch.float64
    a: WeightedMovingAverage = field(init=False)
    g: WeightedMovingAverage = field(init=False)
    repeats: WeightedMovingAverage = field(init=False)
    a_inv: torch.Tensor | None = None
    g_inv: torch.Tensor | None = None

    def __post_init__(self):
        z = lambda *s: torch.zeros(*s, dtype=self.dtype, device=self.device)
        self.a = WeightedMovingAverage(z(self.in_dim, self.in_dim))
        self.g = WeightedMovingAverage(z(self.out_dim, self.out_dim))
        self.repeats = WeightedMovingAverage(torch.ones((), dtype=self.dtype, device=self.device), 1.0)

    def update(self, sum_in, sum_out, mask_rows: float, *, logical_batch: int, batch_size: int,
               ema_old: float, ema_new: float):
        """``sum_in = X^T X`` and ``sum_out = dY^T dY`` over the masked rows of all walkers,
        ``mask_rows`` the number of such rows (blocks.py:1186-1203)."""
        self.a.update(torch.as_tensor(sum_in, device=self.device) / float(logical_batch), ema_old, ema_new)
        self.g.update(torch.as_tensor(sum_out, device=self.device) / float(batch_size), ema_old, ema_new)
        self.repeats.update(torch.as_tensor(mask_rows / float(logical_batch), dtype=self.dtype,
                                            device=self.device), ema_old, ema_new)
        return self

    def sync(self, group=None):
        self.a.sync(group); self.g.sync(group); self.repeats.sync(group)
        return self

    def scale(self) -> float:
        r = float(self.repeats.value)
        return 1.0 / (r if r > 0 else 1.0)

    def update_inverse(self, damping: float):
        """Cache ``A'^-1, G'^-1`` of ``scale kron(A, G) + damping I = scale (kron(A, G) +
        damping / scale I)``."""
        a, g = pi_adjusted_kronecker_factors(self.a.value, self.g.value, damping=damping / self.scale())
        self.a_inv, self.g_inv = psd_inv_cholesky(a), psd_inv_cholesky(g)
        return self

    def precondition(self, grad: torch.Tensor) -> torch.Tensor:
        """``(scale kron(A, G) + damping I)^-1 vec(grad)`` as ``A'^-1 grad G'^-1 / scale``."""
        gr = torch.as_tensor(grad, device=self.device).to(self.dtype)
        return (self.a_inv @ gr @ self.g_inv) / self.scale()


@dataclass
class DiagonalBlock:
    """Diagonal block of a scale tag: the moving average of the squared per-sample gradients."""
    shape: tuple
    device: torch.device | str = "cpu"
    dtype: torch.dtype = torch.float64
    diag: WeightedMovingAverage = field(init=False)

    def __post_init__(self):
        self.diag = WeightedMovingAverage(torch.zeros(self.shape, dtype=self.dtype, device=self.device))

    def update(self, sum_sq, *, batch_size: int, ema_old: float, ema_new: float):
        self.diag.update(torch.as_tensor(sum_sq, device=self.device) / float(batch_size), ema_old, ema_new)
        return self

    def sync(self, group=None):
        self.diag.sync(group)
        return self

    def precondition(self, grad, damping: float):
        return torch.as_tensor(grad, device=self.device).to(self.dtype) / (self.diag.value + damping)


@dataclass
class TwoKroneckerBlock:
    """Block of the quadrilinear tag ``T [G, d, d, d]`` viewed as a ``[left, right]`` matrix with
    the balanced axis partition (left ``G d``, right ``d d``): moving averages of the normalised
    marginals from ``two_kron_marginals`` and the repeat count."""
    left_dim: int
    right_dim: int
    device: torch.device | str = "cpu"
    dtype: torch.dtype = torch.float64
    left: WeightedMovingAverage = field(init=False)
    right: WeightedMovingAverage = field(init=False)
    repeats: WeightedMovingAverage = field(init=False)
    left_inv: torch.Tensor | None = None
    right_inv: torch.Tensor | None = None

    EPSILON_FLOOR = 1e-6                   # spin_blocks.py:370 (_MATPOWER_EPSILON_FLOOR)

    def __post_init__(self):
        # identity with unit weight, as the reference initialises both marginals (:282-303)
        eye = lambda n: torch.eye(n, dtype=self.dtype, device=self.device)
        self.left = WeightedMovingAverage(eye(self.left_dim), 1.0)
        self.right = WeightedMovingAverage(eye(self.right_dim), 1.0)
        self.repeats = WeightedMovingAverage(torch.ones((), dtype=self.dtype, device=self.device), 1.0)

    def update(self, sigma_left, sigma_right, repeats: float, *, ema_old: float, ema_new: float):
        self.left.update(torch.as_tensor(sigma_left, device=self.device), ema_old, ema_new)
        self.right.update(torch.as_tensor(sigma_right, device=self.device), ema_old, ema_new)
        self.repeats.update(torch.as_tensor(repeats, dtype=self.dtype, device=self.device), ema_old, ema_new)
        return self

    def sync(self, group=None):
        self.left.sync(group); self.right.sync(group); self.repeats.sync(group)
        return self

    def scale(self) -> float:
        r = float(self.repeats.value)
        return 1.0 / (r if r > 0 else 1.0)

    def update_inverse(self, damping: float):
        l, r = pi_adjusted_kronecker_factors(floor_matrix_avg_diag(self.left.value, self.EPSILON_FLOOR),
                                             floor_matrix_avg_diag(self.right.value, self.EPSILON_FLOOR),
                                             damping=damping / self.scale())
        self.left_inv, self.right_inv = psd_inv_cholesky(l), psd_inv_cholesky(r)
        return self

    def precondition(self, grad_T: torch.Tensor) -> torch.Tensor:
        g = torch.as_tensor(grad_T, device=self.device).to(self.dtype)
        m = g.reshape(self.left_dim, self.right_dim)
        return ((self.left_inv @ m @ self.right_inv) / self.scale()).reshape(g.shape)


__all__ = ["DenseBlock", "DiagonalBlock", "TwoKroneckerBlock", "WeightedMovingAverage",
           "floor_matrix_avg_diag", "pi_adjusted_kronecker_factors", "psd_inv_cholesky"]
