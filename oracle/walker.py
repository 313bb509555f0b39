"""CPU restatement of the walker-batch operators: the compiled binary-merge-tree
executor (log-psi), the forward-Laplacian local energy and the spin estimator.

TEST INFRASTRUCTURE: checker for the CUDA kernels; never imported by the package.
Parity unpinned: the reference ships no golden vectors for these operators and
cannot be run where this was written. The forward-Laplacian recurrences below are
pinned against a dense fp64 autodiff Hessian of the executor (``energy_dense_autodiff``).

Follows:
  * executor       src/hamiltonzero/compiled/execute.py:24-118,
                   src/hamiltonzero/model/model.py:31-37 (leaf RMS, eps 1e-30),
                   opcodes src/hamiltonzero/compiled/types.py:15-19
  * SU(2) chart    src/hamiltonzero/energy/kernel.py:20-37
  * Laplacian      the calculus of src/hamiltonzero/energy/custom_lap.py: value, Jacobian
                   w.r.t. the 3N chart coordinates and W-weighted Laplacian are pushed
                   through linear maps (:630-725), products (:408-483), sqrt/log/div
                   (:136-181) and the quadrilinear merge (:1318-1389), a node at block
                   size k keeping the Jacobian of its own 3k coordinates only
  * energy         src/hamiltonzero/energy/kernel.py:80-119
  * spin           src/hamiltonzero/observables.py:15-59
"""
from __future__ import annotations

import numpy as np

MERGE, CARRY_LEFT, CARRY_RIGHT, EMPTY = 0, 1, 2, 3
LEAF_EPS = 1e-30


def _cast(wf, dtype):
    g = lambda a: np.asarray(a, dtype=dtype)
    return dict(Wq=g(wf.q_weight), lV=g(wf.leaf_V), lU=g(wf.leaf_U), lh=g(wf.leaf_h),
                T=g(wf.merge_T), mV=g(wf.merge_V), mU=g(wf.merge_U),
                mh=[g(h) for h in wf.merge_h], op=[np.asarray(o) for o in wf.opcodes],
                rV=g(wf.readout_V), rU=g(wf.readout_U), rh=g(wf.readout_h),
                eps=dtype(wf.merge_eps))


def quadrilinear(T, ua, ub):
    """einsum('ijkl,Bik,Bil->Bij') on [..., G*d_r] vectors (execute.py:34-52)."""
    G, d = T.shape[0], T.shape[1]
    lead = ua.shape[:-1]
    a = ua.reshape(-1, G, d)
    b = ub.reshape(-1, G, d)
    tmp = np.einsum("ijkl,Bil->Bijk", T, b, optimize=True)
    out = np.einsum("Bijk,Bik->Bij", tmp, a, optimize=True)
    return out.reshape(*lead, G * d)


def execute_wavefunction(wf, q, dtype=np.float64):
    """``(log_abs [...], phase [...])`` for routed walkers ``q [..., N, 4]``."""
    p = _cast(wf, dtype)
    q = np.asarray(q, dtype=dtype)
    z = q @ p["Wq"]
    u_raw = ((z @ p["lV"]) * p["lh"]) @ p["lU"]                    # _factorized_apply
    rms = np.sqrt(np.mean(u_raw * u_raw, axis=-1, keepdims=True) + dtype(LEAF_EPS))
    u = u_raw / rms
    s = np.log(rms)[..., 0]
    for h, op in zip(p["mh"], p["op"]):
        ul, ur = u[..., 0::2, :], u[..., 1::2, :]
        sl, sr = s[..., 0::2], s[..., 1::2]
        raw = quadrilinear(p["T"], ul, ur)
        out = raw + ((raw @ p["mV"]) * h) @ p["mU"]
        scale = np.sqrt(np.mean(out * out, axis=-1) + p["eps"])
        cu = out / scale[..., None]
        cs = sl + sr + np.log(scale)
        both, left, right = ((op == c).astype(dtype) for c in (MERGE, CARRY_LEFT, CARRY_RIGHT))
        u = both[:, None] * cu + left[:, None] * ul + right[:, None] * ur
        s = both * cs + left * sl + right * sr
    psi = ((u[..., 0, :] @ p["rV"]) * p["rh"]) @ p["rU"]
    re, im = psi[..., 0], psi[..., 1]
    return 0.5 * np.log(re * re + im * im) + s[..., 0], np.arctan2(im, re)


# ------------------------------------------------------------------ chart
def chart_basis(q):
    """Rows c = x, y, z of d(chart)/dz_c at z = 0 for walkers q [..., N, 4]
    (kernel.py:20-37: u1 = z_z, u2 = z_y, u3 = z_x). Returns [..., N, 3, 4].
    The second derivative of the chart is -delta_ab * q."""
    q0, q1, q2, q3 = (q[..., i] for i in range(4))
    d_u1 = np.stack([-q1, q0, q3, -q2], axis=-1)
    d_u2 = np.stack([-q2, -q3, q0, q1], axis=-1)
    d_u3 = np.stack([-q3, q2, -q1, q0], axis=-1)
    return np.stack([d_u3, d_u2, d_u1], axis=-2)


# ------------------------------------------------------------------ forward Laplacian
def _normalise(out, J, L, W, eps):
    """out [M,d], J [M,m,d], L [M,d], W [M,m,m]: jets of u = out/sqrt(mean(out^2)+eps)
    and of log sqrt(.)."""
    d = out.shape[-1]
    y = np.mean(out * out, axis=-1) + eps                                   # [M]
    a = np.einsum("Mad,Md->Ma", J, out, optimize=True)                      # J out
    dy = (2.0 / d) * a                                                      # [M,m]
    gram = np.einsum("Mab,Mad,Mbd->M", W, J, J, optimize=True)              # tr(W J J^T)
    lap_y = (2.0 / d) * (np.einsum("Md,Md->M", out, L) + gram)
    Wdy = np.einsum("Mab,Mb->Ma", W, dy)
    dyWdy = np.einsum("Ma,Ma->M", dy, Wdy)
    # log sigma = 0.5 log y
    s_val = 0.5 * np.log(y)
    s_jac = 0.5 * dy / y[:, None]
    s_lap = 0.5 * (lap_y / y - dyWdy / (y * y))
    # r = y^-1/2
    r = y ** -0.5
    dr = -0.5 * (y ** -1.5)[:, None] * dy
    lap_r = -0.5 * y ** -1.5 * lap_y + 0.75 * y ** -2.5 * dyWdy
    Wdr = -0.5 * (y ** -1.5)[:, None] * Wdy
    u = out * r[:, None]
    Ju = J * r[:, None, None] + dr[:, :, None] * out[:, None, :]
    Lu = L * r[:, None] + out * lap_r[:, None] + 2.0 * np.einsum("Ma,Mad->Md", Wdr, J)
    return u, Ju, Lu, s_val, s_jac, s_lap


def forward_laplacian(wf, frame, q, dtype=np.float64, trace=None):
    """Jets of (log|psi|, phase) at z = 0 for walkers q [B,N,4]:
    value [B,2], jac [B,3N,2], lap [B,2] with lap = sum_ab J_eff[a,b] d_a d_b f.
    ``trace`` (a list) receives one dict of intermediate jets per tree level."""
    p = _cast(wf, dtype)
    q = np.asarray(q, dtype=dtype)
    B, N, _ = q.shape
    W = [np.asarray(w, dtype=dtype) for w in frame.w_levels]
    d_m = p["lU"].shape[1]
    G, d_r = p["T"].shape[0], p["T"].shape[1]

    # leaves: everything up to u_raw is linear in the quaternion
    leaf_map = np.einsum("or,nr,rm->nom", p["Wq"] @ p["lV"], p["lh"], p["lU"])   # [N,4,d_m]
    dq = chart_basis(q)                                                          # [B,N,3,4]
    val = np.einsum("bno,nom->bnm", q, leaf_map)
    J = np.einsum("bnco,nom->bncm", dq, leaf_map)                                # [B,N,3,d_m]
    trW = np.trace(W[0], axis1=-2, axis2=-1)                                     # [N]
    L = -trW[None, :, None] * val
    M = B * N
    Wb = np.broadcast_to(W[0][None], (B, N, 3, 3)).reshape(M, 3, 3)
    u, Ju, Lu, s, Js, Ls = _normalise(val.reshape(M, d_m), J.reshape(M, 3, d_m),
                                      L.reshape(M, d_m), Wb, dtype(LEAF_EPS))
    k = 1
    u = u.reshape(B, N, d_m); Ju = Ju.reshape(B, N, 3, d_m); Lu = Lu.reshape(B, N, d_m)
    s = s.reshape(B, N); Js = Js.reshape(B, N, 3); Ls = Ls.reshape(B, N)
    if trace is not None:
        trace.append(dict(u=u, J=Ju, L=Lu, s=s, Js=Js, Ls=Ls, leaf_map=leaf_map))

    for lvl, (h, op) in enumerate(zip(p["mh"], p["op"])):
        nodes = u.shape[1] // 2
        m = 3 * k
        ul, ur = u[:, 0::2], u[:, 1::2]
        Jl, Jr = Ju[:, 0::2], Ju[:, 1::2]                  # [B,nodes,m,d_m]
        Ll, Lr = Lu[:, 0::2], Lu[:, 1::2]
        W2 = W[lvl + 1]                                    # [nodes, 2m, 2m]
        Woff = W2[:, :m, m:]
        # A_R[b,n,i,j,k] = sum_l T[i,j,k,l] u_R[i,l];  A_L[b,n,i,j,l] = sum_k T[i,j,k,l] u_L[i,k]
        url = ur.reshape(B, nodes, G, d_r); ull = ul.reshape(B, nodes, G, d_r)
        A_R = np.einsum("ijkl,bnil->bnijk", p["T"], url, optimize=True)
        A_L = np.einsum("ijkl,bnik->bnijl", p["T"], ull, optimize=True)
        raw = np.einsum("bnijk,bnik->bnij", A_R, ull).reshape(B, nodes, d_m)
        Jl4 = Jl.reshape(B, nodes, m, G, d_r); Jr4 = Jr.reshape(B, nodes, m, G, d_r)
        Jraw = np.concatenate([
            np.einsum("bnijk,bnaik->bnaij", A_R, Jl4, optimize=True),
            np.einsum("bnijl,bnail->bnaij", A_L, Jr4, optimize=True)], axis=2
        ).reshape(B, nodes, 2 * m, d_m)
        Y = np.einsum("nac,bncil->bnail", Woff, Jr4, optimize=True)      # W_off J_R
        C = np.einsum("bnaik,bnail->bnikl", Jl4, Y, optimize=True)       # [B,nodes,G,d_r,d_r]
        cross = np.einsum("ijkl,bnikl->bnij", p["T"], C, optimize=True).reshape(B, nodes, d_m)
        Lraw = (np.einsum("bnijk,bnik->bnij", A_R, Ll.reshape(B, nodes, G, d_r))
                + np.einsum("bnijl,bnil->bnij", A_L, Lr.reshape(B, nodes, G, d_r))
                ).reshape(B, nodes, d_m) + 2.0 * cross
        # out = raw + ((raw V) * h) U, a linear map applied to value, Jacobian rows, Laplacian
        F = lambda x, hh: x + ((x @ p["mV"]) * hh) @ p["mU"]
        out = F(raw, h[None])
        Jout = F(Jraw, h[None, :, None, :])
        Lout = F(Lraw, h[None])
        Mn = B * nodes
        Wb = np.broadcast_to(W2[None], (B, nodes, 2 * m, 2 * m)).reshape(Mn, 2 * m, 2 * m)
        cu, cJ, cL, sv, sJ, sL = _normalise(out.reshape(Mn, d_m), Jout.reshape(Mn, 2 * m, d_m),
                                            Lout.reshape(Mn, d_m), Wb, p["eps"])
        cu = cu.reshape(B, nodes, d_m); cJ = cJ.reshape(B, nodes, 2 * m, d_m)
        cL = cL.reshape(B, nodes, d_m)
        sl, sr = s[:, 0::2], s[:, 1::2]
        cs = sl + sr + sv.reshape(B, nodes)
        cJs = np.concatenate([Js[:, 0::2], Js[:, 1::2]], axis=2) + sJ.reshape(B, nodes, 2 * m)
        cLs = Ls[:, 0::2] + Ls[:, 1::2] + sL.reshape(B, nodes)
        zJ = np.zeros_like(Jl); zs = np.zeros_like(Js[:, 0::2])
        both, left, right = ((op == c).astype(dtype) for c in (MERGE, CARRY_LEFT, CARRY_RIGHT))
        b1, l1, r1 = both[None, :, None], left[None, :, None], right[None, :, None]
        u = b1 * cu + l1 * ul + r1 * ur
        Lu = b1 * cL + l1 * Ll + r1 * Lr
        Ju = (b1[..., None] * cJ + l1[..., None] * np.concatenate([Jl, zJ], axis=2)
              + r1[..., None] * np.concatenate([zJ, Jr], axis=2))
        s = both * cs + left * sl + right * sr
        Ls = both * cLs + left * Ls[:, 0::2] + right * Ls[:, 1::2]
        Js = (b1 * cJs + l1 * np.concatenate([Js[:, 0::2], zs], axis=2)
              + r1 * np.concatenate([zs, Js[:, 1::2]], axis=2))
        k *= 2
        if trace is not None:
            trace.append(dict(raw=raw, Jraw=Jraw, Lraw=Lraw, out=out, Jout=Jout, Lout=Lout,
                              u=u, J=Ju, L=Lu, s=s, Js=Js, Ls=Ls))

    # root readout: psi = ((u V) * h) U, then log|psi| + s and atan2
    R = lambda x: ((x @ p["rV"]) * p["rh"]) @ p["rU"]
    psi = R(u[:, 0]); Jpsi = R(Ju[:, 0]); Lpsi = R(Lu[:, 0])      # [B,2], [B,3N,2], [B,2]
    Wf = W[-1][0]                                                   # full J_eff
    x, y = psi[:, 0], psi[:, 1]
    Jx, Jy = Jpsi[:, :, 0], Jpsi[:, :, 1]
    WJx = Jx @ Wf.T; WJy = Jy @ Wf.T
    Qxx = np.einsum("ba,ba->b", Jx, WJx); Qyy = np.einsum("ba,ba->b", Jy, WJy)
    Qxy = np.einsum("ba,ba->b", Jx, WJy)
    rho = x * x + y * y
    drho = 2.0 * (x[:, None] * Jx + y[:, None] * Jy)
    lap_rho = 2.0 * (x * Lpsi[:, 0] + y * Lpsi[:, 1] + Qxx + Qyy)
    drWdr = np.einsum("ba,ba->b", drho, drho @ Wf.T)
    la_val = 0.5 * np.log(rho) + s[:, 0]
    la_jac = 0.5 * drho / rho[:, None] + Js[:, 0]
    la_lap = 0.5 * (lap_rho / rho - drWdr / (rho * rho)) + Ls[:, 0]
    ph_val = np.arctan2(y, x)
    ph_jac = (x[:, None] * Jy - y[:, None] * Jx) / rho[:, None]
    ph_lap = ((-y * Lpsi[:, 0] + x * Lpsi[:, 1]) / rho
              + (2.0 * x * y * (Qxx - Qyy) + 2.0 * (y * y - x * x) * Qxy) / (rho * rho))
    value = np.stack([la_val, ph_val], axis=-1)
    jac = np.stack([la_jac, ph_jac], axis=-1)
    lap = np.stack([la_lap, ph_lap], axis=-1)
    return value, jac, lap


def local_energy(wf, frame, q, dtype=np.float64):
    """``(total, exchange, casimir, field)`` complex, shape q.shape[:-2] (kernel.py:80-119)."""
    q = np.asarray(q)
    lead = q.shape[:-2]
    N = q.shape[-2]
    value, jac, lap = forward_laplacian(wf, frame, q.reshape(-1, N, 4), dtype)
    g = jac[:, :, 0] + 1j * jac[:, :, 1]
    Jf = np.asarray(frame.J_eff, dtype=dtype)
    quad = np.einsum("ba,ac,bc->b", g, Jf, g)
    fld = 1j * np.einsum("ic,bic->b", np.asarray(frame.one_body_field, dtype=dtype),
                         0.5 * g.reshape(-1, N, 3))
    total = (lap[:, 0] + 1j * lap[:, 1]) + quad + dtype(frame.radial_const) + fld
    exchange = total - fld
    rs = lambda a: a.reshape(lead)
    return rs(total), rs(exchange), rs(np.zeros_like(total)), rs(fld)


def local_spin(wf, mask, q, dtype=np.float64):
    """``-i/2 * d(log|psi| + i phase)/dz`` masked, complex [..., N, 3] (observables.py:15-59).
    The Jacobian is taken from the forward jets (same derivative as the reference's jacrev)."""
    q = np.asarray(q)
    lead = q.shape[:-2]
    N = q.shape[-2]

    class _F:   # a frame with zero weights: only the Jacobian is used
        w_levels = [np.zeros((N // k, 3 * k, 3 * k)) for k in (1 << i for i in range(N.bit_length()))]
    _, jac, _ = forward_laplacian(wf, _F, q.reshape(-1, N, 4), dtype)
    g = (jac[:, :, 0] + 1j * jac[:, :, 1]).reshape(-1, N, 3)
    out = -0.5j * g * np.asarray(mask, dtype=dtype)[None, :, None]
    return out.reshape(*lead, N, 3)


# ------------------------------------------------------------------ dense autodiff check
def energy_dense_autodiff(wf, frame, q_single):
    """Independent fp64 evaluation for ONE walker: torch autograd builds the full
    3N x 3N Hessian of (log|psi|, phase) as functions of the chart coordinates, then
    lap = sum(J_eff * Hess). Slow (O(N) double-backward passes); small N only."""
    import torch

    tt = lambda a: torch.tensor(np.asarray(a, dtype=np.float64))
    p = dict(Wq=tt(wf.q_weight), lV=tt(wf.leaf_V), lU=tt(wf.leaf_U), lh=tt(wf.leaf_h),
             T=tt(wf.merge_T), mV=tt(wf.merge_V), mU=tt(wf.merge_U),
             mh=[tt(h) for h in wf.merge_h], rV=tt(wf.readout_V), rU=tt(wf.readout_U),
             rh=tt(wf.readout_h))
    ops = [torch.tensor(np.asarray(o).astype(np.int64)) for o in wf.opcodes]
    q = tt(q_single)
    N = q.shape[0]
    G, d_r = p["T"].shape[0], p["T"].shape[1]

    def f(zflat):
        z = zflat.reshape(N, 3)
        zx, zy, zz = z[:, 0], z[:, 1], z[:, 2]
        u0 = 1.0 - 0.5 * (zx * zx + zy * zy + zz * zz)
        u1, u2, u3 = zz, zy, zx
        q0, q1, q2, q3 = q[:, 0], q[:, 1], q[:, 2], q[:, 3]
        qp = torch.stack([q0 * u0 - q1 * u1 - q2 * u2 - q3 * u3,
                          q0 * u1 + q1 * u0 + q2 * u3 - q3 * u2,
                          q0 * u2 - q1 * u3 + q2 * u0 + q3 * u1,
                          q0 * u3 + q1 * u2 - q2 * u1 + q3 * u0], dim=-1)
        u_raw = (((qp @ p["Wq"]) @ p["lV"]) * p["lh"]) @ p["lU"]
        rms = torch.sqrt((u_raw * u_raw).mean(-1, keepdim=True) + LEAF_EPS)
        u = u_raw / rms
        s = torch.log(rms)[:, 0]
        for h, op in zip(p["mh"], ops):
            ul, ur = u[0::2], u[1::2]
            sl, sr = s[0::2], s[1::2]
            raw = torch.einsum("ijkl,nik,nil->nij", p["T"], ul.reshape(-1, G, d_r),
                               ur.reshape(-1, G, d_r)).reshape(ul.shape)
            out = raw + ((raw @ p["mV"]) * h) @ p["mU"]
            scale = torch.sqrt((out * out).mean(-1) + wf.merge_eps)
            cu = out / scale[:, None]
            cs = sl + sr + torch.log(scale)
            both, left, right = ((op == c).double() for c in (MERGE, CARRY_LEFT, CARRY_RIGHT))
            u = both[:, None] * cu + left[:, None] * ul + right[:, None] * ur
            s = both * cs + left * sl + right * sr
        psi = ((u[0] @ p["rV"]) * p["rh"]) @ p["rU"]
        return torch.stack([0.5 * torch.log(psi[0] ** 2 + psi[1] ** 2) + s[0],
                            torch.atan2(psi[1], psi[0])])

    z0 = torch.zeros(3 * N, dtype=torch.float64)
    value = f(z0).numpy()
    jac = torch.autograd.functional.jacobian(f, z0).numpy().T                    # [3N,2]
    Jf = np.asarray(frame.J_eff, dtype=np.float64)
    lap = np.array([
        (Jf * torch.autograd.functional.hessian(lambda z, i=i: f(z)[i], z0).numpy()).sum()
        for i in range(2)])
    g = jac[:, 0] + 1j * jac[:, 1]
    fld = 1j * np.sum(np.asarray(frame.one_body_field, np.float64) * 0.5 * g.reshape(N, 3))
    total = (lap[0] + 1j * lap[1]) + g @ Jf @ g + float(frame.radial_const) + fld
    return dict(value=value, jac=jac, lap=lap, total=total, field=fld)


# ------------------------------------------------------------------ reverse pass
def logpsi_vjp(wf, q, cot_log_abs, cot_phase, with_factors=False, leaf_mask=None):
    """fp64 reverse pass by torch autograd over a restatement of the executor
    (compiled/model.py:179-310 computes the same values with KFAC tags): gradients of
    ``sum_w cot_log_abs[w] log|psi_w| + cot_phase[w] phase_w`` with respect to every
    parameter array and to ``q``. Returns ``(grads: dict, dq [B,N,4], log_abs, phase)`` and,
    with ``with_factors`` (True, or "marginals" to add the sums behind the two-Kronecker marginals
    of the quadrilinear tag), a fifth item: the per-tag sums of ``x x^T`` / ``dy dy^T`` under the
    structural masks (optim/blocks.py:1122-1204) and the squared per-walker scale gradients
    (blocks.py:1288-1415)."""
    import torch

    tt = lambda a: torch.tensor(np.asarray(a, dtype=np.float64), requires_grad=True)
    p = dict(q_weight=tt(wf.q_weight), leaf_V=tt(wf.leaf_V), leaf_U=tt(wf.leaf_U),
             leaf_h=tt(wf.leaf_h), merge_T=tt(wf.merge_T), merge_V=tt(wf.merge_V),
             merge_U=tt(wf.merge_U), readout_V=tt(wf.readout_V), readout_U=tt(wf.readout_U),
             readout_h=tt(wf.readout_h))
    mh = [tt(h) for h in wf.merge_h]
    ops = [torch.tensor(np.asarray(o).astype(np.int64)) for o in wf.opcodes]
    qt = tt(np.asarray(q, dtype=np.float64).reshape(-1, wf.n_sites, 4))
    G, d_r = p["merge_T"].shape[0], p["merge_T"].shape[1]
    keep = []

    def k(x):
        x.retain_grad()
        keep.append(x)
        return x

    z = k(qt @ p["q_weight"])
    vz = k(z @ p["leaf_V"])
    mixed = k(vz * p["leaf_h"])
    u_raw = k(mixed @ p["leaf_U"])
    rms = torch.sqrt((u_raw * u_raw).mean(-1, keepdim=True) + LEAF_EPS)
    u = u_raw / rms
    s = torch.log(rms)[..., 0]
    levels = []
    for h, op in zip(mh, ops):
        ul, ur = u[:, 0::2], u[:, 1::2]
        sl, sr = s[:, 0::2], s[:, 1::2]
        B, n = ul.shape[0], ul.shape[1]
        raw = k(torch.einsum("ijkl,bnik,bnil->bnij", p["merge_T"], ul.reshape(B, n, G, d_r),
                             ur.reshape(B, n, G, d_r)).reshape(ul.shape))
        vx = k(raw @ p["merge_V"])
        mixed_l = k(vx * h)
        corr = k(mixed_l @ p["merge_U"])
        out = raw + corr
        scale = torch.sqrt((out * out).mean(-1) + wf.merge_eps)
        cu = out / scale[..., None]
        cs = sl + sr + torch.log(scale)
        both, left, right = ((op == c).double() for c in (MERGE, CARRY_LEFT, CARRY_RIGHT))
        u = both[None, :, None] * cu + left[None, :, None] * ul + right[None, :, None] * ur
        s = both[None] * cs + left[None] * sl + right[None] * sr
        levels.append((raw, vx, mixed_l, corr, both, ul, ur))
    u_root = u[:, 0]
    vr = k(u_root @ p["readout_V"])
    mixr = k(vr * p["readout_h"])
    psi = k(mixr @ p["readout_U"])
    log_abs = 0.5 * torch.log(psi[:, 0] ** 2 + psi[:, 1] ** 2) + s[:, 0]
    phase = torch.atan2(psi[:, 1], psi[:, 0])
    ca = torch.tensor(np.asarray(cot_log_abs, dtype=np.float64).reshape(-1))
    cp = torch.tensor(np.asarray(cot_phase, dtype=np.float64).reshape(-1))
    loss = (ca * log_abs).sum() + (cp * phase).sum()
    loss.backward()
    zero = lambda x: np.zeros(tuple(x.shape)) if x.grad is None else x.grad.numpy()
    out = {name: zero(x) for name, x in p.items()}
    out["merge_h"] = [zero(x) for x in mh]
    res = (out, zero(qt), log_abs.detach().numpy(), phase.detach().numpy())
    if not with_factors:
        return res
    n_ = lambda x: x.detach().numpy()
    g_ = lambda x: np.zeros(tuple(x.shape)) if x.grad is None else x.grad.numpy()
    gram = lambda a: np.einsum("ri,rj->ij", a.reshape(-1, a.shape[-1]), a.reshape(-1, a.shape[-1]))
    lm = np.ones(wf.n_sites) if leaf_mask is None else np.asarray(leaf_mask, dtype=np.float64)
    lm3 = lm[None, :, None]
    f = dict(q_in=gram(n_(qt) * lm3), q_out=gram(g_(z)),
             leaf_V_in=gram(n_(z) * lm3), leaf_V_out=gram(g_(vz)),
             leaf_U_in=gram(n_(mixed) * lm3), leaf_U_out=gram(g_(u_raw)),
             leaf_h_diag=((n_(vz) * g_(mixed) * lm3) ** 2).sum(0),
             readout_V_in=gram(n_(u_root)), readout_V_out=gram(g_(vr)),
             readout_U_in=gram(n_(mixr)), readout_U_out=gram(g_(psi)),
             readout_h_diag=((n_(vr) * g_(mixr)) ** 2).sum(0))
    d, r = wf.merge_V.shape
    f.update(merge_V_in=np.zeros((d, d)), merge_V_out=np.zeros((r, r)), merge_U_in=np.zeros((r, r)),
             merge_U_out=np.zeros((d, d)), merge_h_diag=[])
    # quadrilinear tag: sums behind the two-Kronecker marginals over the axis split (i, j | k, l)
    # (optim/spin_blocks.py:140-171: _two_kron_marginal_from_merge, _merge_gradient_trace)
    G, d_r = wf.merge_T.shape[0], wf.merge_T.shape[1]
    if with_factors == "marginals":
        f.update(merge_T_left=np.zeros((G * d_r, G * d_r)), merge_T_right=np.zeros((d_r * d_r, d_r * d_r)),
                 merge_T_stats=np.zeros(2))
    for raw, vx, mixed_l, corr, both, ul, ur in (levels if with_factors == "marginals" else []):
        keep = np.broadcast_to(both.numpy()[None, :], raw.shape[:2]).reshape(-1)
        dy = g_(raw).reshape(-1, G, d_r) * keep[:, None, None]
        ua = n_(ul).reshape(-1, G, d_r) * keep[:, None, None]
        ub = n_(ur).reshape(-1, G, d_r) * keep[:, None, None]
        ga = np.einsum("nik,nIk->niI", ua, ua) * np.einsum("nil,nIl->niI", ub, ub)
        f["merge_T_left"] += np.einsum("niI,nij,nIJ->ijIJ", ga, dy, dy,
                                       optimize=True).reshape(G * d_r, G * d_r)
        wgt = (dy * dy).sum(-1)
        f["merge_T_right"] += np.einsum("ni,nik,nil,niK,niL->klKL", wgt, ua, ub, ua, ub,
                                        optimize=True).reshape(d_r * d_r, d_r * d_r)
        f["merge_T_stats"] += np.array([(wgt * (ua * ua).sum(-1) * (ub * ub).sum(-1)).sum(), keep.sum()])
    for raw, vx, mixed_l, corr, both, ul, ur in levels:
        m3 = both.numpy()[None, :, None]
        f["merge_V_in"] += gram(n_(raw) * m3)
        f["merge_V_out"] += gram(g_(vx) * m3)
        f["merge_U_in"] += gram(n_(mixed_l) * m3)
        f["merge_U_out"] += gram(g_(corr) * m3)
        f["merge_h_diag"].append(((n_(vx) * g_(mixed_l) * m3) ** 2).sum(0))
    return res + (f,)
