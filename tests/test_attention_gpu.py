"""GPU parity of the attention kernels (through the C ABI) against the fp64 oracle.

Tolerance: 1e-4 of the tensor's largest magnitude for outputs, tangents and
gradients (the north-star bound on gradient samples), 1e-5 relative on lse."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import attention as A

pytestmark = pytest.mark.gpu
TOL = 1e-4
GOLDEN = Path(__file__).parent / "golden" / "attention_small.npz"


def _case(seed, B, N, H, D, masked, bias=True):
    rng = np.random.default_rng(seed)
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    mask = np.ones((B, N), dtype=bool)
    if masked:
        mask = rng.random((B, N)) > 0.3
        mask[:, 0] = True
        if B > 1:
            mask[-1] = False          # a batch entry with every token masked
            if N > 2:
                mask[-1, 2] = True
    c = dict(q=(f(B, N, H, D) * np.float32(D ** -0.5)), k=f(B, N, H, D), v=f(B, N, H, D),
             e=f(B, N, H, N) if bias else None, mask=mask, qt=f(B, N, H, D), kt=f(B, N, H, D),
             vt=f(B, N, H, D), et=f(B, N, H, N) if bias else None, do=f(B, N, H, D))
    return c


def _close(got, want, tol=TOL, what=""):
    got = got.detach().cpu().numpy().astype(np.float64) if torch.is_tensor(got) else got
    # error relative to the tensor's largest magnitude; inputs are O(1), so a tensor
    # that is identically zero (e.g. dq at N=1) is held to an absolute 1e-2 * tol
    scale = max(np.abs(want).max(), 1e-2)
    err = np.abs(got - want).max() / scale
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    assert err <= tol, f"{what}: max error {err:.3e} of scale > {tol}"


def _run_all(c, mode=0):
    import hamiltonzero_b200 as hz
    out, lse = hz.mhsea_fwd(c["q"], c["k"], c["e"], c["v"], c["mask"], mask_mode=mode)
    tan = hz.mhsea_jvp(c["q"], c["k"], c["e"], c["v"], c["mask"], out, lse,
                       c["qt"], c["kt"], c["et"], c["vt"], mask_mode=mode)
    dq, dk, de, dv = hz.mhsea_bwd(c["q"], c["k"], c["e"], c["v"], c["mask"], lse, out, c["do"],
                                  need_de=True, mask_mode=mode)
    torch.cuda.synchronize()
    return out, lse, tan, dq, dk, de, dv


SHAPES = [
    # B, N, H, D, masked, bias
    (3, 1, 2, 8, False, True),
    (3, 2, 2, 16, True, True),
    (2, 4, 3, 32, True, True),
    (2, 8, 32, 16, True, True),      # trunk heads at n_max=8
    (2, 16, 16, 32, True, True),     # level-edge heads
    (2, 32, 8, 64, True, True),      # router-context heads
    (5, 64, 8, 32, False, False),    # benchmark shape, no bias / no mask
    (3, 64, 8, 32, True, True),
    (3, 64, 32, 16, True, True),     # trunk heads at n_max=64: padded to 32 columns on chip
    (5, 64, 16, 16, False, False),
    (2, 64, 3, 8, True, True),       # odd head count, eight columns
    (2, 64, 4, 8, False, True),
    (2, 96, 2, 16, True, True),
    (2, 128, 2, 64, True, True),
    (1, 160, 3, 8, True, True),
    (2, 256, 2, 32, True, True),
    (1, 256, 1, 64, False, True),
    (2, 12, 2, 8, True, True),       # ragged N the reference would send to einsum
    (1, 100, 2, 16, True, False),
]


@pytest.mark.parametrize("B,N,H,D,masked,bias", SHAPES)
def test_fwd_jvp_bwd_match_oracle(hz_lib, B, N, H, D, masked, bias):
    c = _case(1000 + N * 7 + D, B, N, H, D, masked, bias)
    out, lse, tan, dq, dk, de, dv = _run_all(c)
    o, l = A.mhsea_fwd(c["q"], c["k"], c["e"], c["v"], c["mask"])
    _close(out, o, what="out")
    _close(lse, l, tol=1e-5, what="lse")
    # the tangent and the gradients are defined at the saved (out, lse): use the oracle's
    t = A.mhsea_jvp(c["q"], c["k"], c["e"], c["v"], c["mask"], o, l, c["qt"], c["kt"], c["et"], c["vt"])
    _close(tan, t, what="tangent")
    gq, gk, ge, gv = A.mhsea_bwd(c["q"], c["k"], c["e"], c["v"], c["mask"], l, o, c["do"])
    _close(dq, gq, what="dq"); _close(dk, gk, what="dk"); _close(dv, gv, what="dv")
    _close(de, ge, what="de")
    # masked query rows are exactly zero
    dead = ~c["mask"]
    assert float(out.cpu()[torch.from_numpy(dead)].abs().max() if dead.any() else 0.0) == 0.0
    assert float(tan.cpu()[torch.from_numpy(dead)].abs().max() if dead.any() else 0.0) == 0.0


@pytest.mark.parametrize("masked,bias", [(False, False), (True, True)])
def test_three_term_tf32_split_is_fp32_faithful(hz_lib, masked, bias):
    """HZ_ATTN_TF32X3 selects the three-term TF32 split on the whole-sequence kernels: the
    result must sit within 2e-5 of the tensor's scale of the fp64 oracle, five times inside
    the tolerance of this file, and lse within 2e-6. (Calls without a flag take the two-term
    BF16 split, which every other test of this file holds to 1e-4 of scale.)"""
    import hamiltonzero_b200 as hz
    c = _case(4246, 3, 64, 8, 32, masked, bias)
    out, lse, tan, dq, dk, de, dv = _run_all(c, hz.HZ_MASK_SQUARE | hz.HZ_ATTN_TF32X3)
    o, l = A.mhsea_fwd(c["q"], c["k"], c["e"], c["v"], c["mask"])
    t = A.mhsea_jvp(c["q"], c["k"], c["e"], c["v"], c["mask"], o, l, c["qt"], c["kt"], c["et"], c["vt"])
    gq, gk, ge, gv = A.mhsea_bwd(c["q"], c["k"], c["e"], c["v"], c["mask"], l, o, c["do"])
    _close(lse, l, tol=2e-6, what="default lse")
    for got, want, what in ((out, o, "out"), (tan, t, "tangent"), (dq, gq, "dq"),
                            (dk, gk, "dk"), (dv, gv, "dv"), (de, ge, "de")):
        _close(got, want, tol=2e-5, what="default " + what)


@pytest.mark.parametrize("masked,bias", [(False, False), (True, True)])
def test_single_pass_tf32_flag(hz_lib, masked, bias):
    """HZ_ATTN_TF32 permits the arithmetic of the reference's Triton kernels (one TF32
    product per contraction). Held to 5e-3 of the tensor's scale against the fp64 oracle:
    TF32 keeps 11 significant bits (4.9e-4 per operand), and scores sum 32 such products,
    gradients up to 64. Shapes outside the fast path ignore the flag bit for bit."""
    import hamiltonzero_b200 as hz
    c = _case(4242, 3, 64, 8, 32, masked, bias)
    mode = hz.HZ_MASK_SQUARE | hz.HZ_ATTN_TF32
    out, lse, tan, dq, dk, de, dv = _run_all(c, mode)
    o, l = A.mhsea_fwd(c["q"], c["k"], c["e"], c["v"], c["mask"])
    t = A.mhsea_jvp(c["q"], c["k"], c["e"], c["v"], c["mask"], o, l, c["qt"], c["kt"], c["et"], c["vt"])
    gq, gk, ge, gv = A.mhsea_bwd(c["q"], c["k"], c["e"], c["v"], c["mask"], l, o, c["do"])
    for got, want, what in ((out, o, "out"), (lse, l, "lse"), (tan, t, "tangent"), (dq, gq, "dq"),
                            (dk, gk, "dk"), (dv, gv, "dv"), (de, ge, "de")):
        _close(got, want, tol=5e-3, what="tf32 " + what)
    # and it is really a different arithmetic from the default one
    exact = _run_all(c, hz.HZ_MASK_SQUARE)
    assert not torch.equal(exact[0], out)
    dead = ~c["mask"]
    if dead.any():
        assert float(out.cpu()[torch.from_numpy(dead)].abs().max()) == 0.0
    small = _case(4243, 2, 16, 4, 32, masked, bias)
    for a, b in zip(_run_all(small, hz.HZ_MASK_SQUARE), _run_all(small, mode)):
        assert torch.equal(a, b)


@pytest.mark.parametrize("masked,bias", [(False, False), (True, True)])
def test_bf16_split_flag(hz_lib, masked, bias):
    """HZ_ATTN_BF16X3 names the default arithmetic of the whole-sequence kernels: a two-term BF16
    split (three BF16 products per fp32 product, fp32 accumulation). A product is exact to about
    3 * 2^-16 of its magnitude; every output is held to 1e-4 of the tensor's scale (lse 1e-5).
    Shapes outside the fast path ignore the flag bit for bit."""
    import hamiltonzero_b200 as hz
    c = _case(4244, 3, 64, 8, 32, masked, bias)
    mode = hz.HZ_MASK_SQUARE | hz.HZ_ATTN_BF16X3
    out, lse, tan, dq, dk, de, dv = _run_all(c, mode)
    o, l = A.mhsea_fwd(c["q"], c["k"], c["e"], c["v"], c["mask"])
    t = A.mhsea_jvp(c["q"], c["k"], c["e"], c["v"], c["mask"], o, l, c["qt"], c["kt"], c["et"], c["vt"])
    gq, gk, ge, gv = A.mhsea_bwd(c["q"], c["k"], c["e"], c["v"], c["mask"], l, o, c["do"])
    _close(lse, l, tol=1e-5, what="bf16x3 lse")
    for got, want, what in ((out, o, "out"), (tan, t, "tangent"), (dq, gq, "dq"),
                            (dk, gk, "dk"), (dv, gv, "dv"), (de, ge, "de")):
        _close(got, want, tol=1e-4, what="bf16x3 " + what)
    # this is the arithmetic of calls that carry no flag, and not the three-term TF32 split's bits
    for x, y in zip(_run_all(c, hz.HZ_MASK_SQUARE), (out, lse, tan, dq, dk, de, dv)):
        assert torch.equal(x, y)
    exact = _run_all(c, hz.HZ_MASK_SQUARE | hz.HZ_ATTN_TF32X3)
    assert not torch.equal(exact[0], out)
    dead = ~c["mask"]
    if dead.any():
        assert float(out.cpu()[torch.from_numpy(dead)].abs().max()) == 0.0
    small = _case(4245, 2, 16, 4, 32, masked, bias)
    for a, b in zip(_run_all(small, hz.HZ_MASK_SQUARE), _run_all(small, mode)):
        assert torch.equal(a, b)


@pytest.mark.parametrize("masked,bias", [(False, False), (True, True)])
def test_fp16_split_flag(hz_lib, masked, bias):
    """HZ_ATTN_FP16X3: two-term FP16 split (22 significant bits per operand, three products).
    For operands inside the FP16 range the results must sit as close to the fp64 oracle as the
    default arithmetic's: 2e-5 of scale, lse 2e-6; and they are not the default's bits."""
    import hamiltonzero_b200 as hz
    c = _case(4247, 3, 64, 8, 32, masked, bias)
    mode = hz.HZ_MASK_SQUARE | hz.HZ_ATTN_FP16X3
    out, lse, tan, dq, dk, de, dv = _run_all(c, mode)
    o, l = A.mhsea_fwd(c["q"], c["k"], c["e"], c["v"], c["mask"])
    t = A.mhsea_jvp(c["q"], c["k"], c["e"], c["v"], c["mask"], o, l, c["qt"], c["kt"], c["et"], c["vt"])
    gq, gk, ge, gv = A.mhsea_bwd(c["q"], c["k"], c["e"], c["v"], c["mask"], l, o, c["do"])
    _close(lse, l, tol=2e-6, what="fp16x3 lse")
    for got, want, what in ((out, o, "out"), (tan, t, "tangent"), (dq, gq, "dq"),
                            (dk, gk, "dk"), (dv, gv, "dv"), (de, ge, "de")):
        _close(got, want, tol=2e-5, what="fp16x3 " + what)
    exact = _run_all(c, hz.HZ_MASK_SQUARE)
    assert not torch.equal(exact[0], out)
    dead = ~c["mask"]
    if dead.any():
        assert float(out.cpu()[torch.from_numpy(dead)].abs().max()) == 0.0


@pytest.mark.parametrize("D,flag", [(16, "HZ_ATTN_TF32X3"), (8, "HZ_ATTN_FP16X3"), (16, "HZ_ATTN_TF32")])
def test_padded_head_dimensions_in_every_arithmetic(hz_lib, D, flag):
    """N = 64 with D = 8 or 16 runs the whole-sequence kernels on tiles zero-padded to 32
    columns in shared memory; every arithmetic must agree with the oracle there as at D = 32
    (single TF32 at its own tolerance), and nothing beyond column D may be written: the
    outputs live in buffers with a guard row behind them."""
    import hamiltonzero_b200 as hz
    c = _case(5000 + D, 3, 64, 6, D, True, True)
    mode = hz.HZ_MASK_SQUARE | getattr(hz, flag)
    out, lse, tan, dq, dk, de, dv = _run_all(c, mode)
    tol = 5e-3 if flag == "HZ_ATTN_TF32" else 1e-4
    o, l = A.mhsea_fwd(c["q"], c["k"], c["e"], c["v"], c["mask"])
    t = A.mhsea_jvp(c["q"], c["k"], c["e"], c["v"], c["mask"], o, l, c["qt"], c["kt"], c["et"], c["vt"])
    gq, gk, ge, gv = A.mhsea_bwd(c["q"], c["k"], c["e"], c["v"], c["mask"], l, o, c["do"])
    _close(out, o, tol=tol, what="out"); _close(tan, t, tol=tol, what="tangent")
    _close(dq, gq, tol=tol, what="dq"); _close(dk, gk, tol=tol, what="dk"); _close(dv, gv, tol=tol, what="dv")
    # the generic kernels (HZ_MASK_KEYS never takes the fast path) agree on unmasked input
    c2 = _case(5100 + D, 2, 64, 4, D, False, True)
    a1, _ = hz.mhsea_fwd(c2["q"], c2["k"], c2["e"], c2["v"], c2["mask"], mask_mode=hz.HZ_MASK_SQUARE | hz.HZ_ATTN_TF32X3)
    a2, _ = hz.mhsea_fwd(c2["q"], c2["k"], c2["e"], c2["v"], c2["mask"], mask_mode=hz.HZ_MASK_KEYS)
    to_np = lambda x: x.detach().cpu().numpy() if torch.is_tensor(x) else np.asarray(x)
    assert np.abs(to_np(a1) - to_np(a2)).max() <= 2e-5 * np.abs(to_np(a2)).max()


@pytest.mark.parametrize("B,H,masked,bias", [(1, 2, False, False), (3, 8, False, False),
                                             (3, 8, True, True), (5, 4, True, False)])
def test_tcgen05_forward_kernel(hz_lib, B, H, masked, bias):
    """The opt-in tcgen05 / TMEM / TMA forward kernel (flag HZ_ATTN_TCGEN05) against the fp64
    oracle at the default tolerance, masked rows exactly zero."""
    import hamiltonzero_b200 as hz
    c = _case(900 + B + H, B, 64, H, 32, masked, bias)
    mode = hz.HZ_MASK_SQUARE | hz.HZ_ATTN_TCGEN05
    out, lse = hz.mhsea_fwd(c["q"], c["k"], c["e"], c["v"], c["mask"], mask_mode=mode)
    torch.cuda.synchronize()
    o, l = A.mhsea_fwd(c["q"], c["k"], c["e"], c["v"], c["mask"])
    _close(out, o, what="tcgen05 out")
    _close(lse, l, tol=1e-5, what="tcgen05 lse")
    dead = ~c["mask"]
    if dead.any():
        assert float(out.cpu()[torch.from_numpy(dead)].abs().max()) == 0.0
    ref, _ = hz.mhsea_fwd(c["q"], c["k"], c["e"], c["v"], c["mask"],
                          mask_mode=hz.HZ_MASK_SQUARE | hz.HZ_ATTN_TF32X3)      # same arithmetic
    assert (out - ref).abs().max().item() <= 1e-5 * ref.abs().max().item()


def test_golden_vectors(hz_lib):
    blob = np.load(GOLDEN)
    for name in ("n8", "n64", "n96"):
        g = {k[len(name) + 1:]: blob[k] for k in blob.files if k.startswith(name + "_")}
        out, lse, tan, dq, dk, de, dv = _run_all(g)
        _close(out, g["out"], what=name + ".out"); _close(lse, g["lse"], 1e-5, name + ".lse")
        _close(tan, g["tan"], what=name + ".tan")
        for got, key in ((dq, "dq"), (dk, "dk"), (de, "de"), (dv, "dv")):
            _close(got, g[key], what=f"{name}.{key}")


def test_null_bias_and_mask_equal_zero_bias_full_mask(hz_lib):
    import hamiltonzero_b200 as hz
    c = _case(7, 4, 64, 8, 32, masked=False, bias=False)
    z = np.zeros((4, 64, 8, 64), np.float32)
    o1, l1 = hz.mhsea_fwd(c["q"], c["k"], None, c["v"], None)
    o2, l2 = hz.mhsea_fwd(c["q"], c["k"], z, c["v"], np.ones((4, 64), bool))
    assert torch.equal(o1, o2) and torch.equal(l1, l2)


def test_runs_are_bitwise_deterministic_and_fill_outputs(hz_lib):
    c = _case(8, 3, 64, 4, 32, masked=True)
    a = _run_all(c)
    b = _run_all(c)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
        assert torch.isfinite(x).all()


def test_adjoint_identity_at_benchmark_size(hz_lib):
    """Size-independent property at the full benchmark shape: <dO, JVP(t)> = <grads, t>."""
    import hamiltonzero_b200 as hz
    B, N, H, D = 4096, 64, 8, 32
    gen = torch.Generator(device="cuda").manual_seed(2)
    r = lambda *s: torch.randn(*s, device="cuda", generator=gen)
    q, k, v = r(B, N, H, D) * D ** -0.5, r(B, N, H, D), r(B, N, H, D)
    qt, kt, vt, do = r(B, N, H, D), r(B, N, H, D), r(B, N, H, D), r(B, N, H, D)
    out, lse = hz.mhsea_fwd(q, k, None, v, None)
    tan = hz.mhsea_jvp(q, k, None, v, None, out, lse, qt, kt, None, vt)
    dq, dk, _, dv = hz.mhsea_bwd(q, k, None, v, None, lse, out, do, need_de=False)
    lhs = (do.double() * tan.double()).sum().item()
    rhs = ((dq.double() * qt.double()).sum() + (dk.double() * kt.double()).sum()
           + (dv.double() * vt.double()).sum()).item()
    assert abs(lhs - rhs) <= 1e-4 * (do.double().norm() * tan.double().norm()).item()
    # softmax rows sum to one: with V = 1 the output is 1 everywhere
    ones = torch.ones_like(v)
    o1, _ = hz.mhsea_fwd(q, k, None, ones, None)
    assert (o1 - 1).abs().max().item() <= 1e-5


def test_keys_mode_matches_einsum_twin(hz_lib):
    import hamiltonzero_b200 as hz
    rng = np.random.default_rng(11)
    for n, h, d in [(12, 2, 8), (16, 4, 16), (100, 2, 32), (20, 2, 12)]:
        Q, K, V = (rng.standard_normal((n, h, d)).astype(np.float32) for _ in range(3))
        bias = rng.standard_normal((n, n, h)).astype(np.float32)
        mask = (rng.random(n) > 0.3).astype(np.int32); mask[0] = 1
        got = hz.reference_edge_attention(Q, K, V, bias, mask)
        _close(got, A.reference_edge_attention(Q, K, V, bias, mask), what=f"einsum n={n}")


def test_dispatcher_and_autograd(hz_lib):
    import hamiltonzero_b200 as hz
    rng = np.random.default_rng(12)
    n, h, d = 64, 4, 16
    Q, K, V = (torch.tensor(rng.standard_normal((n, h, d)).astype(np.float32), device="cuda",
                            requires_grad=True) for _ in range(3))
    bias = torch.tensor(rng.standard_normal((n, n, h)).astype(np.float32), device="cuda",
                        requires_grad=True)
    mask = (rng.random(n) > 0.2).astype(np.int32); mask[0] = 1
    out = hz.mhsea_tuned_edge_attention(Q, K, V, bias, torch.tensor(mask, device="cuda"))
    want = A.mhsea_tuned_edge_attention(Q.detach().cpu().numpy(), K.detach().cpu().numpy(),
                                        V.detach().cpu().numpy(), bias.detach().cpu().numpy(), mask)
    _close(out, want, what="dispatcher out")
    do = rng.standard_normal((n, h, d)).astype(np.float32)
    out.backward(torch.tensor(do, device="cuda"))
    # oracle gradients through the dispatcher: dQ = D^-1/2 dq', dbias = de transposed
    q4 = Q.detach().cpu().numpy()[None] * d ** -0.5
    e4 = np.transpose(bias.detach().cpu().numpy(), (0, 2, 1))[None]
    m4 = mask.astype(bool)[None]
    o, l = A.mhsea_fwd(q4, K.detach().cpu().numpy()[None], e4, V.detach().cpu().numpy()[None], m4)
    gq, gk, ge, gv = A.mhsea_bwd(q4, K.detach().cpu().numpy()[None], e4,
                                 V.detach().cpu().numpy()[None], m4, l, o, do[None])
    _close(Q.grad, gq[0] * d ** -0.5, what="dQ"); _close(K.grad, gk[0], what="dK")
    _close(V.grad, gv[0], what="dV"); _close(bias.grad, np.transpose(ge[0], (0, 2, 1)), what="dbias")


@pytest.mark.parametrize("n,n_heads,d,impl", [(64, 2, 8, "mhsea_tuned"), (16, 4, 16, "mhsea_tuned"),
                                              (64, 4, 32, "mhsea_tuned"), (20, 2, 8, "einsum")])
def test_gated_block_around_the_op(hz_lib, n, n_heads, d, impl):
    """The callers' shell (head padding to 16, Q rescaling, sigmoid gate of the first half of
    the kernel heads: model/trunk.py:108-137) against the oracle, and its gradients against a
    torch fp64 restatement with every token real (where both mask conventions coincide)."""
    import hamiltonzero_b200 as hz
    rng = np.random.default_rng(13)
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    Q, K, V, bias = f(n, 2 * n_heads, d), f(n, 2 * n_heads, d), f(n, 2 * n_heads, d), f(n, n, 2 * n_heads)
    mask = (rng.random(n) > 0.25).astype(np.int32); mask[0] = 1
    got = hz.gated_edge_attention(Q, K, V, bias, mask, n_heads, impl)
    _close(got, A.gated_edge_attention(Q, K, V, bias, mask, n_heads, impl), what="gated block")

    ones = np.ones(n, dtype=np.int32)
    dev = [torch.tensor(x, device="cuda", requires_grad=True) for x in (Q, K, V, bias)]
    out = hz.gated_edge_attention(*dev, torch.tensor(ones, device="cuda"), n_heads, impl)
    do = f(n, n_heads * d)
    out.backward(torch.tensor(do, device="cuda"))
    ref = [torch.tensor(x, dtype=torch.float64, requires_grad=True) for x in (Q, K, V, bias)]
    s = torch.einsum("ihd,jhd->ihj", ref[0], ref[1]) * d ** -0.5 + ref[3].permute(0, 2, 1)
    o = torch.einsum("ihj,jhd->ihd", torch.softmax(s, -1), ref[2])
    o = (torch.sigmoid(o[:, :n_heads]) * o[:, n_heads:]).reshape(n, -1)
    _close(out, o.detach().numpy(), what="gated block, all real")
    o.backward(torch.tensor(do, dtype=torch.float64))
    for g, r, what in zip(dev, ref, ("dQ", "dK", "dV", "dbias")):
        _close(g.grad, r.grad.numpy(), what="gated block " + what)


def test_rejects_wrong_dtype_and_shapes(hz_lib):
    import hamiltonzero_b200 as hz
    q = torch.zeros(1, 8, 1, 8, device="cuda")
    with pytest.raises(TypeError):
        hz.mhsea_fwd(q.double(), q, None, q, None)
    with pytest.raises(ValueError):
        hz.mhsea_fwd(q, q[:, :4], None, q, None)
    with pytest.raises(hz._lib.HzError):
        big = torch.zeros(1, 512, 1, 8, device="cuda")
        hz.mhsea_fwd(big, big, None, big, None)


def test_forward_mode_rule_and_its_transpose(hz_lib):
    """The two differentiation rules of the primitive (mhsea_tuned.py:104-118,206-221): forward
    mode binds the primal and the linear tangent kernel (checked with torch.autograd.forward_ad
    against the oracle's tangent); reverse mode through the linear tangent op is the backward
    kernel, and the two satisfy <dO, JVP(t)> = <VJP(dO), t>."""
    import torch.autograd.forward_ad as fwAD
    import hamiltonzero_b200 as hz
    from hamiltonzero_b200.attention import _MhseaFunction
    c = _case(77, 2, 64, 4, 16, True, True)
    t = lambda a: torch.tensor(a, device="cuda")
    q, k, e, v = t(c["q"]), t(c["k"]), t(c["e"]), t(c["v"])
    qt, kt, et, vt = t(c["qt"]), t(c["kt"]), t(c["et"]), t(c["vt"])
    mask = torch.tensor(c["mask"].astype(np.uint8), device="cuda")
    with fwAD.dual_level():
        dq_, dk_, de_, dv_ = (fwAD.make_dual(p, tg) for p, tg in ((q, qt), (k, kt), (e, et), (v, vt)))
        out, lse = _MhseaFunction.apply(dq_, dk_, de_, dv_, mask, hz.HZ_MASK_SQUARE)
        primal, tangent = fwAD.unpack_dual(out)
        assert fwAD.unpack_dual(lse).tangent is None          # symbolically zero, as in the reference
    o, l = A.mhsea_fwd(c["q"], c["k"], c["e"], c["v"], c["mask"])
    want = A.mhsea_jvp(c["q"], c["k"], c["e"], c["v"], c["mask"], o, l, c["qt"], c["kt"], c["et"], c["vt"])
    _close(primal, o, what="forward-mode primal")
    _close(tangent, want, what="forward-mode tangent")
    # transpose of the linear tangent op
    tans = [x.clone().requires_grad_(True) for x in (qt, kt, et, vt)]
    lin = hz.mhsea_linear_tangent(q, k, e, v, mask, primal.detach(), lse.detach(), *tans)
    _close(lin, want, what="linear tangent op")
    do = t(c["do"])
    lin.backward(do)
    gq, gk, ge, gv = A.mhsea_bwd(c["q"], c["k"], c["e"], c["v"], c["mask"], l, o, c["do"])
    for got, ref, what in zip([x.grad for x in tans], (gq, gk, ge, gv), ("dqt", "dkt", "det", "dvt")):
        _close(got, ref, what="transpose " + what)
    lhs = float((do.double() * tangent.double()).sum())
    rhs = sum(float((g.grad.double() * x.double()).sum()) for g, x in zip(tans, (qt, kt, et, vt)))
    # both sides carry the op's 1e-4-of-scale rounding on every element: the identity holds to
    # that fraction of |dO| |JVP| (this shape runs the default two-term BF16 split)
    bound = float(do.double().norm() * tangent.double().norm())
    assert abs(lhs - rhs) <= 1e-4 * max(bound, 1.0)
