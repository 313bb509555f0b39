"""GPU parity of the walker-batch operators (through the C ABI) against the fp64 oracle.

Tolerances (north star: 1e-5 relative on log-amplitudes, 1e-4 relative on local-energy
and spin samples). The local energy is a sum of cancelling terms (Laplacian, quadratic
form, radial constant), each far larger than the total; an fp32 evaluation - the
reference's own precision - is accurate to about 1e-7 of those terms, not of the total.
Energies are therefore held to 1e-4 relative to max(|E|, 1e-2 * term scale), and the
test also checks the error against the term scale at 1e-5."""
import numpy as np
import pytest
import torch

from hamiltonzero_b200 import systems as S
from oracle import walker as W

pytestmark = pytest.mark.gpu

SMALL = dict(d_o=8, d_m=64, d_r=32, r_leaf=16, r_merge=16, r_ro=8)
MID = dict(d_o=16, d_m=256, d_r=32, r_leaf=32, r_merge=64, r_ro=16)


def _problem(n, dims, n_real=None, seed=0, p=0.5, graph=None):
    n_real = n if n_real is None else n_real
    if graph is None:
        graph = S.erdos_renyi_exchange_graph(n_real, p, seed=7) if n_real > 1 else S.chain_graph(1)
    frame = S.frame_from_graph(graph, n)
    wf = S.synthetic_wavefunction(seed, n, n_real=n_real, **dims)
    return frame, wf


def _check_energy(got, ref, scale, what):
    got = [np.asarray(g, dtype=np.complex128) for g in got]
    total, exchange, casimir, field = got
    err = np.abs(total - ref[0])
    assert np.isfinite(total.view(np.float64)).all(), what
    assert (err / scale).max() <= 1e-5, f"{what}: {(err / scale).max():.2e} of the term scale"
    rel = err / np.maximum(np.abs(ref[0]), 1e-2 * scale)
    assert rel.max() <= 1e-4, f"{what}: relative error {rel.max():.2e}"
    ferr = np.abs(field - ref[3]) / max(np.abs(ref[3]).max(), 1e-3)
    assert ferr.max() <= 1e-4, f"{what}: field channel {ferr.max():.2e}"
    np.testing.assert_allclose(exchange, total - field, rtol=0, atol=1e-5 * scale.max())
    assert np.all(casimir == 0)


def _term_scale(wf, frame, q):
    _, _, lap = W.forward_laplacian(wf, frame, q.reshape(-1, q.shape[-2], 4))
    return np.abs(lap[:, 0] + 1j * lap[:, 1]) + abs(float(frame.radial_const)) + 1.0


CASES = [
    # n, dims, n_real, walkers
    (1, SMALL, None, 7),
    (2, SMALL, None, 9),
    (4, SMALL, None, 9),
    (8, SMALL, None, 17),
    (8, SMALL, 5, 6),
    (16, SMALL, 11, 6),
    (16, MID, None, 5),
    (4, MID, None, 5),               # the second level is the root
    (4, MID, 3, 4),
    (8, MID, None, 9),               # more walkers than one coefficient tile of 8
    (16, MID, 6, 5),                 # second-level node carrying its left child
    (16, MID, 5, 5),                 # ... which itself carries a leaf
    (16, MID, 13, 4),
    (32, MID, 19, 4),
    (64, SMALL, None, 3),
    (128, MID, 100, 2),              # 7 levels, ragged
    (256, SMALL, None, 2),           # the largest supported tree (the 16x16 lattice of the largest benchmark configuration)
]


@pytest.mark.parametrize("n,dims,n_real,walkers", CASES)
def test_logpsi_energy_spin_match_oracle(hz_lib, n, dims, n_real, walkers):
    import hamiltonzero_b200 as hz
    frame, wf = _problem(n, dims, n_real)
    q = S.random_unit_quaternions(np.random.default_rng(n + walkers), (walkers, n))
    cw = hz.CompiledWaveFunction(wf)
    la, ph = cw(q)
    la0, ph0 = W.execute_wavefunction(wf, q)
    assert np.abs(la - la0).max() <= 1e-5 * np.abs(la0).max() + 1e-5
    # the phase accumulates one rounding per tree level: 2e-5 rad up to 32 sites, 5e-5 above
    assert np.abs(np.angle(np.exp(1j * (ph - ph0)))).max() <= (2e-5 if n <= 32 else 5e-5)
    got = hz.vmc_energy_custom_lap_compiled(cw, frame, q)
    ref = W.local_energy(wf, frame, q)
    _check_energy(got, ref, _term_scale(wf, frame, q), f"N={n}")
    spin = hz.local_spin(cw, frame, q)
    spin0 = W.local_spin(wf, frame.mask, q)
    assert np.abs(spin - spin0).max() <= 1e-4 * max(np.abs(spin0).max(), 1e-2)
    if n_real is not None:
        assert np.all(spin[:, n_real:] == 0)


def test_config1_chain8_full_model(hz_lib):
    """The smallest benchmark configuration: 8-site open Heisenberg chain, default model sizes, walkers x
    replicas of random Sz=0 basis states as corner quaternions (a 64-walker sample is
    compared with the oracle; the full 256 x 8 batch is checked for consistency)."""
    import hamiltonzero_b200 as hz
    n = 8
    frame = S.frame_from_graph(S.chain_graph(n), n)
    wf = S.synthetic_wavefunction(0, n)
    rng = np.random.default_rng(1)
    bits = np.stack([rng.permutation(np.arange(n) % 2) for _ in range(256 * 8)]).reshape(256, 8, n)
    q = S.corner_quaternions(bits)
    cw = hz.CompiledWaveFunction(wf)
    la, ph = cw(q)
    assert la.shape == (256, 8)
    tot = hz.vmc_energy_custom_lap_compiled(cw, frame, q)
    assert tot[0].shape == (256, 8)
    sub = q[:8]
    la0, ph0 = W.execute_wavefunction(wf, sub)
    assert np.abs(la[:8] - la0).max() <= 1e-5 * np.abs(la0).max()
    assert np.abs(np.angle(np.exp(1j * (ph[:8] - ph0)))).max() <= 2e-5
    ref = W.local_energy(wf, frame, sub)
    _check_energy([t[:8].reshape(-1) for t in tot], [r.reshape(-1) for r in ref],
                  _term_scale(wf, frame, sub), "chain-8")
    # the same basis state always gives the same sample
    flat_bits = bits.reshape(-1, n)
    _, first, inverse = np.unique(flat_bits, axis=0, return_index=True, return_inverse=True)
    e = tot[0].reshape(-1)
    assert np.abs(e - e[first][inverse]).max() == 0.0


def test_config4_er64_full_model_sample(hz_lib):
    """The headline benchmark configuration: 64-site Erdos-Renyi graph, random 3x3 exchange and
    fields, default model sizes, uniformly random +-1/2 spins; two walkers against the oracle."""
    import hamiltonzero_b200 as hz
    n = 64
    frame = S.frame_from_graph(S.erdos_renyi_exchange_graph(64, 0.1, seed=7), n)
    wf = S.synthetic_wavefunction(0, n)
    q = S.corner_quaternions(np.random.default_rng(4).integers(0, 2, (2, n)))
    cw = hz.CompiledWaveFunction(wf)
    la, ph = cw(q)
    la0, ph0 = W.execute_wavefunction(wf, q)
    assert np.abs(la - la0).max() <= 1e-5 * np.abs(la0).max()
    assert np.abs(np.angle(np.exp(1j * (ph - ph0)))).max() <= 5e-5
    got = hz.vmc_energy_custom_lap_compiled(cw, frame, q)
    ref = W.local_energy(wf, frame, q)
    _check_energy(got, ref, _term_scale(wf, frame, q), "ER-64")
    spin = hz.local_spin(cw, frame, q)
    spin0 = W.local_spin(wf, frame.mask, q)
    assert np.abs(spin - spin0).max() <= 1e-4 * np.abs(spin0).max()


def test_j1j2_4x4_full_model_sample(hz_lib):
    """The 16-site benchmark configuration: periodic 4x4 J1-J2 lattice (J1 = 1 on nearest
    neighbours, J2 = 0.5 on diagonals, no field), default model sizes, random Sz = 0 corner
    walkers; three walkers against the oracle."""
    import hamiltonzero_b200 as hz
    n = 16
    frame = S.frame_from_graph(S.j1j2_square_graph(4), n)
    wf = S.synthetic_wavefunction(0, n)
    rng = np.random.default_rng(3)
    bits = np.stack([rng.permutation(np.arange(n) % 2) for _ in range(3)])
    q = S.corner_quaternions(bits)
    cw = hz.CompiledWaveFunction(wf)
    la, ph = cw(q)
    la0, ph0 = W.execute_wavefunction(wf, q)
    assert np.abs(la - la0).max() <= 1e-5 * np.abs(la0).max()
    assert np.abs(np.angle(np.exp(1j * (ph - ph0)))).max() <= 5e-5
    got = hz.vmc_energy_custom_lap_compiled(cw, frame, q)
    ref = W.local_energy(wf, frame, q)
    _check_energy(got, ref, _term_scale(wf, frame, q), "J1-J2 4x4")
    spin = hz.local_spin(cw, frame, q)
    spin0 = W.local_spin(wf, frame.mask, q)
    assert np.abs(spin - spin0).max() <= 1e-4 * np.abs(spin0).max()


@pytest.mark.parametrize("n,n_real,walkers", [(128, None, 1), (128, 100, 1), (256, None, 1)])
def test_wide_trees_at_default_model_sizes(hz_lib, n, n_real, walkers):
    """Seven- and eight-level trees at the full carrier width (d_m = 1536, rank 256): log-psi,
    the four energy channels and the spin of one walker against the oracle."""
    import hamiltonzero_b200 as hz
    n_r = n if n_real is None else n_real
    frame = S.frame_from_graph(S.erdos_renyi_exchange_graph(n_r, 0.05, seed=7), n)
    wf = S.synthetic_wavefunction(0, n, n_real=n_r)
    q = S.random_unit_quaternions(np.random.default_rng(n), (walkers, n))
    cw = hz.CompiledWaveFunction(wf)
    la, ph = cw(q)
    la0, ph0 = W.execute_wavefunction(wf, q)
    assert np.abs(la - la0).max() <= 1e-5 * np.abs(la0).max()
    assert np.abs(np.angle(np.exp(1j * (ph - ph0)))).max() <= 5e-5
    got = hz.vmc_energy_custom_lap_compiled(cw, frame, q)
    ref = W.local_energy(wf, frame, q)
    _check_energy(got, ref, _term_scale(wf, frame, q), f"N={n} full width")
    spin = hz.local_spin(cw, frame, q)
    spin0 = W.local_spin(wf, frame.mask, q)
    assert np.abs(spin - spin0).max() <= 1e-4 * np.abs(spin0).max()
    if n_real is not None:
        assert np.all(spin[:, n_real:] == 0)


def test_j1j2_4x4_full_batch_properties(hz_lib):
    """The 16-site configuration at its full size (4096 walkers, default model sizes) through
    size-independent properties: finite samples, exchange = total - field (no field: exactly
    total), zero field channel, bitwise equality with the same walkers evaluated on their own
    and under another chunking, and eight of them against the oracle."""
    import hamiltonzero_b200 as hz
    n, B = 16, 4096
    frame = S.frame_from_graph(S.j1j2_square_graph(4), n)
    wf = S.synthetic_wavefunction(0, n)
    rng = np.random.default_rng(3)
    bits = np.stack([rng.permutation(np.arange(n) % 2) for _ in range(B)])
    q = torch.as_tensor(S.corner_quaternions(bits), device="cuda")
    cw = hz.CompiledWaveFunction(wf)
    dfr = hz.DeviceEnergyFrame(frame)
    tot, exc, cas, fld = hz.vmc_energy_custom_lap_compiled(cw, dfr, q, chunk_size=None)
    assert tot.shape == (B,)
    assert torch.isfinite(torch.view_as_real(tot)).all()
    assert (fld == 0).all() and (cas == 0).all() and torch.equal(exc, tot)
    again = hz.vmc_energy_custom_lap_compiled(cw, dfr, q, chunk_size=512)
    assert torch.equal(again[0], tot)
    # a global SU(2) rotation of every site leaves the isotropic Hamiltonian's samples unchanged
    # only up to the wavefunction, so the invariant used here is the basis-state one: equal
    # spin configurations give equal samples
    _, first, inverse = np.unique(bits, axis=0, return_index=True, return_inverse=True)
    e = tot.cpu().numpy()
    assert np.abs(e - e[first][inverse]).max() == 0.0
    pick = torch.cat([q[:5], q[-3:]])
    alone = hz.vmc_energy_custom_lap_compiled(cw, dfr, pick)
    assert torch.equal(alone[0], torch.cat([tot[:5], tot[-3:]]))
    ref = W.local_energy(wf, frame, pick.cpu().numpy())
    _check_energy([a.cpu().numpy() for a in alone], ref, _term_scale(wf, frame, pick.cpu().numpy()),
                  "J1-J2 4x4 full batch sample")


def test_leaf_map_scale_does_not_change_the_result(hz_lib):
    """log-psi minus the leaf scale and every energy channel are invariant under a rescaling of
    the leaf map (the leaf carriers are RMS-normalised), so the kernels must not depend on its
    magnitude: the leaf weights scaled by 1e-4 and by 1e+4 give the oracle's values."""
    import hamiltonzero_b200 as hz
    n = 16
    frame, wf = _problem(n, MID)
    q = S.random_unit_quaternions(np.random.default_rng(12), (4, n))
    base = W.local_energy(wf, frame, q)
    scale = _term_scale(wf, frame, q)
    leaf_U = np.array(wf.leaf_U, copy=True)
    for factor in (1e-4, 1e4):
        wf.leaf_U = (leaf_U * factor).astype(np.float32)
        cw = hz.CompiledWaveFunction(wf)
        la, _ = cw(q)
        la0, _ = W.execute_wavefunction(wf, q)
        assert np.abs(la - la0).max() <= 1e-5 * np.abs(la0).max() + 1e-5
        got = hz.vmc_energy_custom_lap_compiled(cw, frame, q)
        ref = W.local_energy(wf, frame, q)
        np.testing.assert_allclose(ref[0], base[0], rtol=2e-6, atol=2e-6)     # fp32 rounding of the scaled weights
        _check_energy(got, ref, scale, f"leaf map x {factor:g}")
    wf.leaf_U = leaf_U


def test_results_do_not_depend_on_chunk_size(hz_lib):
    import hamiltonzero_b200 as hz
    frame, wf = _problem(8, MID)
    q = S.random_unit_quaternions(np.random.default_rng(3), (37, 8))
    cw = hz.CompiledWaveFunction(wf)
    a = hz.vmc_energy_custom_lap_compiled(cw, frame, q, chunk_size=None)
    b = hz.vmc_energy_custom_lap_compiled(cw, frame, q, chunk_size=5)
    c = hz.vmc_energy_custom_lap_compiled(cw, frame, q, chunk_size=16)
    for x, y, z in zip(a, b, c):
        assert np.array_equal(x, y) and np.array_equal(x, z)
    la1, _ = cw(q, chunk_size=3)
    la2, _ = cw(q)
    assert np.array_equal(la1, la2)


def test_er64_energy_is_reproducible_and_chunk_independent(hz_lib):
    """At the benchmark size every reduction of the energy pass runs in a fixed order: the same
    walkers give the same bits on a second call and under another chunking."""
    import hamiltonzero_b200 as hz
    n = 64
    frame = S.frame_from_graph(S.erdos_renyi_exchange_graph(64, 0.1, seed=7), n)
    wf = S.synthetic_wavefunction(0, n)
    q = S.corner_quaternions(np.random.default_rng(5).integers(0, 2, (7, n)))
    cw = hz.CompiledWaveFunction(wf)
    a = hz.vmc_energy_custom_lap_compiled(cw, frame, q)
    b = hz.vmc_energy_custom_lap_compiled(cw, frame, q)
    c = hz.vmc_energy_custom_lap_compiled(cw, frame, q, chunk_size=3)
    for x, y, z in zip(a, b, c):
        assert np.array_equal(x, y) and np.array_equal(x, z)


def test_er64_full_batch_properties(hz_lib):
    """The headline configuration at its full size (16384 walkers, 64 sites, default model
    sizes) through size-independent properties: every sample finite, exchange = total - field,
    field = -sum h.spin, and the first and last walkers of the batch bitwise equal to the same
    walkers evaluated on their own (chunk and position independence)."""
    import hamiltonzero_b200 as hz
    n, B = 64, 16384
    frame = S.frame_from_graph(S.erdos_renyi_exchange_graph(64, 0.1, seed=7), n)
    wf = S.synthetic_wavefunction(0, n)
    q = torch.as_tensor(S.corner_quaternions(np.random.default_rng(4).integers(0, 2, (B, n))),
                        device="cuda")
    cw = hz.CompiledWaveFunction(wf)
    dfr = hz.DeviceEnergyFrame(frame)
    tot, exc, cas, fld = hz.vmc_energy_custom_lap_compiled(cw, dfr, q, chunk_size=1024)
    spin = hz.local_spin(cw, dfr, q, chunk_size=1024)
    assert tot.shape == (B,) and spin.shape == (B, n, 3)
    assert torch.isfinite(torch.view_as_real(tot)).all() and torch.isfinite(torch.view_as_real(spin)).all()
    assert (exc - (tot - fld)).abs().max().item() <= 1e-3
    assert (cas == 0).all()
    lhs = -(dfr.field.to(torch.complex64)[None] * spin).sum((1, 2))
    # two evaluations by different passes (the energy pass and the value-and-gradient pass), each
    # held to 1e-4 of the sample scale: their difference to the sum of the two tolerances. The
    # largest samples of 16384 corner walkers sit next to nodes of the wavefunction (|field| up
    # to 180 against a typical 2), where both passes are least accurate.
    assert (lhs - fld).abs().max().item() <= 2e-4 * fld.abs().max().item()
    pick = torch.cat([q[:5], q[-3:]])
    alone = hz.vmc_energy_custom_lap_compiled(cw, dfr, pick)
    assert torch.equal(alone[0], torch.cat([tot[:5], tot[-3:]]))
    # and those eight against the oracle
    ref = W.local_energy(wf, frame, pick.cpu().numpy())
    _check_energy([a.cpu().numpy() for a in alone], ref, _term_scale(wf, frame, pick.cpu().numpy()),
                  "ER-64 full batch sample")


def test_field_channel_equals_h_dot_spin_at_scale(hz_lib):
    """Size-independent property on a larger batch: field = -sum_ic h_ic spin_ic."""
    import hamiltonzero_b200 as hz
    frame, wf = _problem(16, MID, p=0.3)
    q = torch.as_tensor(S.random_unit_quaternions(np.random.default_rng(5), (2048, 16)),
                        device="cuda")
    cw = hz.CompiledWaveFunction(wf)
    dfr = hz.DeviceEnergyFrame(frame)
    tot = hz.vmc_energy_custom_lap_compiled(cw, dfr, q, chunk_size=512)
    spin = hz.local_spin(cw, dfr, q, chunk_size=512)
    h = dfr.field.to(torch.complex64)
    lhs = -(h[None] * spin).sum((1, 2))
    assert (lhs - tot[3]).abs().max().item() <= 1e-4 * tot[3].abs().max().item()
    assert torch.isfinite(torch.view_as_real(tot[0])).all()


def test_operators_run_on_the_callers_stream(hz_lib):
    """The library only enqueues on the stream it is given (an XLA handler passes its own):
    the attention passes, log-psi and the energy pass issued on a side stream, behind a kernel
    that keeps that stream busy, return the same bits as on the default stream."""
    import hamiltonzero_b200 as hz
    frame, wf = _problem(32, MID)
    q = torch.as_tensor(S.random_unit_quaternions(np.random.default_rng(8), (40, 32)), device="cuda")
    cw = hz.CompiledWaveFunction(wf)
    dfr = hz.DeviceEnergyFrame(frame)
    gen = torch.Generator(device="cuda").manual_seed(3)
    a = [torch.randn(2, 64, 4, 32, device="cuda", generator=gen) for _ in range(3)]
    ref_la, ref_ph = cw(q)
    ref_e = hz.vmc_energy_custom_lap_compiled(cw, dfr, q)
    ref_o, ref_l = hz.mhsea_fwd(a[0], a[1], None, a[2], None)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    busy = torch.empty(1 << 26, device="cuda")
    with torch.cuda.stream(side):
        for _ in range(20):
            busy.normal_()                      # the side stream is busy when the calls arrive
        la, ph = cw(q)
        e = hz.vmc_energy_custom_lap_compiled(cw, dfr, q)
        o, l = hz.mhsea_fwd(a[0], a[1], None, a[2], None)
    side.synchronize()
    assert torch.equal(la, ref_la) and torch.equal(ph, ref_ph)
    for x, y in zip(e, ref_e):
        assert torch.equal(x, y)
    assert torch.equal(o, ref_o) and torch.equal(l, ref_l)


def test_walker_argument_checks(hz_lib):
    import hamiltonzero_b200 as hz
    frame, wf = _problem(4, SMALL)
    cw = hz.CompiledWaveFunction(wf)
    with pytest.raises(ValueError):
        cw(np.zeros((3, 8, 4), np.float32))
    bad = S.synthetic_wavefunction(0, 4, d_o=8, d_m=64, d_r=16, r_leaf=16, r_merge=16, r_ro=8)
    with pytest.raises(hz._lib.HzError):
        hz.CompiledWaveFunction(bad)(np.zeros((1, 4, 4), np.float32))


def test_device_wait_timeout_is_reported_and_cleared(hz_lib):
    """A bounded device wait that runs out is a status, not a hang: the self-test kernel waits
    about a millisecond on a barrier nothing arrives at, records the code and returns; the host
    reads HZ_ERR_TIMEOUT from the workspace's status word; the next operator call with that
    workspace clears it and returns correct values (no poisoned outputs, context intact)."""
    import ctypes
    import hamiltonzero_b200 as hz
    frame, wf = _problem(8, SMALL)
    cw = hz.CompiledWaveFunction(wf)
    q = torch.as_tensor(S.random_unit_quaternions(np.random.default_rng(2), (5, 8)), device="cuda")
    la0, ph0 = cw(q)
    ws = cw._workspace
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = ctypes.c_void_p(ws.data_ptr())
    assert hz_lib.hz_workspace_status(ptr, stream) == 0
    assert hz_lib.hz_selftest_wait_timeout(ptr, ws.numel(), stream) == 0
    assert hz_lib.hz_workspace_status(ptr, stream) == 9                 # HZ_ERR_TIMEOUT
    assert b"wait" in hz_lib.hz_status_string(9)
    # a forward pass that finds a non-zero status word poisons its outputs: keep the word set by
    # handing the next call a fresh status only through its own clearing
    la1, ph1 = cw(q)
    assert hz_lib.hz_workspace_status(ptr, stream) == 0
    assert torch.equal(la1, la0) and torch.equal(ph1, ph0)
    assert hz_lib.hz_selftest_wait_timeout(None, 256, stream) == 1
    assert hz_lib.hz_selftest_wait_timeout(ptr, 16, stream) == 7
