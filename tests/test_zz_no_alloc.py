"""hz_logpsi_static: the log-psi entry point that allocates nothing (its scratch is a fixed
array inside the library, for hosts that cannot pass a workspace and must not let the
library call cudaMalloc). Called through the C ABI, twice in a row, and compared with
hz_logpsi on the same walkers. Collected last so that a run that stops at the first
failure has already run every other test; it also passes alone in a fresh process."""
import ctypes

import numpy as np
import pytest
import torch

from hamiltonzero_b200 import systems as S

pytestmark = pytest.mark.gpu

DIMS = dict(d_o=16, d_m=256, d_r=32, r_leaf=32, r_merge=64, r_ro=16)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def test_static_scratch_entry_point_matches_workspace_entry_point(hz_lib):
    import hamiltonzero_b200 as hz
    n, walkers = 16, 4096          # enough walkers that the 32 MiB array forces several chunks
    wf = S.synthetic_wavefunction(3, n, n_real=13, **DIMS)
    cw = hz.CompiledWaveFunction(wf)
    rng = np.random.default_rng(9)
    assert hz_lib.hz_static_scratch_bytes() == 32 << 20
    one = hz_lib.hz_walker_workspace_bytes(ctypes.byref(cw.c), 0, 1)
    assert 0 < one * walkers and one * walkers > hz_lib.hz_static_scratch_bytes()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):          # the second call finds the first call's leftovers in the array
        q = torch.as_tensor(S.random_unit_quaternions(rng, (walkers, n)), device="cuda")
        ref_la, ref_ph = cw(q)                                     # hz_logpsi, torch workspace
        la = torch.full((walkers,), float("nan"), device="cuda")
        ph = torch.full((walkers,), float("nan"), device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        # free bytes as the driver counts them: unlike torch's own counter this also sees a
        # cudaMalloc made inside the library. The first call may still load kernel code, so
        # the driver-level comparison is made on the second one.
        free_before, _ = torch.cuda.mem_get_info()
        st = hz_lib.hz_logpsi_static(ctypes.byref(cw.c), _ptr(q), walkers, _ptr(la), _ptr(ph),
                                     stream)
        assert st == 0, hz_lib.hz_status_string(st)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert torch.cuda.memory_allocated() == before
        if call == 1:
            assert free_after >= free_before, "the call took device memory from the driver"
        assert torch.isfinite(la).all() and torch.isfinite(ph).all()
        # same tolerance as the log-psi parity tests: 1e-5 relative, 2e-5 rad
        assert (la - ref_la).abs().max().item() <= 1e-5 * ref_la.abs().max().item() + 1e-5
        d = torch.angle(torch.exp(1j * (ph - ref_ph).to(torch.complex64))).abs().max().item()
        assert d <= 2e-5


def test_static_entry_point_refuses_what_does_not_fit_or_would_allocate(hz_lib):
    import hamiltonzero_b200 as hz
    from hamiltonzero_b200 import _lib
    null = ctypes.c_void_p(0)
    # one walker of this (wide) wavefunction needs more than 32 MiB of scratch
    wide = S.synthetic_wavefunction(0, 256, d_o=8, d_m=8192, d_r=32, r_leaf=8, r_merge=8, r_ro=8)
    cw = hz.CompiledWaveFunction(wide)
    q = torch.zeros(1, 256, 4, device="cuda")
    out = torch.zeros(2, device="cuda")
    st = hz_lib.hz_logpsi_static(ctypes.byref(cw.c), _ptr(q), 1, _ptr(out), _ptr(out[1:]), null)
    assert st == 8 and b"32 MiB" in hz_lib.hz_status_string(st)
    small = hz.CompiledWaveFunction(S.synthetic_wavefunction(0, 4, **DIMS))
    _lib.stage_timing_enable(True)
    try:
        q4 = torch.zeros(1, 4, 4, device="cuda")
        st = hz_lib.hz_logpsi_static(ctypes.byref(small.c), _ptr(q4), 1, _ptr(out), _ptr(out[1:]),
                                     null)
        assert st == 3
    finally:
        _lib.stage_timing_enable(False)
    # buffers on the host side of the fence: a null output is refused before any launch
    st = hz_lib.hz_logpsi_static(ctypes.byref(small.c), _ptr(q4), 1, null, _ptr(out[1:]), null)
    assert st == 1
    if torch.cuda.device_count() > 1:
        # the array of the current device is used: buffers of another device are refused
        other = torch.zeros(1, 4, 4, device="cuda:1")
        st = hz_lib.hz_logpsi_static(ctypes.byref(small.c), _ptr(other), 1, _ptr(out),
                                     _ptr(out[1:]), null)
        assert st == 10
