"""ctypes binding of libhz_b200.so. There is no fallback: a missing library or a
non-zero status raises."""
from __future__ import annotations

import ctypes
from ctypes import (POINTER, Structure, c_char_p, c_double, c_float, c_int, c_int32,
                    c_longlong, c_uint64, c_void_p)
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libhz_b200.so"


class HzError(RuntimeError):
    def __init__(self, status: int, where: str, text: str, cuda_error: int = 0):
        self.status = status
        self.cuda_error = cuda_error
        extra = f" (cudaError {cuda_error})" if cuda_error else ""
        super().__init__(f"{where}: status {status}: {text}{extra}")


class AttnShape(Structure):
    _fields_ = [("B", c_int32), ("N", c_int32), ("H", c_int32), ("D", c_int32),
                ("mask_mode", c_int32)]


class Wavefunction(Structure):
    _fields_ = [("n_sites", c_int32), ("d_o", c_int32), ("d_m", c_int32), ("d_r", c_int32),
                ("r_leaf", c_int32), ("r_merge", c_int32), ("r_ro", c_int32),
                ("merge_eps", c_float),
                ("q_weight", c_void_p), ("leaf_V", c_void_p), ("leaf_U", c_void_p),
                ("leaf_h", c_void_p), ("merge_T", c_void_p), ("merge_V", c_void_p),
                ("merge_U", c_void_p), ("merge_h", c_void_p), ("opcodes", c_void_p),
                ("readout_V", c_void_p), ("readout_U", c_void_p), ("readout_h", c_void_p)]


class WavefunctionGrads(Structure):
    _fields_ = [("q_weight", c_void_p), ("leaf_V", c_void_p), ("leaf_U", c_void_p),
                ("leaf_h", c_void_p), ("merge_T", c_void_p), ("merge_V", c_void_p),
                ("merge_U", c_void_p), ("merge_h", c_void_p), ("readout_V", c_void_p),
                ("readout_U", c_void_p), ("readout_h", c_void_p)]


class KfacFactors(Structure):
    NAMES = ("q_in", "q_out", "leaf_V_in", "leaf_V_out", "leaf_U_in", "leaf_U_out", "leaf_h_diag",
             "merge_V_in", "merge_V_out", "merge_U_in", "merge_U_out", "merge_h_diag",
             "readout_V_in", "readout_V_out", "readout_U_in", "readout_U_out", "readout_h_diag",
             "merge_T_left", "merge_T_right", "merge_T_stats")
    _fields_ = [("leaf_mask", c_void_p)] + [(n, c_void_p) for n in NAMES]


class EnergyFrame(Structure):
    _fields_ = [("J_eff", c_void_p), ("one_body_field", c_void_p), ("radial_const", c_float)]


class McmcState(Structure):
    _fields_ = [("n_walkers", c_int32), ("n_replicas", c_int32), ("n_sites", c_int32),
                ("step", c_int32), ("seed", c_uint64), ("offset", c_uint64),
                ("q", c_void_p), ("log_p", c_void_p), ("drift", c_void_p), ("beta", c_void_p),
                ("sigma", c_void_p), ("mask", c_void_p), ("m", c_void_p),
                ("n_local_accept", c_void_p), ("n_swap_accept", c_void_p), ("n_swap", c_void_p),
                ("n_haar_accept", c_void_p)]


class McmcNoise(Structure):
    _fields_ = [("haar_scores", c_void_p), ("haar_raw", c_void_p), ("haar_logu", c_void_p),
                ("local_noise", c_void_p), ("local_logu", c_void_p), ("swap_logu", c_void_p)]


_F = c_void_p  # device pointers travel as integers

_SIGNATURES = {
    "hz_status_string": (c_char_p, [c_int]),
    "hz_last_cuda_error": (c_int, []),
    "hz_version": (c_int, []),
    "hz_workspace_status": (c_int, [_F, c_void_p]),
    "hz_selftest_wait_timeout": (c_int, [_F, c_longlong, c_void_p]),
    "hz_stage_count": (c_int, []),
    "hz_stage_name": (c_char_p, [c_int]),
    "hz_stage_timing_enable": (c_int, [c_int]),
    "hz_stage_timing_read": (c_int, [POINTER(c_double), POINTER(c_double), POINTER(c_longlong),
                                     c_int, c_int]),
    "hz_mhsea_fwd": (c_int, [POINTER(AttnShape), _F, _F, _F, _F, _F, _F, _F, c_void_p]),
    "hz_mhsea_jvp": (c_int, [POINTER(AttnShape)] + [_F] * 12 + [c_void_p]),
    "hz_mhsea_bwd": (c_int, [POINTER(AttnShape)] + [_F] * 12 + [c_void_p]),
    "hz_mha_rect_workspace_bytes": (c_longlong, [c_int, c_int, c_int, c_int, c_int]),
    "hz_mha_rect_fwd": (c_int, [c_int, c_int, c_int, c_int, c_int, _F, _F, _F, _F, _F, _F, _F, c_longlong,
                                c_void_p]),
    "hz_fwl2_panel": (c_int, [_F, _F, _F, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "hz_walker_workspace_bytes": (c_longlong, [POINTER(Wavefunction), c_int, c_longlong]),
    "hz_logpsi": (c_int, [POINTER(Wavefunction), _F, c_longlong, _F, _F, _F, c_longlong,
                          c_void_p]),
    "hz_logpsi_grad": (c_int, [POINTER(Wavefunction), _F, c_longlong, _F, _F, _F, _F, c_longlong,
                               c_void_p]),
    "hz_vjp_workspace_bytes": (c_longlong, [POINTER(Wavefunction), c_longlong, c_int]),
    "hz_logpsi_vjp": (c_int, [POINTER(Wavefunction), _F, c_longlong, _F, _F,
                              POINTER(WavefunctionGrads), POINTER(KfacFactors), _F, _F, _F, _F,
                              c_longlong, c_void_p]),
    "hz_mcmc_workspace_bytes": (c_longlong, [POINTER(Wavefunction), c_int, c_int, c_longlong]),
    "hz_mcmc_sweep": (c_int, [POINTER(Wavefunction), POINTER(McmcState), c_int,
                              POINTER(McmcNoise), _F, _F, c_longlong, c_void_p]),
    "hz_static_scratch_bytes": (c_longlong, []),
    "hz_logpsi_static": (c_int, [POINTER(Wavefunction), _F, c_longlong, _F, _F, c_void_p]),
    "hz_local_energy": (c_int, [POINTER(Wavefunction), POINTER(EnergyFrame), _F, c_longlong,
                                _F, _F, _F, _F, _F, c_longlong, c_void_p]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library (once). Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m hamiltonzero_b200.build`. "
            "There is no CPU or PyTorch fallback for these operators.")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status: int, where: str) -> None:
    if status != 0:
        lib = load()
        raise HzError(status, where, lib.hz_status_string(status).decode(),
                      lib.hz_last_cuda_error() if status == 5 else 0)


def stage_timing_enable(on: bool) -> None:
    check(load().hz_stage_timing_enable(1 if on else 0), "hz_stage_timing_enable")


def stage_timing_read(reset: bool = True):
    """``{stage name: (milliseconds, algorithmic fp32 FLOPs, launches)}`` accumulated since the
    last reset; waits for the recorded events."""
    lib = load()
    n = lib.hz_stage_count()
    ms, fl, ln = (c_double * n)(), (c_double * n)(), (c_longlong * n)()
    check(lib.hz_stage_timing_read(ms, fl, ln, n, 1 if reset else 0), "hz_stage_timing_read")
    return {lib.hz_stage_name(i).decode(): (ms[i], fl[i], ln[i]) for i in range(n)}


def exported_signatures():
    return dict(_SIGNATURES)
