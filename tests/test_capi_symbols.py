"""The C-ABI library loads on a machine without a GPU and exports every symbol that
include/*.h declares (no compute calls here)."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    names = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names.update(re.findall(r"\b(hz_[a-z0-9_]+)\s*\(", text))
    return names


def test_every_declared_symbol_is_exported(hz_lib):
    declared = _declared_symbols()
    assert {"hz_mhsea_fwd", "hz_mhsea_jvp", "hz_mhsea_bwd"} <= declared
    for name in sorted(declared):
        assert hasattr(hz_lib, name), f"{name} declared in include/ but not exported"


def test_binding_table_covers_the_header(hz_lib):
    from hamiltonzero_b200 import _lib
    assert set(_lib.exported_signatures()) == _declared_symbols()


def test_status_strings_and_argument_checks(hz_lib):
    from hamiltonzero_b200._lib import AttnShape
    assert hz_lib.hz_status_string(0) == b"ok"
    assert hz_lib.hz_version() >= 100
    shape = AttnShape(1, 8, 1, 8, 0)
    null = ctypes.c_void_p(0)
    # argument validation happens before any CUDA call, so it is testable on CPU
    assert hz_lib.hz_mhsea_fwd(ctypes.byref(shape), null, null, null, null, null, null, null, null) == 1
    bad = AttnShape(1, 8, 1, 12, 0)
    assert hz_lib.hz_mhsea_fwd(ctypes.byref(bad), null, null, null, null, null, null, null, null) == 3
    big = AttnShape(1, 512, 1, 8, 0)
    assert hz_lib.hz_mhsea_fwd(ctypes.byref(big), null, null, null, null, null, null, null, null) == 3
    neg = AttnShape(0, 8, 1, 8, 0)
    assert hz_lib.hz_mhsea_fwd(ctypes.byref(neg), null, null, null, null, null, null, null, null) == 2


def test_walker_entry_points_check_arguments_before_any_cuda_call(hz_lib):
    """hz_logpsi_static, hz_logpsi and hz_workspace_status refuse null and malformed arguments
    with a status, on a machine without a GPU."""
    from hamiltonzero_b200._lib import Wavefunction
    null = ctypes.c_void_p(0)
    assert hz_lib.hz_logpsi_static(None, null, 1, null, null, null) == 1
    assert hz_lib.hz_workspace_status(null, null) == 1
    wf = Wavefunction(n_sites=6, d_o=8, d_m=64, d_r=32, r_leaf=8, r_merge=8, r_ro=8)
    assert hz_lib.hz_logpsi_static(ctypes.byref(wf), null, 1, null, null, null) == 2   # not a power of two
    wf = Wavefunction(n_sites=8, d_o=8, d_m=64, d_r=16, r_leaf=8, r_merge=8, r_ro=8)
    assert hz_lib.hz_logpsi_static(ctypes.byref(wf), null, 1, null, null, null) == 3   # group width
    assert hz_lib.hz_walker_workspace_bytes(ctypes.byref(wf), 1, 4) == -1
    assert b"wait" in hz_lib.hz_status_string(9) and b"device" in hz_lib.hz_status_string(10)
