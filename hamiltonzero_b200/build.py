"""In-tree build of libhz_b200.so (CUDA, sm_100a only).

``python -m hamiltonzero_b200.build`` compiles every ``csrc/*.cu`` with nvcc and
links one shared library next to this file. The library is the product: the
Python modules of this package only marshal pointers into its C ABI
(``include/hz_b200.h``).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libhz_b200.so"
OBJ_DIR = PKG_DIR / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
] + os.environ.get("HZ_NVCC_EXTRA", "").split()      # e.g. -DHZ_MC_PROF for the in-kernel cycle counters


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libhz_b200.so cannot be built")
    return exe


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile csrc/*.cu into libhz_b200.so; a no-op when sources are unchanged."""
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + \
        sorted((PKG_DIR.parent / "include").glob("*.h"))
    stamp = OBJ_DIR / "stamp.txt"
    digest = _digest(sources + headers)
    if not force and LIB_PATH.exists() and stamp.exists() and stamp.read_text() == digest:
        return LIB_PATH
    OBJ_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            sys.stderr.write(res.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(compile_one, sources))
    cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *[str(o) for o in objs],
           "-gencode", "arch=compute_100a,code=sm_100a"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    stamp.write_text(digest)
    return LIB_PATH


FFI_LIB_PATH = PKG_DIR / "libhz_ffi.so"


def jaxlib_include_dir():
    """Directory that holds xla/ffi/api/ffi.h (shipped inside jaxlib), or None."""
    try:
        import jaxlib  # noqa: F401
    except Exception:
        return None
    inc = Path(jaxlib.__file__).resolve().parent / "include"
    return inc if (inc / "xla" / "ffi" / "api" / "ffi.h").exists() else None


def build_ffi(force: bool = False):
    """Compile csrc/hz_ffi.cc (the XLA FFI handlers around the C ABI) into libhz_ffi.so. Returns
    None, without failing, where jaxlib's headers are absent: the handlers are then simply not
    available, and everything else in the package works without them."""
    inc = jaxlib_include_dir()
    if inc is None:
        return None
    src = CSRC / "hz_ffi.cc"
    if not force and FFI_LIB_PATH.exists() and FFI_LIB_PATH.stat().st_mtime >= src.stat().st_mtime:
        return FFI_LIB_PATH
    build()
    cmd = [_nvcc(), "-x", "cu", "-std=c++17", "-O2", "-Xcompiler", "-fPIC", "-shared", "-I", str(inc),
           str(src), "-o", str(FFI_LIB_PATH), "-L", str(PKG_DIR), "-l:libhz_b200.so",
           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for hz_ffi.cc:\n{res.stdout}\n{res.stderr}")
    return FFI_LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_ffi(force="--force" in sys.argv) or "libhz_ffi.so: jaxlib headers not found, skipped")
