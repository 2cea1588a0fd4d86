"""In-tree build of the native library (CUDA kernels for sm_100a + the C++ step executor).

`python -m saber_engine_b200.build` compiles every source under `csrc/` with nvcc / g++ and links
`_lib/libsaber_b200.so` next to the package.  nvcc cross-compiles for sm_100a without a GPU.  The
library has a plain C ABI and is loaded with ctypes (`saber_engine_b200.ops.native`), so it does not
depend on the torch C++ ABI and builds in seconds.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OUT_DIR = ROOT / "_lib"
OBJ_DIR = OUT_DIR / "obj"
LIB_NAME = "libsaber_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-march=x86-64-v3"]


def cuda_home() -> Path:
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and Path(cand, "bin", "nvcc").exists():
            return Path(cand)
    nvcc = shutil.which("nvcc")
    if nvcc:
        return Path(nvcc).resolve().parent.parent
    raise RuntimeError("nvcc not found: set CUDA_HOME")


def sources() -> list[Path]:
    out = []
    for pat in ("**/*.cu", "**/*.cpp"):
        out += sorted(CSRC.glob(pat))
    return out


def _digest(src: Path, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.glob("**/*.h")) + sorted(CSRC.glob("**/*.cuh")):
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _compile(src: Path, verbose: bool) -> tuple[Path, str]:
    home = cuda_home()
    obj = OBJ_DIR / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
    stamp = obj.with_suffix(".sha")
    if src.suffix == ".cu":
        cmd = [str(home / "bin" / "nvcc"), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    else:
        cmd = ["g++", *CXX_FLAGS, f"-I{home / 'include'}", "-c", str(src), "-o", str(obj)]
    dg = _digest(src, cmd)
    if obj.exists() and stamp.exists() and stamp.read_text() == dg:
        return obj, ""
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    stamp.write_text(dg)
    return obj, (res.stdout + res.stderr) if verbose else ""


def build(verbose: bool = False) -> Path:
    """Compile (incrementally) and link the native library; returns its path."""
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    srcs = sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, verbose), srcs))
    objs = [str(o) for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    home = cuda_home()
    lib = OUT_DIR / LIB_NAME
    newest = max(Path(o).stat().st_mtime for o in objs)
    if lib.exists() and lib.stat().st_mtime >= newest:
        return lib
    cmd = ["g++", "-shared", "-o", str(lib), *objs, f"-L{home / 'lib64'}", "-lcudart_static",
           "-lrt", "-lpthread", "-ldl"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    return lib


def lib_path() -> Path:
    return OUT_DIR / LIB_NAME


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
