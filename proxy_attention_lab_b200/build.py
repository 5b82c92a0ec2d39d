"""Build libpal_b200.so (CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

Usage: ``python proxy_attention_lab_b200/build.py [--force] [--verbose]``.
The library is written next to this file so that it travels with the source tree.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libpal_b200.so"
OBJ_DIR = HERE / "build"
SOURCES = ["api.cu", "fill_kv_pages.cu", "decode.cu", "prefill_mma.cu", "prefill_tcgen05.cu", "prefill_tcgen05_d32_t16.cu", "prefill_tcgen05_d32_t32.cu", "prefill_tcgen05_d80_t16.cu", "prefill_tcgen05_d80_t32.cu", "prefill_tcgen05_d96_t16.cu", "prefill_tcgen05_d96_t32.cu", "prefill_tcgen05_d64_t16.cu", "prefill_tcgen05_d64_t32.cu", "prefill_tcgen05_d128_t16.cu",
           "prefill_tcgen05_d128_t32.cu", "prefill_tcgen05_d256_t16.cu", "prefill_tcgen05_d256_t32.cu", "prefill_tcgen05_pair_d128.cu", "prefill_tcgen05_pair_d256.cu", "decode_static.cu", "decode_exchange.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the library cannot be built")
    return exe


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    sources = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + sorted((HERE.parent / "include").glob("*.h"))
    OBJ_DIR.mkdir(exist_ok=True)
    hdr_digest = _digest(headers)
    nvcc = _nvcc()
    extra = ["-Xptxas", "-v"] if verbose else []
    extra += os.environ.get("PAL_EXTRA_NVCC_FLAGS", "").split()

    def compile_one(src: Path):
        obj = OBJ_DIR / (src.stem + ".o")
        stamp = OBJ_DIR / (src.stem + ".stamp")
        want = hashlib.sha256((hdr_digest + _digest([src]) + " ".join(NVCC_FLAGS + extra)).encode()).hexdigest()
        if not force and obj.exists() and stamp.exists() and stamp.read_text() == want:
            return obj, False, ""
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        stamp.write_text(want)
        return obj, True, r.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        results = list(ex.map(compile_one, sources))
    objs = [r[0] for r in results]
    if verbose:
        for r in results:
            if r[2]:
                print(r[2])
    if force or any(r[1] for r in results) or not LIB.exists():
        cmd = [nvcc, "-shared", "-o", str(LIB), *[str(o) for o in objs], "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    build_fastpath(force=force)
    return LIB


def fastpath_path() -> Path:
    import sysconfig

    return HERE / ("_pal_fast" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def build_fastpath(force: bool = False) -> Path:
    """Compile csrc/torch_fastpath.cpp (the C++ front of the Python operators) against this interpreter's torch and link it
    to libpal_b200.so; written next to the library.  Host code only: no GPU code lives in it."""
    import sysconfig

    import pybind11
    import torch
    from torch.utils import cpp_extension

    src = CSRC / "torch_fastpath.cpp"
    out = fastpath_path()
    OBJ_DIR.mkdir(exist_ok=True)
    stamp = OBJ_DIR / "torch_fastpath.stamp"
    want = hashlib.sha256((_digest([src, HERE.parent / "include" / "pal_b200.h"]) + torch.__version__ + sys.version).encode()).hexdigest()
    if not force and out.exists() and stamp.exists() and stamp.read_text() == want:
        return out
    cuda_home = os.environ.get("CUDA_HOME") or "/usr/local/cuda"
    includes = [*cpp_extension.include_paths(), pybind11.get_include(), sysconfig.get_paths()["include"],
                str(Path(cuda_home) / "include"), str(HERE.parent / "include")]
    torch_lib = cpp_extension.library_paths()[0]
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-DTORCH_EXTENSION_NAME=_pal_fast",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}",
           *[f"-I{i}" for i in includes], str(src), "-o", str(out),
           f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10", "-lc10_cuda",
           f"-L{HERE}", "-l:libpal_b200.so", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building the operator fast path failed:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(want)
    return out


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
