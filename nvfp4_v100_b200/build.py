"""Build recipe for the C-ABI library (``libnvfp4_b200.so``).

Compiles every ``csrc/*.cu`` for sm_100a with nvcc (cross-compiles without a GPU), links them into
one shared library next to this file, and recreates the ``kernels/<name>.dll`` aliases the
reference's loader expects (``ctypes.CDLL(os.path.join(KDIR, "nvfp4_gemv.dll"))``,
reference: pipeline/_qwen38_infer.py:37-38,61-62,430,593,862; experiments/_qwen38_p9_fuse.py:34).
``dlopen`` ignores file extensions, so the aliases are symlinks to the one library.

Run as ``python -m nvfp4_v100_b200.build`` or call :func:`build`.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_NAME = "libnvfp4_b200.so"
LIB_PATH = os.path.join(PKG_DIR, LIB_NAME)
KDIR = os.path.join(PKG_DIR, "kernels")
OBJ_DIR = os.path.join(PKG_DIR, "build")

# names under which the reference loads its per-kernel DLLs
DLL_ALIASES = [
    "nvfp4_gemv.dll",
    "nvfp4_cuda_v5.dll",
    "nvfp4_rmsnorm.dll",
    "nvfp4_attn_decode.dll",
    "nvfp4_rope_silu.dll",
    "nvfp4_dn_fused.dll",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=default",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the NVFP4 kernels cannot be built")
    return exe


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stamp(paths: list[str]) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.encode())
        with open(p, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def make_aliases() -> None:
    os.makedirs(KDIR, exist_ok=True)
    for name in DLL_ALIASES:
        link = os.path.join(KDIR, name)
        if os.path.islink(link) or os.path.exists(link):
            os.remove(link)
        os.symlink(os.path.join("..", LIB_NAME), link)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile and link the library if sources changed; return its path."""
    srcs = sources()
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    stamp = _stamp(srcs + hdrs)
    stamp_file = os.path.join(OBJ_DIR, "stamp.txt")
    if (not force and os.path.exists(LIB_PATH) and os.path.exists(stamp_file)
            and open(stamp_file).read().strip() == stamp):
        make_aliases()
        return LIB_PATH
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in srcs:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", os.path.join(os.path.dirname(PKG_DIR), "include"),
               "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
        objs.append(obj)
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stdout.write(out.decode(errors="replace"))
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    link = [nvcc, "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    if r.returncode != 0:
        sys.stdout.write(r.stdout.decode(errors="replace"))
        raise RuntimeError("link failed")
    with open(stamp_file, "w") as fh:
        fh.write(stamp)
    make_aliases()
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
