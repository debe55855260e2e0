"""In-tree build of the C-ABI libraries (nvcc, sm_100a only).

``python -m smoltts_b200.build`` compiles ``csrc/*.cu`` into ``smoltts_b200/_lib/``: ``libsmoltts_b200.so`` (DualAR decode
engine + Mimi decoder, target ``"core"``) and ``libsmoltts_b200_lm.so`` (hybrid language-model engine, target ``"lm"``).
A model loads -- and, when sources changed, builds -- only the library it runs on.  nvcc cross-compiles without a GPU, so this
also runs in the CPU-only build container; the .so is git-ignored but travels to the
GPU box with the repo snapshot.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "_lib")
LIB_PATH = os.path.join(LIB_DIR, "libsmoltts_b200.so")
STAMP = os.path.join(LIB_DIR, "build.stamp")
SOURCES = ["decode_kernel.cu", "ll2_kernel.cu", "capi.cu", "mimi_kernels.cu"]
HEADERS = ["common.cuh", "dev_model.h", "sampler.cuh", "umma.cuh", "tc_phases.cuh", "tmap_host.h", os.path.join("..", "..", "include", "smoltts_b200.h"),
           os.path.join("..", "..", "include", "smoltts_b200_mimi.h")]
LM_LIB_PATH = os.path.join(LIB_DIR, "libsmoltts_b200_lm.so")
# target -> (library, stamp, sources, headers)
TARGETS = {
    "core": (LIB_PATH, STAMP, SOURCES, HEADERS),
    "lm": (LM_LIB_PATH, os.path.join(LIB_DIR, "build_lm.stamp"), ["lm_kernels.cu"],
           ["common.cuh", "dev_model.h", "sampler.cuh", "umma.cuh", "tmap_host.h", "lm_mechanisms.cuh", "lm_sigmoid_linear.cuh",
            os.path.join("..", "..", "include", "smoltts_b200.h"), os.path.join("..", "..", "include", "smoltts_b200_lm.h")]),
}

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def _digest(target: str = "core") -> str:
    _, _, sources, headers = TARGETS[target]
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for name in sources + headers:
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    return h.hexdigest()


def is_current(target: str = "core") -> bool:
    lib, stamp = TARGETS[target][:2]
    if not (os.path.exists(lib) and os.path.exists(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == _digest(target)


def build(force: bool = False, verbose: bool = False, target: str = "core") -> str:
    """Compile one library if its sources changed; returns its path."""
    lib, stamp, sources, _ = TARGETS[target]
    if not force and is_current(target):
        return lib
    os.makedirs(LIB_DIR, exist_ok=True)
    extra = os.environ.get("SMOL_EXTRA_NVCC", "").split()
    tmp = f"{lib}.{os.getpid()}.tmp"          # concurrent first calls must never load a half-written library
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, *[os.path.join(CSRC, s) for s in sources], "-o", tmp, "-lcudart"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log = proc.stdout + proc.stderr
    with open(os.path.join(LIB_DIR, f"build_{target}.log"), "w") as f:
        f.write(" ".join(cmd) + "\n" + log)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{log[-6000:]}")
    os.replace(tmp, lib)
    if verbose:
        print(log)
    with open(stamp, "w") as f:
        f.write(_digest(target))
    return lib


if __name__ == "__main__":
    for tgt in TARGETS:
        if "--only" in sys.argv and sys.argv[sys.argv.index("--only") + 1] != tgt:
            continue
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, target=tgt))
