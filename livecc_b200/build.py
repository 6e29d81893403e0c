"""Builds liblivecc_sm100a.so in-tree with nvcc for sm_100a (no torch dependency in the library).

`python -m livecc_b200.build` or `livecc_b200.build.build()`; nvcc cross-compiles without a GPU.
The .so is git-ignored but travels to the GPU box with the gpurun snapshot.
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
LIB_PATH = PKG_DIR / "liblivecc_sm100a.so"
OBJ_DIR = PKG_DIR / "build"

# A profile is the subset of csrc/*.cu one model family needs; it links into a library of its own, so that serving that
# family alone compiles nothing else. The full library (profile None) holds every source and exports a superset.
PROFILES = {
    "seq": ["cabi_core", "gemm_tcgen05", "sampling", "linear_any", "recurrent", "recurrent_chunked", "attn_local", "rowops", "rotary", "attn_latent",
            "hyper", "moe", "seq_model"],
}


def lib_path(profile: str | None = None) -> Path:
    return LIB_PATH if profile is None else PKG_DIR / f"liblivecc_{profile}_sm100a.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the sm_100a extension cannot be built")
    return nvcc


def _sources(profile: str | None = None) -> list[Path]:
    if profile is None:
        return sorted(CSRC.glob("*.cu"))
    return [CSRC / f"{name}.cu" for name in PROFILES[profile]]


def _fingerprint(src: Path) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    for hdr in sorted(list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list((PKG_DIR.parent / "include").glob("*.h"))):
        h.update(hdr.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False, profile: str | None = None) -> Path:
    """Compile csrc/*.cu (all of them, or one profile's subset) to objects cached by content hash and link the library."""
    nvcc = _nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    out_path = lib_path(profile)
    objs: list[Path] = []
    jobs = []
    for src in _sources(profile):
        obj = OBJ_DIR / (src.stem + ".o")
        stamp = OBJ_DIR / (src.stem + ".sha")
        fp = _fingerprint(src)
        objs.append(obj)
        if not force and obj.exists() and stamp.exists() and stamp.read_text() == fp:
            continue
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
        jobs.append((cmd, stamp, fp))

    def run(job):
        cmd, stamp, fp = job
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        if ptxas_info or verbose:
            sys.stderr.write(r.stderr)
        stamp.write_text(fp)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(run, jobs))
    stale = not out_path.exists() or any(o.stat().st_mtime > out_path.stat().st_mtime for o in objs)
    if jobs or stale or force:
        tmp = out_path.with_suffix(f".tmp{os.getpid()}")
        cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, out_path)
    return out_path


if __name__ == "__main__":
    prof = next((a.split("=", 1)[1] for a in sys.argv if a.startswith("--profile=")), None)
    p = build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv, profile=prof)
    print(p)
