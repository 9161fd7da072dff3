"""In-tree native build: nvcc for the sm_100a kernel library, g++ for the host runtime.

``python -m exo_b200.build`` (or ``build_all()``) produces

* ``exo_b200/ops/_kernels.so``   – every CUDA kernel behind ``extern "C"`` launchers (ctypes);
* ``exo_b200/native/_exo_native.so`` – message bus, discovery, pidfile, NVML topology (pybind11).

Objects are cached by source hash under ``build/`` so a rebuild only recompiles what changed.
This stands where the reference has its Nix/uv packaging of prebuilt MLX wheels
(``python/parts.nix:23-41``); here the kernels are ours, so the build is part of the package.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
REPO = ROOT.parent
BUILD = REPO / "build"
NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fvisibility=hidden"]


def _hash(paths: list[Path], extra: str = "") -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} {cmd[-1]}")
    if r.stderr.strip() and os.environ.get("EXO_BUILD_VERBOSE"):
        sys.stderr.write(r.stderr)


def build_kernels(verbose: bool = False, force: bool = False) -> Path:
    src_dir = ROOT / "ops" / "csrc"
    out = ROOT / "ops" / "_kernels.so"
    srcs = sorted(src_dir.glob("*.cu"))
    hdrs = sorted(src_dir.glob("*.cuh")) + sorted(src_dir.glob("*.h"))
    hdr_hash = _hash(hdrs, " ".join(NVCC_FLAGS + ARCH))
    objdir = BUILD / "kernels"
    objdir.mkdir(parents=True, exist_ok=True)
    flags = list(NVCC_FLAGS)
    if verbose:
        flags += ["-Xptxas", "-v"]
    if os.environ.get("EXO_KERNEL_CHECKS") == "1":
        flags += ["-DEXO_KERNEL_CHECKS=1"]

    def compile_one(s: Path) -> tuple[Path, bool]:
        tag = _hash([s], hdr_hash + str(flags))
        o = objdir / f"{s.stem}.{tag}.o"
        if o.exists() and not force:
            return o, False
        for old in objdir.glob(f"{s.stem}.*.o"):
            old.unlink()
        cmd = [NVCC, *ARCH, *flags, "-I", str(src_dir), "-c", str(s), "-o", str(o)]
        if verbose:
            r = subprocess.run(cmd, capture_output=True, text=True)
            sys.stderr.write(r.stderr)
            if r.returncode:
                raise RuntimeError(f"nvcc failed on {s.name}")
        else:
            _run(cmd)
        return o, True

    with ThreadPoolExecutor(max_workers=min(8, len(srcs) or 1)) as ex:
        res = list(ex.map(compile_one, srcs))
    objs = [o for o, _ in res]
    if any(ch for _, ch in res) or not out.exists() or force:
        _run([NVCC, *ARCH, "-shared", "-o", str(out), *map(str, objs), "-lcudart"])
    return out


def build_native(force: bool = False) -> Path | None:
    src_dir = ROOT / "native" / "csrc"
    srcs = sorted(src_dir.glob("*.cc"))
    if not srcs:
        return None
    out = ROOT / "native" / "_exo_native.so"
    tag_file = BUILD / "native.tag"
    tag = _hash(srcs + sorted(src_dir.glob("*.h")))
    if out.exists() and tag_file.exists() and tag_file.read_text() == tag and not force:
        return out
    import pybind11
    BUILD.mkdir(exist_ok=True)
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", str(src_dir),
           "-I", "/usr/local/cuda/include"]
    _run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-pthread", *inc,
          *map(str, srcs), "-o", str(out), "-ldl"])
    tag_file.write_text(tag)
    return out


def build_all(verbose: bool = False, force: bool = False) -> None:
    build_kernels(verbose=verbose, force=force)
    build_native(force=force)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print("built:", ROOT / "ops" / "_kernels.so")
