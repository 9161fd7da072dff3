"""Measured HBM and NVLink figures of one GPU, for the placement planner.

    python -m exo_b200.utils.link_probe --gpu 0            # prints one JSON object

The probe (``ops/csrc/probe.cu``) times plain device and peer copies with CUDA events.  It runs in a process of
its own so that a node's controller never holds CUDA contexts on its peers; the result is cached per GPU UUID
under the cache directory (links do not change while the machine is up).  This is the part the reference's
telemetry plays for Thunderbolt / RDMA links (``src/exo/utils/info_gatherer/info_gatherer.py:444-462``).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
from pathlib import Path


def measure_here(gpu: int, peers: list[int], copy_mib: int = 256) -> dict:
    """Run the probes in this process on ``gpu`` (needs the kernel library and a CUDA device)."""
    import torch
    from ..ops import cuda as K
    lib = K.load()
    lib.exo_probe_hbm_copy.restype, lib.exo_probe_hbm_copy.argtypes = C.c_double, [C.c_size_t, C.c_int]
    lib.exo_probe_peer_copy.restype = C.c_int
    lib.exo_probe_peer_copy.argtypes = [C.c_int, C.c_size_t, C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double)]
    torch.cuda.set_device(gpu)
    out: dict = {"gpu": gpu, "hbm_gbps": round(lib.exo_probe_hbm_copy(1 << 30, 5), 1), "peers": {}}
    for j in peers:
        g, lat = C.c_double(0.0), C.c_double(0.0)
        rc = lib.exo_probe_peer_copy(j, copy_mib << 20, 5, C.byref(g), C.byref(lat))
        out["peers"][str(j)] = ({"gbps": round(g.value, 1), "latency_us": round(lat.value, 2)} if rc == 0 else {"error": rc})
    return out


def cache_path(uuid: str) -> Path:
    from ..shared import constants
    return constants.EXO_CACHE_HOME / f"link_probe_{uuid or 'gpu'}.json"


def measure(gpu: int, peers: list[int], uuid: str = "", timeout_s: float = 120.0) -> dict | None:
    """Cached result for this GPU, or a fresh one from a child process; ``None`` when the probe cannot run."""
    path = cache_path(uuid)
    try:
        cached = json.loads(path.read_text())
        if cached.get("gpu") == gpu and set(cached.get("peers", {})) >= {str(p) for p in peers}:
            return cached
    except (OSError, ValueError):
        pass
    try:
        r = subprocess.run([sys.executable, "-m", "exo_b200.utils.link_probe", "--gpu", str(gpu), "--peers",
                            ",".join(map(str, peers))], capture_output=True, text=True, timeout=timeout_s,
                           env={**os.environ, "PYTHONPATH": os.pathsep.join(sys.path)})
        res = json.loads(r.stdout.strip().splitlines()[-1])
    except (OSError, ValueError, IndexError, subprocess.TimeoutExpired):
        return None
    try:
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text(json.dumps(res))
    except OSError:
        pass
    return res


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpu", type=int, default=0)
    ap.add_argument("--peers", default="", help="comma-separated peer GPU indices (default: every other GPU)")
    a = ap.parse_args(argv)
    import torch
    n = torch.cuda.device_count()
    peers = [int(x) for x in a.peers.split(",") if x] if a.peers else [j for j in range(n) if j != a.gpu]
    print(json.dumps(measure_here(a.gpu, peers)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
