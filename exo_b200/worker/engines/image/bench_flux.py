"""Time FLUX.1 denoising steps on one GPU: ``python -m exo_b200.worker.engines.image.bench_flux --size 1024 --steps 4``.

Full-size architecture (19 joint + 38 single blocks, 3072 wide, 11.9 B parameters) with weights drawn from a seed in
bf16 and pseudo text features of the real shapes (512 T5 positions); times whole denoising steps with CUDA events after
warm-up steps, and the VAE decode once.  Prints one JSON line."""
from __future__ import annotations

import argparse
import json

import torch

from .flux import FluxConfig, FluxModel, transformer_shapes


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--schnell", action="store_true")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    cfg = FluxConfig(guidance_embeds=not a.schnell, dynamic_shift=not a.schnell, text_len=256 if a.schnell else 512)
    m = FluxModel.random(cfg, device=dev, dtype=torch.bfloat16)
    gh, gw = m.grid(a.size, a.size)
    lat = torch.randn(cfg.latent_channels, gh * cfg.patch, gw * cfg.patch, device=dev)
    txt, pooled = m.encode_text("a lighthouse on a cliff at dusk, oil painting")
    ts = m.schedule(a.steps + a.warmup, gh * gw)
    for i in range(a.warmup):
        lat = lat + (ts[i + 1] - ts[i]) * m.velocity(lat, ts[i], txt, pooled)
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    torch.cuda.synchronize()
    e0.record()
    for i in range(a.warmup, a.warmup + a.steps):
        lat = lat + (ts[i + 1] - ts[i]) * m.velocity(lat, ts[i], txt, pooled)
    e1.record()
    img = m.decode(lat)
    e2.record()
    torch.cuda.synchronize()
    step_ms = e0.elapsed_time(e1) / a.steps
    params = sum(torch.Size(s).numel() for s in transformer_shapes(cfg).values())
    tokens = gh * gw + cfg.text_len
    H = cfg.hidden
    flops = 2.0 * (params - 2 * 19 * 6 * H * H - 38 * 3 * H * H) * tokens + 4.0 * cfg.n_blocks * tokens * tokens * H   # GEMMs + attention
    print(json.dumps({"metric": "flux_seconds_per_step", "value": step_ms / 1e3, "size": a.size, "steps": a.steps, "warmup": a.warmup,
                      "tokens": tokens, "params": params, "tflops": flops / step_ms / 1e9, "vae_decode_ms": e1.elapsed_time(e2),
                      "image": list(img.shape), "dtype": "bf16", "data": "synthetic",
                      "peak_gb": torch.cuda.max_memory_allocated(dev) / 2 ** 30}))


if __name__ == "__main__":
    main()
