"""Time FLUX.1 denoising steps: ``python -m exo_b200.worker.engines.image.bench_flux --size 1024 --steps 4`` on one GPU, or under
``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m exo_b200.worker.engines.image.bench_flux`` with
the blocks split into N pipeline stages (one whole-image step that fills the key / value caches, then patch steps in which
every stage works on a different row patch).

Full-size architecture (19 joint + 38 single blocks, 3072 wide, 11.9 B parameters) with weights drawn from a seed in
bf16 and pseudo text features of the real shapes (512 T5 positions); times whole denoising steps with CUDA events after
warm-up steps (the maximum over ranks), and the VAE decode once.  Prints one JSON line.  ``--tiny --device cpu`` runs
the same code on a toy configuration (gloo ranks) to check the schedule without a GPU."""
from __future__ import annotations

import argparse
import datetime
import json
import os
import time

import torch
import torch.distributed as dist

from .flux import FluxConfig, FluxModel, transformer_shapes
from .pipeline import DiffusionRunner


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--schnell", action="store_true")
    ap.add_argument("--tiny", action="store_true", help="a toy configuration (schedule checks)")
    ap.add_argument("--device", default="cuda")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    cuda = a.device == "cuda"
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo", timeout=datetime.timedelta(seconds=60), **({"device_id": dev} if cuda else {}))
    if a.tiny:
        cfg = FluxConfig(n_joint=2, n_single=2, n_heads=2, head_dim=32, text_dim=48, pooled_dim=24, axes_dims=(8, 12, 12), text_len=16,
                         vae_channels=(32, 64), vae_groups=8, vae_scale=2)
    else:
        cfg = FluxConfig(guidance_embeds=not a.schnell, dynamic_shift=not a.schnell, text_len=256 if a.schnell else 512)
    per = -(-cfg.n_blocks // world)
    blocks = range(min(cfg.n_blocks, rank * per), min(cfg.n_blocks, (rank + 1) * per))
    m = FluxModel.random(cfg, blocks=blocks, device=dev, dtype=torch.bfloat16 if cuda else torch.float32)
    gh, gw = m.grid(a.size, a.size)
    tokens = gh * gw + cfg.text_len
    n_steps = a.steps + a.warmup
    sync = (lambda: torch.cuda.synchronize(dev)) if cuda else (lambda: None)
    if world == 1:
        lat = torch.randn(cfg.latent_channels, gh * cfg.patch, gw * cfg.patch, device=dev)
        txt, pooled = m.encode_text("a lighthouse on a cliff at dusk, oil painting")
        ts = m.schedule(n_steps, gh * gw)
        for i in range(a.warmup):
            lat = lat + (ts[i + 1] - ts[i]) * m.velocity(lat, ts[i], txt, pooled)
        sync()
        t0 = time.perf_counter()
        for i in range(a.warmup, n_steps):
            lat = lat + (ts[i + 1] - ts[i]) * m.velocity(lat, ts[i], txt, pooled)
        sync()
        step_s = (time.perf_counter() - t0) / a.steps
        t1 = time.perf_counter()
        img = m.decode(lat)
        sync()
        decode_ms, hops = 1e3 * (time.perf_counter() - t1), 0
    else:
        # the serving schedule: the runner's generator, timed from the end of the warm-up steps (one whole-image step + patch steps)
        groups = [dist.new_group(list(range(world)))]
        r = DiffusionRunner(m, rank=rank, world=world, num_sync_steps=1, pipe_groups=groups)
        marks: list[float] = []
        real_decode = m.decode

        def stamped_decode(lat: torch.Tensor) -> torch.Tensor:           # the previews mark step boundaries; only the last is decoded
            sync()
            marks.append(time.perf_counter())
            return real_decode(lat) if len(marks) == n_steps else torch.zeros(1, 1, 3, dtype=torch.uint8)
        m.decode = stamped_decode
        # previews after every step from the end of the warm-up on: partial_images = steps, `every` = 1
        t_begin = time.perf_counter()
        out = None
        for kind, rgb, _i, _n in r.generate("a lighthouse on a cliff at dusk, oil painting", a.size, a.size, n_steps, 0,
                                            partial_images=n_steps - 1):
            out = rgb
        sync()
        t_end = time.perf_counter()
        # marks: one per preview (after steps 1 .. n_steps-1) and one for the final image
        stamps = [t_begin] + marks
        step_s = (stamps[n_steps] - stamps[a.warmup]) / a.steps if len(stamps) > n_steps else (t_end - t_begin) / n_steps
        worst = torch.tensor([step_s], dtype=torch.float64, device=dev if cuda else "cpu")
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        step_s = float(worst)
        img, decode_ms, hops = out, 1e3 * (t_end - marks[-1]) if marks else 0.0, r.n_patch_hops
    if rank == 0:
        params = sum(torch.Size(s).numel() for s in transformer_shapes(cfg).values())
        H = cfg.hidden
        flops = 2.0 * (params - 2 * cfg.n_joint * 6 * H * H - cfg.n_single * 3 * H * H) * tokens + 4.0 * cfg.n_blocks * tokens * tokens * H
        print(json.dumps({"metric": "flux_seconds_per_step", "value": step_s, "n_gpus": world, "size": a.size, "steps": a.steps, "warmup": a.warmup,
                          "tokens": tokens, "params": params, "tflops": flops / step_s / 1e12, "vae_decode_ms": decode_ms, "patch_hops": hops,
                          "image": list(img.shape), "dtype": "bf16" if cuda else "fp32", "data": "synthetic",
                          "schedule": "single rank" if world == 1 else f"{world} pipeline stages, 1 whole-image step then row patches",
                          "peak_gb": torch.cuda.max_memory_allocated(dev) / 2 ** 30 if cuda else 0.0}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
