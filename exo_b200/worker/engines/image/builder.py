"""Image engine behind the runner: builder (rank group, model) and the serving loop.

Reference roles: ``MfluxBuilder`` / ``DistributedImageModel`` / ``generate_image``
(``src/exo/worker/engines/image/{builder,distributed_model,generate}.py``).  One generation runs
at a time; rank 0 announces each job (and, every denoising step, whether it was cancelled) to the
other ranks over a host-side broadcast, so every rank makes the same sequence of collective calls
without holding request state of its own.  Finished and partial images are encoded (PNG / JPEG /
WebP), base64'd and cut into ``EXO_MAX_CHUNK_SIZE`` pieces; the last piece of the last image of a
bench request carries the generation statistics.
"""
from __future__ import annotations

import base64
import datetime
import io
import os
import time
from collections import deque
from collections.abc import Iterable, Iterator
from typing import Any

import torch
import torch.distributed as dist

from ....api.types import ImageEditsTaskParams, ImageGenerationStats, ImageGenerationTaskParams
from ....shared import constants
from ....shared.base import Memory, TaskId
from ....shared.messages import GenerationTask, ImageEdits, ImageGeneration
from ....shared.wire import BoundInstance, CfgShardMetadata, ImageChunk, NvlinkInstance
from ..base import Builder, Cancelled, Engine, Finished, LoadProgress, StepItem
from .dit import Dit, DitConfig, steps_for_quality
from .pipeline import DiffusionRunner


def parse_size(size: str | None) -> tuple[int, int]:
    if not size or size == "auto":
        return 1024, 1024
    try:
        w, h = (int(x) for x in size.split("x"))
        if w > 0 and h > 0:
            return w, h
    except ValueError:
        pass
    raise ValueError(f"Invalid size format: '{size}'. Expected 'WIDTHxHEIGHT' (e.g., '1024x1024')")


def encode_image(rgb: torch.Tensor, fmt: str) -> bytes:
    from PIL import Image
    buf = io.BytesIO()
    Image.fromarray(rgb.cpu().numpy(), "RGB").save(buf, format={"jpg": "JPEG", "jpeg": "JPEG", "png": "PNG", "webp": "WEBP"}[fmt.lower()])
    return buf.getvalue()


def decode_image(data: bytes) -> torch.Tensor:
    import numpy as np
    from PIL import Image
    with Image.open(io.BytesIO(data)) as im:
        return torch.from_numpy(np.array(im.convert("RGB")))


def image_chunks(model_id: str, data: bytes, fmt: str, image_index: int, partial: tuple[int, int] | None,
                 stats: ImageGenerationStats | None) -> Iterator[ImageChunk]:
    b64 = base64.b64encode(data).decode("ascii")
    n = constants.EXO_MAX_CHUNK_SIZE
    pieces = [b64[i:i + n] for i in range(0, len(b64), n)] or [""]
    for i, piece in enumerate(pieces):
        last = i == len(pieces) - 1
        yield ImageChunk(model=model_id, data=piece, chunk_index=i, total_chunks=len(pieces), image_index=image_index,
                         is_partial=partial is not None, partial_index=None if partial is None else partial[0],
                         total_partials=None if partial is None else partial[1],
                         stats=stats if (last and partial is None) else None, format=fmt,
                         finish_reason="stop" if (last and partial is None) else None)


class ImageEngine(Engine):
    def __init__(self, runner: DiffusionRunner, model_id: str, rank: int, world: int, control_group=None):
        self.runner, self.model_id, self.rank, self.world, self.group = runner, model_id, rank, world, control_group
        self.queue: deque[GenerationTask] = deque()
        self.active: set[str] = set()              # follower: ids it was handed
        self.cancelled: set[str] = set()
        self.current: tuple[TaskId, Iterator[StepItem]] | None = None
        self.peak = 0

    # ---- host-side agreement between the ranks ----
    def _bcast(self, obj: Any = None) -> Any:
        if self.world == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=0, group=self.group)
        return box[0]

    def warmup(self) -> None:
        for _ in self.runner.generate("warmup", 64, 64, 2, 0):
            pass

    def submit(self, task: GenerationTask) -> None:
        if self.rank == 0:
            self.queue.append(task)
        else:
            self.active.add(str(task.task_id))

    def cancel(self, task_id: TaskId) -> None:
        self.cancelled.add(str(task_id))

    @property
    def has_work(self) -> bool:
        return bool(self.queue) or self.current is not None or bool(self.active)

    # ---- one job, on every rank ----
    def _job(self, task_id: str, p: ImageGenerationTaskParams | ImageEditsTaskParams, edit: bool) -> Iterator[StepItem]:
        width, height = parse_size(p.size)
        init = None
        if edit:
            init = decode_image(base64.b64decode(p.image_data))
            if p.size in (None, "auto"):
                height, width = init.shape[0], init.shape[1]
        adv = p.advanced_params
        table = getattr(self.runner.m, "default_steps", None)            # the model's own step counts per quality level
        steps = (adv.num_inference_steps if adv and adv.num_inference_steps else None) or \
            (table.get(p.quality or "medium", table["medium"]) if table else steps_for_quality(p.quality or "medium"))
        seed = adv.seed if adv and adv.seed is not None else 0
        guidance = adv.guidance if adv and getattr(adv, "guidance", None) is not None else None
        partials = p.partial_images if (p.stream and p.partial_images) else 0
        n_img = p.n or 1
        t0 = time.perf_counter()
        stopped = False

        def should_stop() -> bool:
            nonlocal stopped
            stopped = bool(self._bcast(task_id in self.cancelled if self.rank == 0 else None))
            return stopped
        for k in range(n_img):
            for kind, rgb, idx, total in self.runner.generate(
                    p.prompt, height, width, steps, seed + k, guidance=guidance, init_image=init,
                    strength=getattr(p, "image_strength", None) or 0.7, partial_images=partials, should_stop=should_stop):
                stats = None
                if kind == "final" and p.bench and k == n_img - 1:
                    el = time.perf_counter() - t0
                    if torch.cuda.is_available() and self.runner.m.device.type == "cuda":
                        self.peak = torch.cuda.max_memory_allocated(self.runner.m.device)
                    stats = ImageGenerationStats(seconds_per_step=el / max(1, steps * n_img), total_generation_time=el,
                                                 num_inference_steps=steps, num_images=n_img, image_width=width,
                                                 image_height=height, peak_memory_usage=Memory.from_bytes(self.peak))
                if self.rank == 0:
                    yield from image_chunks(self.model_id, encode_image(rgb, p.output_format or "png"), p.output_format or "png", k,
                                            (idx, total) if kind == "partial" else None, stats)
            if stopped:
                yield Cancelled()
                return
        yield Finished()

    def step(self) -> Iterable[tuple[TaskId, StepItem]]:
        if self.rank != 0:
            return self._follow()
        if self.current is None:
            if not self.queue:
                return []
            task = self.queue.popleft()
            tid = str(task.task_id)
            if tid in self.cancelled:
                return [(task.task_id, Cancelled())]
            edit = isinstance(task, ImageEdits)
            self._bcast(("start", tid, task.task_params.model_dump(), edit))
            self.current = (task.task_id, self._job(tid, task.task_params, edit))
        tid, gen = self.current
        out: list[tuple[TaskId, StepItem]] = []
        for item in gen:       # runs the whole job; chunks are handed over as they are produced
            out.append((tid, item))
            if isinstance(item, (Finished, Cancelled)):
                break
        self.current = None
        return out

    def _follow(self) -> list[tuple[TaskId, StepItem]]:
        msg = self._bcast()
        if msg is None or msg[0] == "stop":
            done = [(TaskId(t), Finished()) for t in self.active]
            self.active.clear()
            return done
        _, tid, params, edit = msg
        p = (ImageEditsTaskParams if edit else ImageGenerationTaskParams).model_validate(params)
        for _ in self._job(tid, p, edit):
            pass
        if tid in self.active:
            self.active.discard(tid)
            return [(TaskId(tid), Finished())]
        return []

    def close(self) -> None:
        if self.rank == 0 and self.world > 1:
            try:
                self._bcast(("stop",))
            except RuntimeError:
                pass


class ImageBuilder(Builder):
    def __init__(self, bound_instance: BoundInstance):
        super().__init__(bound_instance)
        sh = bound_instance.bound_shard
        self.card, self.rank, self.world = sh.model_card, sh.device_rank, sh.world_size
        want_cpu = os.environ.get("EXO_DEVICE", "").lower() == "cpu" or not torch.cuda.is_available()
        gpu = sh.gpu_index if sh.gpu_index is not None else int(os.environ.get("EXO_GPU_INDEX", "0"))
        self.device = torch.device("cpu") if want_cpu else torch.device("cuda", gpu)
        self.cfg_parallel = isinstance(sh, CfgShardMetadata)
        self.model: Dit | None = None
        self.control = None
        self.pipe_groups: list | None = None

    def connect(self) -> None:
        if self.world == 1:
            return
        inst = self.bound_instance.instance
        port = inst.rendezvous_port if isinstance(inst, NvlinkInstance) else getattr(inst, "ephemeral_port", 29556)
        backend = "gloo" if self.device.type == "cpu" else "nccl"
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        dist.init_process_group(backend, init_method=f"tcp://127.0.0.1:{port}", rank=self.rank, world_size=self.world,
                                timeout=datetime.timedelta(seconds=int(os.environ.get("EXO_GROUP_TIMEOUT_S", "120"))),
                                **({"device_id": self.device} if backend == "nccl" else {}))
        self.control = dist.new_group(backend="gloo") if backend == "nccl" else dist.group.WORLD
        half = self.world // 2
        groups = [list(range(0, half)), list(range(half, self.world))] if self.cfg_parallel else [list(range(self.world))]
        self.pipe_groups = [dist.new_group(g) for g in groups]

    def _stage(self, n_blocks: int) -> range:
        pipe_world = self.world // 2 if (self.cfg_parallel and self.world % 2 == 0) else self.world
        pipe_rank = self.rank % pipe_world
        per = -(-n_blocks // pipe_world)
        return range(min(n_blocks, pipe_rank * per), min(n_blocks, (pipe_rank + 1) * per))

    def load(self) -> Iterator[LoadProgress]:
        """FLUX.1 checkpoint folders (``transformer/``, ``vae/``, text encoders) load as ``FluxModel``, this stage's blocks
        only; any other card (or a card whose folder is not on disk) gets the seeded stand-in transformer."""
        from ..b200.builder import find_model_dir
        root = find_model_dir(str(self.card.model_id))
        if root is not None and (root / "transformer" / "config.json").exists() and "flux" in str(getattr(self.card, "family", "flux")).lower():
            from .flux import FluxConfig, FluxModel
            blocks = self._stage(FluxConfig.from_folder(root).n_blocks)
            yield LoadProgress(0, len(blocks))
            dtype = torch.float32 if self.device.type == "cpu" else torch.bfloat16
            self.model = FluxModel.from_folder(root, blocks=blocks, device=self.device, dtype=dtype)
            yield LoadProgress(len(blocks), len(blocks))
            return
        cfg = DitConfig.for_card(self.card.n_layers, self.card.hidden_size, self.card.uses_cfg)
        blocks = self._stage(cfg.n_blocks)
        yield LoadProgress(0, len(blocks))
        self.model = Dit(cfg, seed=0, blocks=blocks, device=self.device)
        yield LoadProgress(len(blocks), len(blocks))

    def build(self) -> Engine:
        assert self.model is not None
        sync = os.environ.get("EXO_IMAGE_SYNC_STEPS") or getattr(self.model, "num_sync_steps", 1)
        runner = DiffusionRunner(self.model, rank=self.rank, world=self.world, cfg_parallel=self.cfg_parallel,
                                 num_sync_steps=int(sync), pipe_groups=self.pipe_groups)
        runner.async_patches = os.environ.get("EXO_IMAGE_ASYNC_PATCHES", "1") != "0"     # 0: one step at a time (stages wait for its end)
        return ImageEngine(runner, str(self.card.model_id), self.rank, self.world, self.control)

    def close(self) -> None:
        if dist.is_available() and dist.is_initialized():
            try:
                dist.destroy_process_group()
            except RuntimeError:
                pass
