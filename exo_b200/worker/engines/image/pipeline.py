"""Distributed denoising schedules: pipeline stages, CFG-parallel groups, PipeFusion patches.

Mirrors the roles of the reference's ``DiffusionRunner`` (``src/exo/worker/engines/image/
pipeline/runner.py``): the transformer blocks are split into contiguous ranges over the ranks of a
pipeline group; with classifier-free guidance and an even world the ranks form two mirrored
groups, one denoising the prompt and one the empty prompt, whose last stages swap their
predictions every step (C10); after ``num_sync_steps`` synchronous steps that fill every block's
image K/V cache, the latent is cut into as many row patches as there are stages and the patches
flow through the pipeline back to back, each attending to fresh K/V of its own rows and to the
previous step's K/V of the others (PipeFusion), so all stages are busy at once: the last stage applies the Euler update to
a patch's rows as soon as it has that patch's prediction and hands the updated rows straight back to the first stage, which
starts the next step's patch with them — no stage waits for the end of a step (``_patch_pipeline``; the step-by-step form
``_predict_patches`` remains for models that make two passes per step on one group, and as the oracle of the tests).  Rank layout:
``rank = cfg_rank * pipe_world + pipe_rank``.  Every rank draws the same noise from the seed and
ends every step holding the same latent.
"""
from __future__ import annotations

from collections.abc import Callable, Iterator

import torch
import torch.distributed as dist

from .dit import Dit, timesteps


class DiffusionRunner:
    def __init__(self, model: Dit, *, rank: int = 0, world: int = 1, cfg_parallel: bool = False, num_sync_steps: int = 1,
                 pipe_groups: list | None = None):
        self.m, self.rank, self.world = model, rank, world
        self.cfg_parallel = cfg_parallel and world % 2 == 0 and model.cfg.uses_cfg
        self.pipe_world = world // 2 if self.cfg_parallel else world
        self.cfg_rank, self.pipe_rank = divmod(rank, self.pipe_world)
        self.base = self.cfg_rank * self.pipe_world               # first rank of this pipeline group
        self.group = None if pipe_groups is None else pipe_groups[self.cfg_rank]
        self.num_sync_steps = num_sync_steps
        self.first, self.last = self.pipe_rank == 0, self.pipe_rank == self.pipe_world - 1
        self.n_exchanges = self.n_patch_hops = 0
        self.async_patches = True          # patches flow across step boundaries (False: one step at a time, stages wait for its end)
        self.cancel_every = 4              # in that mode the ranks agree on cancellation every so many steps (it is a host-side sync)

    # ---- p2p helpers (blocking; tensors are tiny next to the compute) ----
    def _send(self, t: torch.Tensor, dst: int) -> None:
        dist.send(t.contiguous().cpu() if t.device.type == "cpu" else t.contiguous(), dst)

    def _recv(self, like: torch.Tensor, src: int) -> torch.Tensor:
        buf = torch.empty_like(like)
        dist.recv(buf, src)
        return buf

    # ---- one prediction of this pipeline group ----
    def _predict_sync(self, lat, t, txt0, pooled, caches) -> torch.Tensor:
        """Whole-image pass through the stages in order; fills the K/V caches.  Returns v on every stage."""
        m = self.m
        gh, gw = lat.shape[1] // m.cfg.patch, lat.shape[2] // m.cfg.patch
        vec = m.time_vec(t, pooled)
        if self.first:
            txt, img = txt0, m.embed_tokens(lat, gh, gw)
        else:
            txt = self._recv(txt0, self.base + self.pipe_rank - 1)
            img = self._recv(torch.empty(gh * gw, m.cfg.hidden, device=m.device, dtype=txt0.dtype), self.base + self.pipe_rank - 1)
        txt, img = m.run_blocks(txt, img, vec, caches, None, (gh, gw))
        if not self.last:
            self._send(txt, self.base + self.pipe_rank + 1)
            self._send(img, self.base + self.pipe_rank + 1)
        v = m.head(img, gh, gw, vec) if self.last else torch.empty_like(lat)
        if self.pipe_world > 1:
            dist.broadcast(v, src=self.base + self.pipe_world - 1, group=self.group)
        return v

    def _predict_patches(self, lat, t, txt0, pooled, caches) -> torch.Tensor:
        """PipeFusion step: row patches flow through the stages one after another."""
        m, P = self.m, self.pipe_world
        gh, gw = lat.shape[1] // m.cfg.patch, lat.shape[2] // m.cfg.patch
        vec = m.time_vec(t, pooled)
        bounds = [(gh * p // P) * gw for p in range(P + 1)]
        tokens_in = m.embed_tokens(lat, gh, gw) if self.first else None
        out = torch.empty(gh * gw, m.cfg.latent_channels * m.cfg.patch ** 2, device=m.device) if self.last else None
        for p in range(P):
            rows = slice(bounds[p], bounds[p + 1])
            n = bounds[p + 1] - bounds[p]
            if self.first:
                txt, img = txt0, tokens_in[rows]
            else:
                txt = self._recv(txt0, self.base + self.pipe_rank - 1)
                img = self._recv(torch.empty(n, m.cfg.hidden, device=m.device, dtype=txt0.dtype), self.base + self.pipe_rank - 1)
            txt, img = m.run_blocks(txt, img, vec, caches, rows, (gh, gw))
            if not self.last:
                self._send(txt, self.base + self.pipe_rank + 1)
                self._send(img, self.base + self.pipe_rank + 1)
                self.n_patch_hops += 1
            else:
                out[rows] = m.head_tokens(img, vec)
        v = m.unpatchify(out, gh, gw) if self.last else torch.empty_like(lat)
        dist.broadcast(v, src=self.base + P - 1, group=self.group)
        return v

    def _patch_pipeline(self, lat, ts, i0, txt0, pooled, caches, guidance, every, sent, partial_images, should_stop):
        """Steps ``i0 ..`` as one continuous flow of row patches (generator of the sampler's events).

        The latent lives in token space (``patchify`` is a permutation, so the Euler update acts row by row).  For step ``i``
        and patch ``p``: the first stage takes the patch's current rows (from step ``i0`` on they come back from the last
        stage), embeds them and runs its blocks; the hidden rows hop stage to stage; the last stage turns them into the
        patch's prediction, combines it with the mirror group's under CFG parallelism, updates the rows and returns them to
        the first stage.  The last stage posts the receive of the next patch BEFORE it sends a patch's rows back, which
        keeps every pair's sends and receives in one order on both sides (blocking transports cannot cycle).  When a preview
        is due, and at the end, the last stage's rows are broadcast to its group and every rank decodes them."""
        m, P = self.m, self.pipe_world
        gh, gw = lat.shape[1] // m.cfg.patch, lat.shape[2] // m.cfg.patch
        bounds = [(gh * p // P) * gw for p in range(P + 1)]
        n_steps = len(ts) - 1
        tok = m.patchify(lat).clone()                                   # [tokens, C * patch²]
        v_all = torch.zeros_like(tok) if self.last else None
        first_rank, last_rank = self.base, self.base + P - 1
        work = [(i, p) for i in range(i0, n_steps) for p in range(P)]
        nxt = None                                                      # last stage: the next patch's input, received early
        have_rows = False                                               # first stage: this step's rows were drained at a boundary

        def preview_due(i: int) -> bool:
            return bool(every) and (i + 1) % every == 0 and sent < partial_images and i + 1 < n_steps

        def cancel_check(i: int) -> bool:                               # the ranks agree on cancellation at the start of step i
            return i > i0 and (i - i0) % self.cancel_every == 0

        def drain() -> None:
            """First stage, before a step-boundary collective: take in every patch's returned rows, so that the last stage's
            sends complete before it enters the collective too."""
            for q in range(P):
                rq = slice(bounds[q], bounds[q + 1])
                tok[rq] = self._recv(tok[rq], last_rank)
        for k, (i, p) in enumerate(work):
            if p == 0 and cancel_check(i):
                if self.first and not have_rows:
                    drain()
                    have_rows = True
                if should_stop():
                    return
            t, t_next = ts[i], ts[i + 1]
            vec = m.time_vec(t, pooled)
            rows = slice(bounds[p], bounds[p + 1])
            n = bounds[p + 1] - bounds[p]
            boundary = p == P - 1 and (preview_due(i) or (i + 1 < n_steps and cancel_check(i + 1)))
            if self.first:
                if i > i0 and not have_rows:
                    tok[rows] = self._recv(tok[rows], last_rank)         # the rows after step i - 1
                if p == P - 1:
                    have_rows = False
                txt, img = txt0, m.embed_tokens(m.unpatchify(tok, gh, gw), gh, gw)[rows]
            elif nxt is not None:
                txt, img = nxt
                nxt = None
            else:
                txt = self._recv(txt0, self.base + self.pipe_rank - 1)
                img = self._recv(torch.empty(n, m.cfg.hidden, device=m.device, dtype=txt0.dtype), self.base + self.pipe_rank - 1)
            txt, img = m.run_blocks(txt, img, vec, caches, rows, (gh, gw))
            if not self.last:
                self._send(txt, self.base + self.pipe_rank + 1)
                self._send(img, self.base + self.pipe_rank + 1)
                self.n_patch_hops += 1
            else:
                v = m.head_tokens(img, vec)
                if guidance is not None:
                    v = self._guided(v, None, guidance)
                v_all[rows] = v
                tok[rows] = tok[rows] + (t_next - t) * v
                if k + 1 < len(work) and not boundary:                   # post the next patch's receive before sending this one back
                    pn = work[k + 1][1]
                    nn = bounds[pn + 1] - bounds[pn]
                    nxt = (self._recv(txt0, last_rank - 1), self._recv(torch.empty(nn, m.cfg.hidden, device=m.device, dtype=txt0.dtype), last_rank - 1))
                if i + 1 < n_steps:
                    self._send(tok[rows], first_rank)
            if p == P - 1 and preview_due(i):
                if self.first:
                    drain()
                    have_rows = True
                x0 = (tok - t_next * v_all) if self.last else torch.empty_like(tok)
                dist.broadcast(x0, src=last_rank, group=self.group)
                yield "partial", m.decode(m.unpatchify(x0, gh, gw)), sent, partial_images
                sent += 1
        dist.broadcast(tok, src=last_rank, group=self.group)
        yield "final", m.decode(m.unpatchify(tok, gh, gw)), 0, 0

    def _guided(self, v: torch.Tensor, v_other_fn: Callable[[], torch.Tensor] | None, guidance: float) -> torch.Tensor:
        """Combine the conditional and unconditional predictions (local second pass, or swap with the mirror group)."""
        if self.cfg_parallel:
            partner = (1 - self.cfg_rank) * self.pipe_world + self.pipe_rank
            if self.cfg_rank == 0:
                self._send(v, partner)
                other = self._recv(v, partner)
            else:
                other = self._recv(v, partner)
                self._send(v, partner)
            self.n_exchanges += 1
            cond, uncond = (v, other) if self.cfg_rank == 0 else (other, v)
            return uncond + guidance * (cond - uncond)
        if v_other_fn is not None:
            uncond = v_other_fn()
            return uncond + guidance * (v - uncond)
        return v

    # ---- the sampler ----
    def generate(self, prompt: str, height: int, width: int, steps: int, seed: int, *, guidance: float | None = None,
                 init_image: torch.Tensor | None = None, strength: float = 0.7, partial_images: int = 0,
                 should_stop: Callable[[], bool] = lambda: False) -> Iterator[tuple[str, torch.Tensor, int, int]]:
        """Yields ``("partial", rgb, index, total)`` previews and finally ``("final", rgb, 0, 0)``
        (or nothing more after ``should_stop()`` turned true; it is evaluated identically on every rank)."""
        m = self.m
        g = m.cfg.guidance if guidance is None else guidance
        gh, gw = m.grid(height, width)
        p = m.cfg.patch
        noise = torch.randn(m.cfg.latent_channels, gh * p, gw * p, generator=torch.Generator().manual_seed(seed)).to(m.device)
        lat = noise
        if hasattr(m, "guidance_value"):
            m.guidance_value = g                            # guidance-distilled models take the scale as an input
        kontext = init_image is not None and getattr(m.cfg, "kontext", False)
        if hasattr(m, "set_context"):
            m.set_context(init_image.to(m.device) if kontext else None, gh, gw)     # the reference picture as extra tokens
        if kontext:
            init_image = None
        if init_image is not None:
            x0 = m.encode_image(init_image.to(m.device), gh, gw)
        ts = m.schedule(steps, gh * gw) if hasattr(m, "schedule") else timesteps(steps, 1.0)
        if init_image is not None:
            skip = min(steps - 1, int(round(steps * (1.0 - strength))))
            ts = ts[skip:]
            lat = ts[0] * noise + (1 - ts[0]) * x0
        use_cfg = m.cfg.uses_cfg
        my_prompt = "" if (self.cfg_parallel and self.cfg_rank == 1) else prompt
        txt, pooled = m.encode_text(my_prompt)
        txt_u, pooled_u = m.encode_text("") if (use_cfg and not self.cfg_parallel) else (None, None)
        caches = {i: [None, None] for i in m.block_range} if self.pipe_world > 1 else None
        caches_u = {i: [None, None] for i in m.block_range} if (caches is not None and txt_u is not None) else None
        n_steps = len(ts) - 1
        every = max(1, n_steps // (partial_images + 1)) if partial_images > 0 else 0
        sent = 0
        for i in range(n_steps):
            if should_stop():
                return
            t, t_next = ts[i], ts[i + 1]
            patches = self.pipe_world > 1 and i >= self.num_sync_steps
            if patches and txt_u is None and self.async_patches:
                yield from self._patch_pipeline(lat, ts, i, txt, pooled, caches, g if use_cfg else None, every, sent, partial_images, should_stop)
                return
            predict = self._predict_patches if patches else self._predict_sync
            if self.pipe_world == 1:
                v = m.velocity(lat, t, txt, pooled)
                other = (lambda: m.velocity(lat, t, txt_u, pooled_u)) if txt_u is not None else None
            else:
                v = predict(lat, t, txt, pooled, caches)
                other = (lambda: predict(lat, t, txt_u, pooled_u, caches_u)) if txt_u is not None else None
            v = self._guided(v, other, g) if use_cfg else v
            lat = lat + (t_next - t) * v
            if every and (i + 1) % every == 0 and sent < partial_images and i + 1 < n_steps:
                x0_hat = lat - t_next * v
                yield "partial", m.decode(x0_hat), sent, partial_images
                sent += 1
        yield "final", m.decode(lat), 0, 0
