"""Per-rank step executor: turns a packed StepPlan into kernel launches.

One executor lives in each GPU process.  A step is: one host→device copy of the packed
plan from pinned memory, the decoder forward over this rank's shard, the vocabulary gather,
sampling on device, and one device→host copy of the sampled ids.  Pure-decode steps (one new
token per sequence) replay a CUDA graph captured per batch bucket, so the per-step host cost
is one memcpy and one graph launch.  This is the role the reference gives to mlx-lm's
``BatchGenerator`` step with its one-step-ahead ``async_eval`` pipelining
(``src/exo/worker/engines/mlx/patches/opt_batch_gen.py:57-136``).
"""
from __future__ import annotations

import os

import numpy as np
import torch

from .. import ops
from ..models.config import ModelConfig
from ..models.transformer import Decoder, KVPool, StepInputs, default_state_snapshots, make_decoder, make_kv_pool
from ..models.weights import ModelWeights, ShardSpec
from .plan import HEADER, PlanLayout, StepPlan, bucket, FLAG_ALL_GREEDY, FLAG_EAGER, FLAG_NO_SAMPLE, STATE_RESTORE, STATE_SAVE

DECODE_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)


class Executor:
    def __init__(self, cfg: ModelConfig, weights: ModelWeights, spec: ShardSpec | None = None, comm=None,
                 n_blocks: int = 256, block_size: int = 16, max_blocks_per_seq: int = 256,
                 max_tokens_per_step: int = 4096, max_seqs: int = 64, device: str | torch.device = "cpu",
                 use_graphs: bool | None = None, pipe=None, n_snapshots: int | None = None):
        self.cfg = cfg
        self.pipe = pipe if (pipe is not None and pipe.pp_size > 1) else None
        self.spec = spec or ShardSpec()
        self.device = torch.device(device)
        self.model = make_decoder(cfg, weights, self.spec, comm)
        self.kv = make_kv_pool(cfg, self.spec, n_blocks, block_size, self.device, max_seqs=max_seqs,
                               n_snapshots=default_state_snapshots(cfg, max_seqs) if n_snapshots is None else n_snapshots)
        self.block_size, self.max_blocks = block_size, max_blocks_per_seq
        self.max_T, self.max_B = max_tokens_per_step, max_seqs
        words = PlanLayout(max(self.max_T, self.max_B), self.max_B, self.max_blocks).words
        self.cuda = self.device.type == "cuda"
        # Pinned staging for the packed plan: a small ring, so that a caller which queues several steps without
        # reading results back never overwrites a buffer whose host-to-device copy is still pending (a slot is
        # reused only after the event recorded behind its copy has completed).
        self.hosts = [torch.zeros(words, dtype=torch.int32, pin_memory=self.cuda) for _ in range(4 if self.cuda else 1)]
        self.hosts_np = [h.numpy() for h in self.hosts]
        self.host_events: list[torch.cuda.Event | None] = [None] * len(self.hosts)
        self.n_runs = 0
        self.dev = torch.zeros(words, dtype=torch.int32, device=self.device)
        self.n_blocks = n_blocks
        self.last_layout: PlanLayout | None = None
        # MLA models whose dimensions the latent-attention kernel does not take (toy configs) run that op as PyTorch
        # ops with host reads of the sequence lengths: such a step cannot be captured
        mla_ok = not cfg.mla or (cfg.kv_lora_rank == 512 and cfg.qk_rope_dim == 64 and cfg.qk_nope_dim == 128
                                 and cfg.v_head_dim == 128 and cfg.dtype == "bf16")
        eager_experts = cfg.expert_bias and bool(cfg.n_experts)      # GPT-OSS experts run as PyTorch ops with host reads
        self.use_graphs = (self.cuda and mla_ok and not eager_experts) if use_graphs is None else (use_graphs and not eager_experts)
        if self.cuda and os.environ.get("EXO_KERNEL_CHECKS") == "1":
            self.use_graphs = False       # the checking flavour synchronises after every op: nothing can be captured
        if self.pipe is not None:
            self.use_graphs = False       # stage hops run on a side stream and wait on the peer: not capturable
        self.graphs: dict[int, tuple[torch.cuda.CUDAGraph, torch.Tensor]] = {}
        self.out_host = torch.zeros(self.max_B, dtype=torch.int32, pin_memory=self.cuda)
        self.prev_sampled = torch.zeros(max(self.max_B, 256), dtype=torch.int32, device=self.device)
        self.last_logits: torch.Tensor | None = None
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.n_launch_steps = 0
        self.launches_per_graph: dict[int, int] = {}

    # ------------------------------------------------------------------ helpers
    def _views(self, L: PlanLayout) -> tuple[StepInputs, dict[str, torch.Tensor]]:
        d = self.dev
        f = d.view(torch.float32)
        inp = StepInputs(
            tokens=d[L.tokens:L.tokens + L.T], positions=d[L.positions:L.positions + L.T],
            slots=d[L.slots:L.slots + L.T], cu_q=d[L.cu_q:L.cu_q + L.B + 1], seq_lens=d[L.seq_lens:L.seq_lens + L.B],
            block_tables=d[L.block_tables:L.block_tables + L.B * L.max_blocks].view(L.B, L.max_blocks),
            logit_rows=d[L.logit_rows:L.logit_rows + L.B], max_q_len=1,
            state_slots=d[L.state_slots:L.state_slots + L.B])
        samp = dict(top_k=d[L.top_k:L.top_k + L.B], temperature=f[L.temperature:L.temperature + L.B],
                    top_p=f[L.top_p:L.top_p + L.B], min_p=f[L.min_p:L.min_p + L.B],
                    uniform=f[L.uniform:L.uniform + L.B], prev_rows=d[L.prev_rows:L.prev_rows + L.B])
        return inp, samp

    def _forward_sample(self, inp: StepInputs, samp: dict[str, torch.Tensor], greedy: bool,
                        from_prev: bool) -> torch.Tensor:
        if from_prev:
            # decode continuation: input token of row b = previous step's sample at prev_rows[b]
            pr = samp["prev_rows"]
            prev = self.prev_sampled[pr.clamp_min(0).long()]
            inp.tokens.copy_(torch.where(pr >= 0, prev, inp.tokens))
        if self.pipe is not None:
            return self._forward_sample_pipelined(inp, samp, greedy)
        logits = self.model.comm.gather_vocab(self.model.forward(inp, self.kv))
        self.last_logits = logits
        ids = self._sample(logits, samp, greedy)
        self.prev_sampled[:ids.numel()].copy_(ids)
        return ids

    def _sample(self, logits: torch.Tensor, samp: dict[str, torch.Tensor], greedy: bool) -> torch.Tensor:
        if greedy:
            ids = ops.argmax(logits[:, :self.cfg.vocab])
        else:
            ids = ops.sample(logits[:, :self.cfg.vocab], samp["temperature"], samp["top_k"], samp["top_p"],
                             samp["min_p"], samp["uniform"])
        return ids.to(torch.int32)

    def _forward_only(self, inp: StepInputs) -> torch.Tensor:
        """A step of prompt chunks none of which ends its sequence: the layers run (the KV cache fills), the vocabulary
        projection and the sampler do not, and with pipeline stages nothing travels back, so a stage starts on the
        next chunk as soon as it has handed this one on (the reference's ``pipeline_parallel_prefill``,
        ``src/exo/worker/engines/mlx/generator/generate.py:164-279``)."""
        spec, pipe = self.spec, self.pipe
        h_in = None
        if pipe is not None and not spec.is_first_stage:
            h_in = pipe.recv_hidden(inp.tokens.shape[0], self.cfg.hidden, self._act_dtype(), self.device)
        out = self.model.forward(inp, self.kv, h_in, need_logits=False)
        if pipe is not None:
            pipe.consumed()
            if not spec.is_last_stage:
                pipe.send_hidden(out)
        return self.prev_sampled[:0]

    def _act_dtype(self) -> torch.dtype:
        return torch.bfloat16 if self.cfg.dtype == "bf16" else torch.float32

    def _forward_sample_pipelined(self, inp: StepInputs, samp: dict[str, torch.Tensor], greedy: bool) -> torch.Tensor:
        """One pipeline stage of a step: receive the residual stream, run this stage's layers, pass
        it on; the last stage samples and its ids go back to every stage of the lane."""
        spec, pipe = self.spec, self.pipe
        h_in = None
        if not spec.is_first_stage:
            h_in = pipe.recv_hidden(inp.tokens.shape[0], self.cfg.hidden, self._act_dtype(), self.device)
        out = self.model.forward(inp, self.kv, h_in)
        pipe.consumed()
        n = inp.logit_rows.numel()
        if spec.is_last_stage:
            logits = self.model.comm.gather_vocab(out)
            self.last_logits = logits
            ids = self._sample(logits, samp, greedy)
        else:
            pipe.send_hidden(out)
            ids = torch.zeros(n, dtype=torch.int32, device=self.device)
        ids = pipe.share_ids(ids)
        self.prev_sampled[:ids.numel()].copy_(ids)
        return ids

    def _validate(self, plan: StepPlan) -> None:
        """Reject a plan that addresses KV storage this rank does not have.  The kernels index the pool with the
        plan's slots and block tables unchecked; the leader's allocator and this rank's pool are sized from an
        agreed block count, and this is the guard behind that agreement."""
        n_slots = self.n_blocks * self.block_size
        if plan.n_tokens and (int(plan.slots.max()) >= n_slots or int(plan.slots.min()) < 0):
            raise ValueError(f"step plan writes KV slot {int(plan.slots.max())} outside this rank's pool of {n_slots} slots")
        if plan.block_tables.size and (int(plan.block_tables.max()) >= self.n_blocks or int(plan.block_tables.min()) < 0):
            raise ValueError(f"step plan reads KV block {int(plan.block_tables.max())} outside this rank's pool of "
                             f"{self.n_blocks} blocks")
        if plan.block_tables.shape[1] > self.max_blocks and plan.is_decode:
            raise ValueError("step plan's block table is wider than this rank's decode graphs")

    # ------------------------------------------------------------------ step
    def run(self, plan: StepPlan, logits_processor=None) -> torch.Tensor:
        """Execute one step; returns the sampled ids ``[n_seqs]`` on device (int32).  The plan's state instructions
        (hybrid models: recurrent state copied from a prefix-cache snapshot into a sequence's seat before the step, or
        from a seat into a snapshot after it) are stream-ordered device copies around the step's kernels."""
        for kind, seat, snap in plan.state_ops:
            if kind == STATE_RESTORE:
                self.kv.restore_state(seat, snap)
        out = self._run_step(plan, logits_processor)
        for kind, seat, snap in plan.state_ops:
            if kind == STATE_SAVE:
                self.kv.save_state(seat, snap)
        return out

    def _run_step(self, plan: StepPlan, logits_processor=None) -> torch.Tensor:
        decode = plan.is_decode
        if decode:
            bB = bucket(plan.n_seqs, DECODE_BUCKETS)
            bT = bB
        else:
            bB, bT = plan.n_seqs, plan.n_tokens
        mb = self.max_blocks if decode else max(1, plan.block_tables.shape[1])
        self._validate(plan)
        slot = self.n_runs % len(self.hosts)
        self.n_runs += 1
        if self.host_events[slot] is not None:
            self.host_events[slot].synchronize()
        L = plan.pack(self.hosts_np[slot], bT, bB, mb)
        self.last_layout = L
        self.dev[:L.words].copy_(self.hosts[slot][:L.words], non_blocking=True)
        if self.cuda:
            ev = self.host_events[slot] or torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self.host_events[slot] = ev
        self.h2d_bytes += L.words * 4
        greedy = bool(plan.flags & FLAG_ALL_GREEDY)
        from_prev = bool(plan.flags & 1)
        self.n_launch_steps += 1
        if decode and self.use_graphs and logits_processor is None and not (plan.flags & FLAG_EAGER):
            key = (bB, greedy, from_prev)
            if key not in self.graphs:
                self._capture(key, L)
            g, out = self.graphs[key]
            g.replay()
            return out[:plan.n_seqs]
        inp, samp = self._views(L)
        inp.max_q_len = plan.max_q_len
        if plan.flags & FLAG_NO_SAMPLE:
            return self._forward_only(inp)
        if logits_processor is None:
            return self._forward_sample(inp, samp, greedy, from_prev)[:plan.n_seqs]
        # slow path (penalties / logit bias / logprobs): processor edits full logits before sampling
        logits = self.model.comm.gather_vocab(self.model.forward(inp, self.kv))[:, :self.cfg.vocab]
        logits = logits_processor(logits[:plan.n_seqs].float())
        self.last_logits = logits
        ids = ops.sample(logits, samp["temperature"][:plan.n_seqs], samp["top_k"][:plan.n_seqs],
                         samp["top_p"][:plan.n_seqs], samp["min_p"][:plan.n_seqs],
                         samp["uniform"][:plan.n_seqs]).to(torch.int32)
        self.prev_sampled[:ids.numel()].copy_(ids)
        return ids

    def _capture(self, key: tuple[int, bool, bool], L: PlanLayout) -> None:
        bB, greedy, from_prev = key
        inp, samp = self._views(L)
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        saved = self.prev_sampled.clone()  # warm-up runs must not disturb the token chain
        with torch.cuda.stream(stream):  # warm-up outside capture (per-device scratch set-up)
            # a recurrent layer's state update is not idempotent (appending the same KV row twice is): the warm-up
            # runs advance the scratch seat instead of the sequences' own
            seats = inp.state_slots.clone() if self.cfg.has_linear_layers else None
            if seats is not None:
                inp.state_slots.zero_()
            for _ in range(2):
                self._forward_sample(inp, samp, greedy, from_prev)
                self.prev_sampled.copy_(saved)
            if seats is not None:
                inp.state_slots.copy_(seats)
        torch.cuda.current_stream(self.device).wait_stream(stream)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        from ..ops import cuda as _k
        before = _k.launch_count
        with torch.cuda.graph(g, stream=stream):
            out = self._forward_sample(inp, samp, greedy, from_prev)
        self.launches_per_graph[bB] = _k.launch_count - before  # own kernels replayed per step
        self.graphs[key] = (g, out)

    def fetch(self, ids: torch.Tensor) -> np.ndarray:
        """Blocking device→host read of a step's sampled ids."""
        n = ids.numel()
        self.out_host[:n].copy_(ids, non_blocking=True)
        if self.cuda:
            torch.cuda.current_stream(self.device).synchronize()
            # the step's kernels have completed: an expired device-side wait (a peer that stopped answering, a stuck
            # pipeline) must end the runner instead of streaming tokens made from unsummed data
            ops.cuda_ops().check_status(self.device)
            if ops.cuda_ops().CHECKS:
                ops.cuda_ops().verify_guards()
        self.d2h_bytes += n * 4
        return self.out_host[:n].numpy().copy()
