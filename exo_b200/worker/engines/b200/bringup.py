"""Bring-up of one rank of a B200 instance, and the leader → follower plan channel.

See ``builder.py`` for the serving engine.  The rank group is a ``torch.distributed`` world on
127.0.0.1 (NCCL for tensors on GPUs, gloo for the small host-side control messages and for CPU
ranks).  Every step the leader broadcasts one control message ``(packed plan | None, finished task
ids, stop flag)``; a follower executes the plan and reports the finished tasks to its own runner.
"""
from __future__ import annotations

import datetime
import os
from collections.abc import Iterable, Iterator
from pathlib import Path
from typing import Any

import numpy as np
import torch
import torch.distributed as dist

from ....engine.engine import Engine as TokenEngine
from ....engine.executor import Executor
from ....engine.plan import HEADER, PlanLayout, StepPlan
from ....models.config import ModelConfig
from ....models.transformer import default_state_snapshots, KVPool
from ....parallel.comm import PipeComm
from ....models.weights import (_DTYPES, RandomSource, SafetensorsSource, ShardSpec, build_weights, fast_random_weights,
                                vocab_shard)
from ....shared import constants
from ....shared.base import TaskId
from ....shared.messages import GenerationTask
from ....shared.wire import BoundInstance, NvlinkInstance
from ..base import Builder, Cancelled, Engine, Finished, LoadProgress, StepItem
from .builder import ServingEngine, find_model_dir
from .tokenizer import eos_ids, load_tokenizer


class PlanChannel:
    """Control messages from rank 0 to the other ranks of the instance, through a shared-memory ring.

    Every step the leader publishes ``(packed plan | None, finished task ids, stop flag)``.  The ranks of an
    instance are processes of one box, so the message is a memcpy into a POSIX shared-memory segment followed by a
    sequence-number store; followers spin on the number (a few microseconds end to end) and acknowledge by storing
    the number they have consumed, which is what lets the leader reuse a slot.  The rendezvous (segment name) and
    the one-off agreements of the bring-up still go through the ``gloo`` group.  This stands where the reference has
    its per-step task / cancel agreement collectives on the CPU stream
    (``src/exo/worker/engines/mlx/utils_mlx.py:833-938``)."""

    SLOTS = 4
    HDR_WORDS = 64           # int64: [0] last published sequence number, [8 + r] last number consumed by rank r

    def __init__(self, group, rank: int, world: int | None = None, slot_bytes: int = 4 << 20):
        from multiprocessing import shared_memory
        self.group, self.rank = group, rank
        self.world = world if world is not None else dist.get_world_size(group)
        self.slot_bytes = slot_bytes
        self.seq = 0
        size = self.HDR_WORDS * 8 + self.SLOTS * slot_bytes
        box: list[Any] = [None]
        if rank == 0:
            self.shm = shared_memory.SharedMemory(create=True, size=size)
            box[0] = self.shm.name
        dist.broadcast_object_list(box, src=0, group=group)
        if rank != 0:
            self.shm = shared_memory.SharedMemory(name=box[0])
            try:        # the leader owns the segment: keep this process's resource tracker from unlinking it at exit
                from multiprocessing import resource_tracker
                resource_tracker.unregister(self.shm._name, "shared_memory")
            except Exception:  # noqa: BLE001
                pass
        self.hdr = np.ndarray((self.HDR_WORDS,), dtype=np.int64, buffer=self.shm.buf)
        if rank == 0:
            self.hdr[:] = 0
        dist.barrier(group=group)
        self.timeout_s = float(os.environ.get("EXO_GROUP_TIMEOUT_S", "120"))

    def _slot(self, seq: int) -> np.ndarray:
        off = self.HDR_WORDS * 8 + (seq % self.SLOTS) * self.slot_bytes
        return np.ndarray((self.slot_bytes // 4,), dtype=np.int32, buffer=self.shm.buf, offset=off)

    @staticmethod
    def _wait(cond, timeout_s: float, what: str) -> None:
        import time
        t0 = None
        spins = 0
        while not cond():
            spins += 1
            if spins < 2000:
                continue
            if t0 is None:
                t0 = time.perf_counter()
            elif time.perf_counter() - t0 > timeout_s:
                raise TimeoutError(f"plan channel: {what}")
            time.sleep(20e-6)

    def send(self, plan: StepPlan | None, finished: list[str], stop: bool = False) -> None:
        seq = self.seq + 1
        # a slot is free once every follower has consumed the message that used it last
        need = seq - self.SLOTS
        if need > 0:
            acks = self.hdr[8 + 1:8 + self.world]
            self._wait(lambda: int(acks.min()) >= need, self.timeout_s, "a follower stopped consuming plans")
        slot = self._slot(seq)
        words = 0
        if plan is not None:
            mb = max(1, plan.block_tables.shape[1])
            words = PlanLayout(plan.n_tokens, plan.n_seqs, mb).words
            if (8 + words) * 4 > self.slot_bytes:
                raise ValueError(f"step plan of {words} words does not fit the plan channel's {self.slot_bytes} byte slots")
            plan.pack(slot[8:], plan.n_tokens, plan.n_seqs, mb)
        # caller-supplied embedding rows of this step (image features): (first row, row count) pairs behind the plan; the rows
        # themselves follow on the device group (``LeaderServingEngine._send_rows``)
        embeds = list(getattr(plan, "embeds", None) or []) if plan is not None else []
        for j, (r0, n_rows) in enumerate(embeds):
            slot[8 + words + 2 * j], slot[8 + words + 2 * j + 1] = r0, n_rows
        words_all = words + 2 * len(embeds)
        tail = ("\n".join(finished)).encode()
        if (8 + words_all) * 4 + len(tail) > self.slot_bytes:
            raise ValueError("plan channel message too large")
        slot[0:5] = (1 if plan is not None else 0, words, len(tail), 1 if stop else 0, len(embeds))
        if tail:
            np.frombuffer(self.shm.buf, dtype=np.uint8, count=len(tail),
                          offset=self.HDR_WORDS * 8 + (seq % self.SLOTS) * self.slot_bytes + (8 + words_all) * 4)[:] = np.frombuffer(tail, np.uint8)
        self.hdr[0] = seq          # published: the payload stores above are ordered before this one (x86 TSO)
        self.seq = seq

    def recv(self) -> tuple[StepPlan | None, list[str], bool]:
        seq = self.seq + 1
        self._wait(lambda: int(self.hdr[0]) >= seq, self.timeout_s, "the leader stopped publishing plans")
        slot = self._slot(seq)
        has_plan, words, n_tail, stop, n_embeds = (int(x) for x in slot[0:5])
        plan = StepPlan.unpack(slot[8:8 + words]) if has_plan else None
        if plan is not None:
            plan.embeds = [(int(slot[8 + words + 2 * j]), int(slot[8 + words + 2 * j + 1])) for j in range(n_embeds)] or None
        finished: list[str] = []
        if n_tail:
            off = self.HDR_WORDS * 8 + (seq % self.SLOTS) * self.slot_bytes + (8 + words + 2 * n_embeds) * 4
            finished = bytes(self.shm.buf[off:off + n_tail]).decode().split("\n")
        self.hdr[8 + self.rank] = seq
        self.seq = seq
        return plan, finished, bool(stop)

    def close(self) -> None:
        if self.rank == 0:
            try:
                self.send(None, [], stop=True)
            except (RuntimeError, TimeoutError, ValueError):
                pass
        shm, self.shm = getattr(self, "shm", None), None
        if shm is None:
            return
        self.hdr = None
        try:
            shm.close()
            if self.rank == 0:
                shm.unlink()
        except (BufferError, FileNotFoundError, OSError):
            pass


class LeaderServingEngine(ServingEngine):
    """Rank 0 of a multi-rank instance: every plan and every completion is broadcast."""

    def warmup(self) -> None:
        super().warmup()
        self.control.send(None, ["warmup"])   # releases the followers' warm-up loop

    def step(self):
        items = list(super().step())
        done = [str(t) for t, it in items if isinstance(it, (Finished, Cancelled))]
        if done:
            self.control.send(None, done)
        return items

    def _sink(self, plan: StepPlan) -> None:
        self.control.send(plan, [])

    def _send_rows(self, patches) -> None:
        """Caller-supplied embedding rows (image features) of the plan just published, to every other rank: one broadcast
        per run of rows on the instance's device group, in the order of the plan's ``embeds`` pairs."""
        exe = self.te.exe
        for _r0, rows in patches:
            dist.broadcast(rows.to(device=exe.device, dtype=_DTYPES[self.cfg.dtype]).contiguous(), src=0)


class FollowerServingEngine(Engine):
    """Ranks > 0: execute broadcast plans; know tasks only by id."""

    def __init__(self, executor: Executor, control: PlanChannel):
        self.exe, self.control = executor, control
        self.active: set[str] = set()
        self.stopped = False

    def warmup(self) -> None:
        self._drain_until_idle()

    def _drain_until_idle(self) -> None:
        # the leader's warm-up generation is a normal request stream that ends with a completion message
        while True:
            plan, finished, stop = self.control.recv()
            if plan is not None:
                self._run(plan)
            if stop:
                self.stopped = True
                return
            if finished:
                return

    def _run(self, plan: StepPlan) -> None:
        """Execute a broadcast plan; embedding rows the leader supplies for it (image features) arrive first."""
        if getattr(plan, "embeds", None):
            cfg = self.exe.model.cfg
            patches = []
            for r0, n_rows in plan.embeds:
                t = torch.empty(n_rows, cfg.hidden, dtype=_DTYPES[cfg.dtype], device=self.exe.device)
                dist.broadcast(t, src=0)
                patches.append((r0, t))
            self.exe.model.embed_patches = patches if self.exe.spec.is_first_stage else None
        self.exe.run(plan)

    def submit(self, task: GenerationTask) -> None:
        self.active.add(str(task.task_id))

    def cancel(self, task_id: TaskId) -> None:
        pass  # the leader decides; its completion message releases the task here

    @property
    def has_work(self) -> bool:
        return bool(self.active) and not self.stopped

    def step(self) -> Iterable[tuple[TaskId, StepItem]]:
        plan, finished, stop = self.control.recv()
        if plan is not None:
            self._run(plan)
        out: list[tuple[TaskId, StepItem]] = []
        for t in finished:
            if t in self.active:
                self.active.discard(t)
                out.append((TaskId(t), Finished()))
        if stop:
            self.stopped = True
            for t in list(self.active):
                out.append((TaskId(t), Finished()))
            self.active.clear()
        return out


class B200Builder(Builder):
    def __init__(self, bound_instance: BoundInstance):
        super().__init__(bound_instance)
        sh = bound_instance.bound_shard
        self.card = sh.model_card
        self.rank, self.world = sh.device_rank, sh.world_size
        self.spec = ShardSpec(tp_rank=sh.tp_rank, tp_size=sh.tp_size, layer_start=sh.start_layer, layer_end=sh.end_layer,
                              pp_rank=sh.pp_rank, pp_size=sh.pp_size)
        want_cpu = os.environ.get("EXO_DEVICE", "").lower() == "cpu" or not torch.cuda.is_available()
        gpu = sh.gpu_index if sh.gpu_index is not None else int(os.environ.get("EXO_GPU_INDEX", "0"))
        self.device = torch.device("cpu") if want_cpu else torch.device("cuda", gpu)
        self.comm = None
        self.tp_group = None
        self.pipe: PipeComm | None = None
        self.control: PlanChannel | None = None
        self.weights = None
        self.cfg: ModelConfig | None = None
        self.model_dir = find_model_dir(str(self.card.model_id))

    def connect(self) -> None:
        sh = self.bound_instance.bound_shard
        if sh.should_timeout:
            import time
            time.sleep(sh.should_timeout)
        if self.world == 1:
            return
        inst = self.bound_instance.instance
        port = inst.rendezvous_port if isinstance(inst, NvlinkInstance) else getattr(inst, "ephemeral_port", 29555)
        backend = "gloo" if self.device.type == "cpu" else "nccl"
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        dist.init_process_group(backend, init_method=f"tcp://127.0.0.1:{port}", rank=self.rank, world_size=self.world,
                                timeout=datetime.timedelta(seconds=int(os.environ.get("EXO_GROUP_TIMEOUT_S", "120"))),
                                **({"device_id": self.device} if backend == "nccl" else {}))
        ctl = dist.new_group(backend="gloo") if backend == "nccl" else dist.group.WORLD
        self.control = PlanChannel(ctl, self.rank, self.world)
        tp, pp = self.spec.tp_size, self.spec.pp_size
        if pp > 1:      # every rank creates every group, in the same order: one per stage, then one per lane
            stage_groups = [dist.new_group([s * tp + t for t in range(tp)]) for s in range(pp)]
            lane_groups = [dist.new_group([s * tp + t for s in range(pp)]) for t in range(tp)]
            self.tp_group = stage_groups[self.spec.pp_rank]
            self.pipe = PipeComm(self.spec.pp_rank, pp, self.spec.tp_rank, tp, lane_groups[self.spec.tp_rank])

    def _config(self) -> ModelConfig:
        if self.model_dir is not None:
            cfg = ModelConfig.from_pretrained(self.model_dir)
        else:
            raise FileNotFoundError(f"no checkpoint directory for {self.card.model_id}")
        cfg.dtype = "fp32" if self.device.type == "cpu" else "bf16"
        return cfg

    def load(self) -> Iterator[LoadProgress]:
        self.cfg = cfg = self._config()
        total = len(self.spec.layers(cfg))
        progress: list[int] = []
        has_weights = self.model_dir is not None and any(self.model_dir.glob("*.safetensors"))
        if has_weights:
            src = SafetensorsSource(self.model_dir, device="cpu",
                                    dtype=torch.float32 if cfg.dtype == "fp32" else torch.bfloat16)
        elif os.environ.get("EXO_RANDOM_INIT", "0") == "1":
            src = RandomSource(seed=0, dtype=torch.float32 if cfg.dtype == "fp32" else torch.bfloat16)
        else:
            raise FileNotFoundError(f"no *.safetensors under {self.model_dir} (set EXO_RANDOM_INIT=1 for random weights)")
        # build_weights reports per layer; it is a plain function, so collect and replay as progress
        self.weights = build_weights(cfg, self.spec, src, self.device, progress=lambda d, t: progress.append(d))
        for d in progress or [total]:
            yield LoadProgress(d, total)

    def _n_blocks(self, cfg: ModelConfig) -> int:
        per_block = max(1, KVPool.bytes_per_block(cfg, self.spec, constants.EXO_KV_BLOCK_SIZE))
        if self.device.type == "cuda":
            free, _total = torch.cuda.mem_get_info(self.device)
            budget = int(free * constants.EXO_GPU_MEMORY_FRACTION)
            # hybrid models: the sequences' recurrent state is allocated beside the paged cache
            seats = max(constants.EXO_MAX_CONCURRENT_REQUESTS, 8)
            budget -= KVPool.state_bytes(cfg, self.spec, seats + default_state_snapshots(cfg, seats))
        else:
            budget = 256 << 20
        cap = int(os.environ.get("EXO_MAX_KV_BLOCKS", "0"))
        n = max(64, budget // per_block)
        n = min(n, cap) if cap else n
        return self._agree_min(n)

    def _agree_min(self, n: int) -> int:
        """The smallest value over the instance's ranks.  Only rank 0's allocator hands out block ids, and every
        rank indexes its own pool with them: a rank with less free memory, or a pipeline stage with more layers or
        the vocabulary head, would otherwise receive slots past the end of its pool."""
        if self.world == 1 or self.control is None or not dist.is_initialized():
            return n
        t = torch.tensor([n], dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.control.group)
        return int(t.item())

    def _graphs(self) -> bool | None:
        """CUDA graphs for decode steps.  Every rank executes the same plans in the same order and the leader marks
        the steps it runs eagerly, so all ranks capture and replay at the same steps; pipeline stages exchange
        activations with blocking point-to-point calls and stay eager."""
        return None if self.spec.pp_size == 1 else False

    def build(self) -> Engine:
        assert self.cfg is not None and self.weights is not None
        cfg = self.cfg
        if self.spec.tp_size > 1:
            # the peer-memory collectives span one tensor-parallel group: the whole instance, or one pipeline stage
            if self.device.type == "cuda" and cfg.dtype == "bf16" and os.environ.get("EXO_COMM", "fused") == "fused":
                from ....parallel.fused import FusedComm
                self.comm = FusedComm(self.device, max_rows=constants.PREFILL_CHUNK, hidden=cfg.hidden,
                                      vocab_shard=vocab_shard(cfg.vocab, self.spec.tp_size), group=self.tp_group)
            else:
                from ....parallel.comm import DistComm
                self.comm = DistComm(self.tp_group)
        n_blocks = self._n_blocks(cfg)
        max_seqs = max(constants.EXO_MAX_CONCURRENT_REQUESTS, 8)
        mbs = min(n_blocks, -(-min(cfg.max_position, 1 << 17) // constants.EXO_KV_BLOCK_SIZE))
        if self.rank != 0:
            exe = Executor(cfg, self.weights, self.spec, self.comm, n_blocks=n_blocks, max_blocks_per_seq=mbs,
                           max_tokens_per_step=constants.PREFILL_CHUNK, max_seqs=max_seqs, device=self.device,
                           use_graphs=self._graphs(), pipe=self.pipe)
            assert self.control is not None
            return FollowerServingEngine(exe, self.control)
        tok = load_tokenizer(self.model_dir, cfg.vocab)
        eos = eos_ids(tok, self.model_dir, cfg.eos_token_ids, str(self.card.model_id))
        cfg.eos_token_ids = eos
        cls = LeaderServingEngine if self.world > 1 else ServingEngine
        te = TokenEngine(cfg, self.weights, self.spec, self.comm, n_blocks=n_blocks, max_seqs=max_seqs,
                         prefill_chunk=constants.PREFILL_CHUNK, max_blocks_per_seq=mbs, device=self.device,
                         use_graphs=self._graphs(), pipe=self.pipe)
        eng = cls(cfg, te, tok, str(self.card.model_id), self.card.family, eos, self.card.reasoning_dialect, self.rank,
                  self.control)
        if self.world > 1:
            te.plan_sink = eng._sink
            te.embed_sink = eng._send_rows
        elif constants.ENABLE_DISAGGREGATION:
            eng.enable_prefill_server()      # its port travels in RunnerReady; the master pairs instances through links
        return eng

    def close(self) -> None:
        try:
            if self.comm is not None and hasattr(self.comm, "close"):
                self.comm.close()
        finally:
            if dist.is_available() and dist.is_initialized():
                try:
                    dist.destroy_process_group()
                except RuntimeError:
                    pass
