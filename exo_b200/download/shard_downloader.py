"""Download of everything one shard needs, with progress, and the downloader interface.

``download_shard`` mirrors the reference's flow (``src/exo/download/download_utils.py:868-1059``):
file list (cached) → allow/ignore filter (``original/*`` and ``metal/*`` are never fetched; image
models skip root-level safetensors because their weights sit in component folders) → a writable
root with room → up to ``max_parallel_downloads`` files at once → per-file and whole-repo
progress (bytes, this-session bytes, speed, ETA, status).  Every rank of a tensor-parallel group
needs every weight file (each reads its slice of every tensor), so the default pattern is
``*``; a pipeline stage may pass layer-derived patterns.  The downloader classes follow
``shard_downloader.py:19-113`` and ``impl_shard_downloader.py:27-275``.
"""
from __future__ import annotations

import asyncio
import time
from abc import ABC, abstractmethod
from collections.abc import AsyncIterator, Awaitable, Callable
from datetime import timedelta
from pathlib import Path
from typing import Literal

from pydantic import BaseModel, ConfigDict, Field

from ..shared import constants
from ..shared.base import Memory, ModelId
from ..shared.cards import ModelCard, ModelTask, card_cache
from ..shared.wire import DownloadProgressData, PipelineShardMetadata, ShardMetadata
from . import hf
from .store import FileListEntry, downloaded_size, resolve_existing_model, select_download_dir_for

Status = Literal["not_started", "in_progress", "complete"]


class RepoFileDownloadProgress(BaseModel):
    model_config = ConfigDict(frozen=True)
    repo_id: str
    repo_revision: str
    file_path: str
    downloaded: Memory
    downloaded_this_session: Memory
    total: Memory
    speed: float
    eta: timedelta
    status: Status
    start_time: float


class RepoDownloadProgress(BaseModel):
    model_config = ConfigDict(frozen=True)
    repo_id: str
    repo_revision: str
    shard: ShardMetadata
    completed_files: int
    total_files: int
    downloaded: Memory
    downloaded_this_session: Memory
    total: Memory
    overall_speed: float
    overall_eta: timedelta
    status: Status
    file_progress: dict[str, RepoFileDownloadProgress] = Field(default_factory=dict)


ProgressCallback = Callable[[ShardMetadata, RepoDownloadProgress], Awaitable[None]]


def _eta_ms(eta: timedelta) -> int:
    return int(eta.total_seconds() * 1000)


def file_progress_data(p: RepoFileDownloadProgress) -> DownloadProgressData:
    return DownloadProgressData(total=p.total, downloaded=p.downloaded, downloaded_this_session=p.downloaded_this_session,
                                completed_files=1 if p.status == "complete" else 0, total_files=1, speed=p.speed,
                                eta_ms=_eta_ms(p.eta), files={})


def progress_data(p: RepoDownloadProgress) -> DownloadProgressData:
    """Wire form of a repo's progress (one level of per-file entries)."""
    return DownloadProgressData(total=p.total, downloaded=p.downloaded, downloaded_this_session=p.downloaded_this_session,
                                completed_files=p.completed_files, total_files=p.total_files, speed=p.overall_speed,
                                eta_ms=_eta_ms(p.overall_eta),
                                files={k: file_progress_data(v) for k, v in p.file_progress.items()})


def repo_progress(shard: ShardMetadata, revision: str, files: dict[str, RepoFileDownloadProgress], t0: float) -> RepoDownloadProgress:
    total = sum((f.total for f in files.values()), Memory())
    done = sum((f.downloaded for f in files.values()), Memory())
    session = sum((f.downloaded_this_session for f in files.values()), Memory())
    elapsed = time.time() - t0
    speed = session.in_bytes / elapsed if elapsed > 0 else 0.0
    eta = timedelta(seconds=(total - done).in_bytes / speed) if speed > 0 else timedelta(0)
    status: Status = ("complete" if all(f.status == "complete" for f in files.values())
                      else "in_progress" if any(f.status == "in_progress" for f in files.values()) else "not_started")
    return RepoDownloadProgress(repo_id=str(shard.model_card.model_id), repo_revision=revision, shard=shard,
                                completed_files=sum(1 for f in files.values() if f.downloaded == f.total),
                                total_files=len(files), downloaded=done, downloaded_this_session=session, total=total,
                                overall_speed=speed, overall_eta=eta, status=status, file_progress=dict(files))


def is_image_model(card: ModelCard) -> bool:
    return ModelTask.TextToImage in card.tasks or ModelTask.ImageToImage in card.tasks


async def download_shard(shard: ShardMetadata, on_progress: ProgressCallback, *, max_parallel_downloads: int = 8,
                         skip_download: bool = False, skip_internet: bool = False, allow_patterns: list[str] | None = None,
                         on_connection_lost: Callable[[], None] = lambda: None) -> tuple[Path, RepoDownloadProgress]:
    model_id, revision = shard.model_card.model_id, "main"
    t0 = time.time()
    try:
        listing = await hf.fetch_file_list_with_cache(model_id, revision, skip_internet=skip_internet,
                                                      on_connection_lost=on_connection_lost)
    except FileNotFoundError:
        return (constants.EXO_DEFAULT_MODELS_DIR / ModelId(model_id).normalize(),
                RepoDownloadProgress(repo_id=str(model_id), repo_revision=revision, shard=shard, completed_files=0, total_files=0,
                                     downloaded=Memory(), downloaded_this_session=Memory(), total=Memory(), overall_speed=0.0,
                                     overall_eta=timedelta(0), status="not_started"))
    files: list[FileListEntry] = list(hf.filter_repo_objects(listing, allow_patterns=allow_patterns or ["*"],
                                                             ignore_patterns=["original/*", "metal/*"], key=lambda f: f.path))
    if is_image_model(shard.model_card):
        files = [f for f in files if "/" in f.path or not f.path.endswith(".safetensors")]
    total = sum(f.size or 0 for f in files)
    if skip_download:
        target = resolve_existing_model(model_id) or constants.EXO_DEFAULT_MODELS_DIR / ModelId(model_id).normalize()
    else:
        target = select_download_dir_for(model_id, files, total) / ModelId(model_id).normalize()
        target.mkdir(parents=True, exist_ok=True)

    prog: dict[str, RepoFileDownloadProgress] = {}
    for f in files:
        have = downloaded_size(target / f.path)
        prog[f.path] = RepoFileDownloadProgress(
            repo_id=str(model_id), repo_revision=revision, file_path=f.path, downloaded=Memory.from_bytes(have),
            downloaded_this_session=Memory(), total=Memory.from_bytes(f.size or 0), speed=0.0, eta=timedelta(0),
            status="complete" if (target / f.path).exists() and have == f.size else "not_started", start_time=time.time())

    pending: set[asyncio.Task] = set()

    async def report(f: FileListEntry, cur: int, tot: int, renamed: bool) -> None:
        prev = prog.get(f.path)
        restarted = prev is None or cur < prev.downloaded.in_bytes
        start = time.time() if restarted else prev.start_time
        session = cur if restarted else prev.downloaded_this_session.in_bytes + (cur - prev.downloaded.in_bytes)
        dt = time.time() - start
        speed = session / dt if dt > 0 else 0.0
        prog[f.path] = RepoFileDownloadProgress(
            repo_id=str(model_id), repo_revision=revision, file_path=f.path, downloaded=Memory.from_bytes(cur),
            downloaded_this_session=Memory.from_bytes(session), total=Memory.from_bytes(tot), speed=speed,
            eta=timedelta(seconds=(tot - cur) / speed) if speed > 0 else timedelta(0),
            status="complete" if cur == tot and renamed else "in_progress", start_time=start)
        await on_progress(shard, repo_progress(shard, revision, prog, t0))

    def schedule(f: FileListEntry, cur: int, tot: int, renamed: bool) -> None:
        t = asyncio.get_running_loop().create_task(report(f, cur, tot, renamed))
        pending.add(t)
        t.add_done_callback(pending.discard)

    sem = asyncio.Semaphore(max_parallel_downloads)

    async def fetch(f: FileListEntry) -> None:
        async with sem:
            await hf.download_file_with_retry(str(model_id), revision, f.path, target,
                                              lambda c, t, r, f=f: schedule(f, c, t, r), on_connection_lost, skip_internet)

    if not skip_download:
        await asyncio.gather(*(fetch(f) for f in files))
        if pending:
            await asyncio.gather(*list(pending), return_exceptions=True)
    final = repo_progress(shard, revision, prog, t0)
    await on_progress(shard, final)
    gguf = next((f for f in files if f.path.endswith(".gguf")), None)
    return (target / gguf.path if gguf else target), final


def full_shard(card: ModelCard) -> PipelineShardMetadata:
    return PipelineShardMetadata(model_card=card, device_rank=0, world_size=1, start_layer=0, end_layer=card.n_layers,
                                 n_layers=card.n_layers)


class ShardDownloader(ABC):
    @abstractmethod
    async def ensure_shard(self, shard: ShardMetadata, config_only: bool = False) -> Path: ...

    @abstractmethod
    def on_progress(self, callback: ProgressCallback) -> None: ...

    @abstractmethod
    def get_shard_download_status(self) -> AsyncIterator[tuple[Path, RepoDownloadProgress]]: ...

    @abstractmethod
    async def get_shard_download_status_for_shard(self, shard: ShardMetadata) -> RepoDownloadProgress: ...


def _empty_progress(shard: ShardMetadata, status: Status = "complete") -> RepoDownloadProgress:
    return RepoDownloadProgress(repo_id=str(shard.model_card.model_id), repo_revision="main", shard=shard, completed_files=0,
                                total_files=0, downloaded=Memory(), downloaded_this_session=Memory(), total=Memory(),
                                overall_speed=0.0, overall_eta=timedelta(0), status=status)


class NoopShardDownloader(ShardDownloader):
    """For nodes started with downloads disabled: everything is reported as already present."""

    async def ensure_shard(self, shard: ShardMetadata, config_only: bool = False) -> Path:
        return Path("/tmp/noop_shard")

    def on_progress(self, callback: ProgressCallback) -> None:
        pass

    async def get_shard_download_status(self) -> AsyncIterator[tuple[Path, RepoDownloadProgress]]:
        return
        yield  # pragma: no cover

    async def get_shard_download_status_for_shard(self, shard: ShardMetadata) -> RepoDownloadProgress:
        return _empty_progress(shard)


class ResumableShardDownloader(ShardDownloader):
    def __init__(self, max_parallel_downloads: int = 8, offline: bool = False):
        self.max_parallel_downloads, self.offline = max_parallel_downloads, offline
        self.callbacks: list[ProgressCallback] = []
        self.internet_ok = not offline

    def on_progress(self, callback: ProgressCallback) -> None:
        self.callbacks.append(callback)

    async def _fan_out(self, shard: ShardMetadata, p: RepoDownloadProgress) -> None:
        for cb in self.callbacks:
            await cb(shard, p)

    def _lost(self) -> None:
        self.internet_ok = False

    def _vision_shard(self, shard: ShardMetadata) -> ShardMetadata | None:
        v = shard.model_card.vision
        if v is None or v.weights_repo == str(shard.model_card.model_id):
            return None
        card = shard.model_card.model_copy(update={"model_id": ModelId(v.weights_repo), "vision": None})
        return full_shard(card)

    async def ensure_shard(self, shard: ShardMetadata, config_only: bool = False) -> Path:
        patterns = ["config.json"] if config_only else None
        path, _ = await download_shard(shard, self._fan_out, max_parallel_downloads=self.max_parallel_downloads,
                                       skip_internet=self.offline, allow_patterns=patterns, on_connection_lost=self._lost)
        vis = self._vision_shard(shard)
        if vis is not None and not config_only:   # encoder weights live in a sibling repo; progress is the main repo's
            async def quiet(_s: ShardMetadata, _p: RepoDownloadProgress) -> None:
                return None
            await download_shard(vis, quiet, max_parallel_downloads=self.max_parallel_downloads,
                                 skip_internet=self.offline, on_connection_lost=self._lost)
        return path

    async def get_shard_download_status_for_shard(self, shard: ShardMetadata) -> RepoDownloadProgress:
        async def quiet(_s: ShardMetadata, _p: RepoDownloadProgress) -> None:
            return None
        _, p = await download_shard(shard, quiet, skip_download=True, skip_internet=self.offline or not self.internet_ok,
                                    on_connection_lost=self._lost)
        return p

    async def get_shard_download_status(self) -> AsyncIterator[tuple[Path, RepoDownloadProgress]]:
        """Status of every known model that has anything on disk (a cheap local scan, no hub traffic)."""
        for card in card_cache.list_all():
            norm = ModelId(card.model_id).normalize()
            if not any((root / norm).is_dir() for root in constants.models_dirs()):
                continue
            try:
                async def quiet(_s: ShardMetadata, _p: RepoDownloadProgress) -> None:
                    return None
                path, p = await download_shard(full_shard(card), quiet, skip_download=True, skip_internet=True)
                yield path, p
            except Exception:
                continue


class SingletonShardDownloader(ShardDownloader):
    """At most one download per shard at a time: concurrent callers await the same task."""

    def __init__(self, inner: ShardDownloader):
        self.inner = inner
        self.active: dict[tuple[str, bool], asyncio.Task[Path]] = {}

    def on_progress(self, callback: ProgressCallback) -> None:
        self.inner.on_progress(callback)

    async def ensure_shard(self, shard: ShardMetadata, config_only: bool = False) -> Path:
        key = (shard.model_dump_json(), config_only)
        if key not in self.active:
            self.active[key] = asyncio.get_running_loop().create_task(self.inner.ensure_shard(shard, config_only))
        try:
            return await asyncio.shield(self.active[key])
        finally:
            t = self.active.get(key)
            if t is not None and t.done():
                self.active.pop(key, None)

    def get_shard_download_status(self) -> AsyncIterator[tuple[Path, RepoDownloadProgress]]:
        return self.inner.get_shard_download_status()

    async def get_shard_download_status_for_shard(self, shard: ShardMetadata) -> RepoDownloadProgress:
        return await self.inner.get_shard_download_status_for_shard(shard)


def exo_shard_downloader(max_parallel_downloads: int = 8, offline: bool = False) -> ShardDownloader:
    return SingletonShardDownloader(ResumableShardDownloader(max_parallel_downloads, offline))
