"""Per-node download coordinator: executes download commands and publishes progress events.

Behaviour of the reference's ``DownloadCoordinator`` (``src/exo/download/coordinator.py:50-475``):
commands addressed to other nodes are ignored; ``StartDownload`` is idempotent while a download is
ongoing, complete or failed; a complete copy anywhere on disk short-circuits to
``DownloadCompleted`` (marked read-only when it sits under a read-only root); offline mode turns a
missing model into ``DownloadFailed``; progress events are throttled to one per second per model;
``CancelDownload`` parks the model as ``DownloadPending`` keeping the byte counts;
``DeleteDownload`` refuses read-only models, cancels an active download, removes the files and
resets the state to pending; every minute what is on disk is re-announced so a restarted master
learns it.
"""
from __future__ import annotations

import time
from pathlib import Path

import anyio

from ..shared import constants
from ..shared.base import Memory, ModelId, NodeId
from ..shared.cards import card_cache
from ..shared.events import Event, NodeDownloadProgress
from ..shared.messages import CancelDownload, DeleteDownload, ForwarderDownloadCommand, StartDownload
from ..shared.wire import (DownloadCompleted, DownloadFailed, DownloadOngoing, DownloadPending, DownloadProgress,
                           ShardMetadata)
from ..utils.async_process import TaskGroup
from ..utils.channels import ChannelClosed, Receiver, Sender
from .shard_downloader import RepoDownloadProgress, ShardDownloader, full_shard, progress_data
from .store import delete_model, is_read_only_model_dir, resolve_existing_model

PROGRESS_INTERVAL_S = 1.0
RESCAN_INTERVAL_S = 60.0


class DownloadCoordinator:
    def __init__(self, node_id: NodeId, shard_downloader: ShardDownloader,
                 download_command_receiver: Receiver[ForwarderDownloadCommand], event_sender: Sender[Event],
                 offline: bool = False):
        self.node_id, self.downloader, self.offline = node_id, shard_downloader, offline
        self.commands, self.events = download_command_receiver, event_sender
        self.download_status: dict[ModelId, DownloadProgress] = {}
        self.active_downloads: dict[ModelId, anyio.CancelScope] = {}
        self._last_progress: dict[ModelId, float] = {}
        self._tg = TaskGroup()
        self._stopped = anyio.Event()
        self.downloader.on_progress(self._on_progress)

    # ---- helpers ----
    @staticmethod
    def _default_dir(model_id: ModelId) -> str:
        return str(constants.EXO_DEFAULT_MODELS_DIR / ModelId(model_id).normalize())

    def _completed(self, shard: ShardMetadata, total: Memory, found: Path | None) -> DownloadCompleted:
        if found is not None:
            return DownloadCompleted(shard_metadata=shard, node_id=self.node_id, total=total, model_directory=str(found),
                                     read_only=is_read_only_model_dir(found))
        return DownloadCompleted(shard_metadata=shard, node_id=self.node_id, total=total,
                                 model_directory=self._default_dir(shard.model_card.model_id))

    async def _set(self, model_id: ModelId, status: DownloadProgress, keep: bool = True) -> None:
        if keep:
            self.download_status[model_id] = status
        try:
            await self.events.send(NodeDownloadProgress(download_progress=status))
        except ChannelClosed:
            pass

    async def _find(self, shard: ShardMetadata) -> Path | None:
        return await anyio.to_thread.run_sync(resolve_existing_model, shard.model_card.model_id, shard.model_card)

    # ---- progress from the downloader ----
    async def _on_progress(self, shard: ShardMetadata, p: RepoDownloadProgress) -> None:
        mid = shard.model_card.model_id
        if p.status == "complete":
            await self._set(mid, self._completed(shard, p.total, await self._find(shard)))
            self._last_progress.pop(mid, None)
        elif p.status == "in_progress" and time.monotonic() - self._last_progress.get(mid, -1e9) > PROGRESS_INTERVAL_S:
            self._last_progress[mid] = time.monotonic()
            await self._set(mid, DownloadOngoing(node_id=self.node_id, shard_metadata=shard, download_progress=progress_data(p),
                                                 model_directory=self._default_dir(mid)))

    # ---- commands ----
    async def _start(self, shard: ShardMetadata) -> None:
        mid = shard.model_card.model_id
        if isinstance(self.download_status.get(mid), (DownloadOngoing, DownloadCompleted, DownloadFailed)):
            return
        found = await self._find(shard)
        if found is not None:
            await self._set(mid, self._completed(shard, shard.model_card.storage_size, found))
            return
        await self._set(mid, DownloadPending(shard_metadata=shard, node_id=self.node_id, model_directory=self._default_dir(mid)))
        try:
            initial = await self.downloader.get_shard_download_status_for_shard(shard)
        except Exception as e:  # noqa: BLE001 - e.g. a gated repo: report, keep serving commands
            await self._set(mid, DownloadFailed(shard_metadata=shard, node_id=self.node_id, error_message=str(e),
                                                model_directory=self._default_dir(mid)))
            return
        if initial.status == "complete" and initial.total_files > 0:
            await self._set(mid, self._completed(shard, initial.total, await self._find(shard)))
            return
        if self.offline:
            await self._set(mid, DownloadFailed(shard_metadata=shard, node_id=self.node_id, model_directory=self._default_dir(mid),
                                                error_message=f"Model files not found locally in offline mode: {mid}"))
            return
        await self._set(mid, DownloadOngoing(node_id=self.node_id, shard_metadata=shard, download_progress=progress_data(initial),
                                             model_directory=self._default_dir(mid)))
        scope = anyio.CancelScope()
        self.active_downloads[mid] = scope
        self._tg.start_soon(self._download, shard, scope)

    async def _download(self, shard: ShardMetadata, scope: anyio.CancelScope) -> None:
        mid = shard.model_card.model_id
        try:
            with scope:
                await self.downloader.ensure_shard(shard)
        except Exception as e:  # noqa: BLE001 - any failure becomes a DownloadFailed event
            await self._set(mid, DownloadFailed(shard_metadata=shard, node_id=self.node_id, error_message=str(e),
                                                model_directory=self._default_dir(mid)))
        finally:
            self.active_downloads.pop(mid, None)

    async def _cancel(self, model_id: ModelId) -> None:
        if model_id not in self.active_downloads or model_id not in self.download_status:
            return
        self.active_downloads[model_id].cancel()
        cur = self.download_status[model_id]
        done, total = Memory(), Memory()
        if isinstance(cur, DownloadOngoing):
            done, total = cur.download_progress.downloaded, cur.download_progress.total
        await self._set(model_id, DownloadPending(shard_metadata=cur.shard_metadata, node_id=self.node_id,
                                                  model_directory=self._default_dir(model_id), downloaded=done, total=total))

    async def _delete(self, model_id: ModelId) -> None:
        cur = self.download_status.get(model_id)
        if isinstance(cur, DownloadCompleted) and cur.read_only:
            return
        if model_id in self.active_downloads:
            self.active_downloads[model_id].cancel()
        await anyio.to_thread.run_sync(delete_model, model_id)
        if cur is not None:
            await self._set(model_id, DownloadPending(shard_metadata=cur.shard_metadata, node_id=self.node_id,
                                                      model_directory=self._default_dir(model_id)), keep=False)
            del self.download_status[model_id]

    async def _command_processor(self) -> None:
        with self.commands as commands:
            async for fc in commands:
                cmd = fc.command
                if cmd.target_node_id != self.node_id:
                    continue
                if isinstance(cmd, StartDownload):
                    await self._start(cmd.shard_metadata)
                elif isinstance(cmd, DeleteDownload):
                    await self._delete(cmd.model_id)
                elif isinstance(cmd, CancelDownload):
                    await self._cancel(cmd.model_id)

    # ---- periodic re-announcement of what is on disk ----
    async def rescan_once(self) -> None:
        async for _path, p in self.downloader.get_shard_download_status():
            mid = p.shard.model_card.model_id
            if mid in self.active_downloads:
                continue
            found = await self._find(p.shard)
            if found is not None:
                status: DownloadProgress = self._completed(p.shard, p.total, found)
            elif isinstance(self.download_status.get(mid), DownloadCompleted):
                continue
            elif p.downloaded_this_session.in_bytes == 0:
                status = DownloadPending(node_id=self.node_id, shard_metadata=p.shard, model_directory=self._default_dir(mid),
                                         downloaded=p.downloaded, total=p.total)
            else:
                status = DownloadOngoing(node_id=self.node_id, shard_metadata=p.shard, download_progress=progress_data(p),
                                         model_directory=self._default_dir(mid))
            await self._set(mid, status)
        if constants.EXO_MODELS_READ_ONLY_DIRS:
            for card in card_cache.list_all():
                mid = card.model_id
                if mid in self.active_downloads or isinstance(self.download_status.get(mid),
                                                              (DownloadCompleted, DownloadOngoing, DownloadFailed)):
                    continue
                found = await anyio.to_thread.run_sync(resolve_existing_model, mid, card)
                if found is not None and is_read_only_model_dir(found):
                    await self._set(mid, self._completed(full_shard(card), card.storage_size, found))

    async def _rescan_loop(self) -> None:
        while True:
            try:
                await self.rescan_once()
            except Exception:  # noqa: BLE001 - a bad directory must not end the loop
                pass
            await anyio.sleep(RESCAN_INTERVAL_S)

    async def run(self) -> None:
        try:
            async with self._tg as tg:
                tg.start_soon(self._command_processor)
                tg.start_soon(self._rescan_loop)
        finally:
            self.commands.close()
            self.events.close()
            self._stopped.set()

    async def shutdown(self) -> None:
        self._tg.cancel_tasks()
        await self._stopped.wait()
