"""Download subsystem against a fake hub on 127.0.0.1: listing, resume, verification, retries, coordinator."""
import asyncio
import hashlib
import json

import anyio
import pytest
from aiohttp import web

from exo_b200.download import hf, store
from exo_b200.download.coordinator import DownloadCoordinator
from exo_b200.download.shard_downloader import (ResumableShardDownloader, SingletonShardDownloader, download_shard,
                                                full_shard)
from exo_b200.shared import constants
from exo_b200.shared.base import Memory, ModelId, NodeId
from exo_b200.shared.cards import ModelCard
from exo_b200.shared.events import NodeDownloadProgress
from exo_b200.shared.messages import (CancelDownload, DeleteDownload, ForwarderDownloadCommand, StartDownload)
from exo_b200.shared.wire import DownloadCompleted, DownloadFailed, DownloadOngoing, DownloadPending
from exo_b200.utils.channels import channel

REPO = "org/tiny"
FILES = {
    "config.json": json.dumps({"model_type": "llama"}).encode(),
    "model.safetensors.index.json": json.dumps({"weight_map": {"model.layers.0.w": "model-00001.safetensors",
                                                               "lm_head": "model-00002.safetensors"}}).encode(),
    "model-00001.safetensors": bytes(range(256)) * 4096,     # 1 MiB, "LFS" (sha256 etag)
    "model-00002.safetensors": b"\x07" * 300_000,
    "original/consolidated.pth": b"never fetched",
}


def git_blob_sha1(b: bytes) -> str:
    return hashlib.sha1(f"blob {len(b)}\0".encode() + b).hexdigest()


class FakeHub:
    def __init__(self):
        self.calls = {"tree": 0, "head": 0, "get": 0, "ranges": []}
        self.fail_gets = 0          # next N GETs answer 500
        self.rate_limit_gets = 0    # next N GETs answer 429 with Retry-After: 0
        self.auth = None            # 401 / 403 on everything
        self.corrupt = set()
        self.truncate_once = set()  # serve only half the body once (connection "drops")

    def app(self):
        a = web.Application()
        a.router.add_get("/api/models/{org}/{name}/tree/{rev}", self.tree)
        a.router.add_route("*", "/{org}/{name}/resolve/{rev}/{path:.*}", self.resolve)
        return a

    async def tree(self, req):
        self.calls["tree"] += 1
        if self.auth:
            return web.Response(status=self.auth)
        return web.json_response([{"type": "file", "path": p, "size": len(b)} for p, b in FILES.items()]
                                 + [{"type": "directory", "path": "original"}])

    async def resolve(self, req):
        path = req.match_info["path"]
        self.calls["resolve"] = self.calls.get("resolve", 0) + 1
        if self.auth:
            return web.Response(status=self.auth)
        if path not in FILES:
            return web.Response(status=404)
        body = FILES[path]
        lfs = path.endswith(".safetensors")
        etag = hashlib.sha256(body).hexdigest() if lfs else git_blob_sha1(body)
        if req.method == "HEAD":
            self.calls["head"] += 1
            return web.Response(status=200, headers={"ETag": f'"{etag}"', "x-linked-size": str(len(body)), "Content-Length": str(len(body))})
        self.calls["get"] += 1
        if self.rate_limit_gets:
            self.rate_limit_gets -= 1
            return web.Response(status=429, headers={"Retry-After": "0"})
        if self.fail_gets:
            self.fail_gets -= 1
            return web.Response(status=500)
        start = 0
        rng = req.headers.get("Range")
        if rng:
            start = int(rng.split("=")[1].split("-")[0])
            self.calls["ranges"].append((path, start))
        data = body[start:]
        if path in self.corrupt:
            data = b"\x00" * len(data)
        if path in self.truncate_once:
            self.truncate_once.discard(path)
            resp = web.StreamResponse(status=206 if rng else 200, headers={"Content-Length": str(len(data))})
            await resp.prepare(req)
            await resp.write(data[: len(data) // 2])
            req.transport.close()
            return resp
        return web.Response(status=206 if rng else 200, body=data)


@pytest.fixture
def env(tmp_path, monkeypatch):
    rw, ro = tmp_path / "models", tmp_path / "ro"
    rw.mkdir(); ro.mkdir()
    monkeypatch.setattr(constants, "EXO_DEFAULT_MODELS_DIR", rw)
    monkeypatch.setattr(constants, "EXO_MODELS_DIRS", (rw,))
    monkeypatch.setattr(constants, "EXO_MODELS_READ_ONLY_DIRS", (ro,))
    monkeypatch.setattr(hf, "BACKOFF_SCALE_S", 0.01)
    monkeypatch.delenv("HF_TOKEN", raising=False)
    monkeypatch.setenv("HF_HOME", str(tmp_path / "hfhome"))
    return rw, ro


def card(model_id=REPO):
    return ModelCard(model_id=ModelId(model_id), storage_size=Memory.from_bytes(sum(map(len, FILES.values()))), n_layers=2,
                     hidden_size=64, supports_tensor=True, tasks=["TextGeneration"])


async def with_hub(fn, monkeypatch):
    hub = FakeHub()
    runner = web.AppRunner(hub.app())
    await runner.setup()
    site = web.TCPSite(runner, "127.0.0.1", 0)
    await site.start()
    port = site._server.sockets[0].getsockname()[1]
    monkeypatch.setenv("HF_ENDPOINT", f"http://127.0.0.1:{port}")
    try:
        return await fn(hub)
    finally:
        await runner.cleanup()


def test_download_shard_verifies_resumes_and_skips_ignored(env, monkeypatch):
    rw, _ = env

    async def body(hub):
        seen = []

        async def on_progress(shard, p):
            seen.append(p)
        target = rw / "org--tiny"
        target.mkdir()
        big = FILES["model-00001.safetensors"]
        (target / "model-00001.safetensors.partial").write_bytes(big[:400_000])      # an interrupted earlier run
        path, final = await download_shard(full_shard(card()), on_progress)
        assert path == target and final.status == "complete" and final.completed_files == final.total_files == 4
        assert ("model-00001.safetensors", 400_000) in hub.calls["ranges"]
        for name, b in FILES.items():
            if name.startswith("original/"):
                assert not (target / name).exists()
            else:
                assert (target / name).read_bytes() == b
        assert not list(target.glob("*.partial"))
        assert final.downloaded_this_session.in_bytes == final.total.in_bytes - 400_000
        assert any(p.status == "in_progress" for p in seen) and seen[-1].status == "complete"
        assert store.is_model_directory_complete(target) and store.resolve_existing_model(ModelId(REPO)) == target
        # second run: nothing is fetched again (sizes match on HEAD)
        gets = hub.calls["get"]
        await download_shard(full_shard(card()), on_progress)
        assert hub.calls["get"] == gets
    asyncio.run(with_hub(body, monkeypatch))


def test_retry_rate_limit_hash_mismatch_and_auth(env, monkeypatch):
    rw, _ = env

    async def body(hub):
        async def quiet(s, p):
            pass
        hub.fail_gets, hub.rate_limit_gets = 2, 1
        hub.truncate_once = {"model-00002.safetensors"}
        _, final = await download_shard(full_shard(card()), quiet, max_parallel_downloads=1)
        assert final.status == "complete"
        assert any(p == "model-00002.safetensors" and s > 0 for p, s in hub.calls["ranges"])   # resumed after the drop
        # corrupted body: hash check fails on every attempt, the partial file is removed
        store.delete_model(ModelId(REPO))
        hub.corrupt = {"config.json"}
        with pytest.raises(RuntimeError, match="remote hash"):
            await download_shard(full_shard(card()), quiet)
        assert not (rw / "org--tiny" / "config.json").exists() and not (rw / "org--tiny" / "config.json.partial").exists()
        # 401 without a token names HF_TOKEN and is not retried
        hub.corrupt, hub.auth = set(), 401
        store.delete_model(ModelId(REPO))
        hits = hub.calls["resolve"]
        with pytest.raises(hf.HuggingFaceAuthenticationError, match="HF_TOKEN"):
            await hf.download_file_with_retry(REPO, "main", "config.json", rw / "org--tiny")
        assert hub.calls["resolve"] == hits + 1
    asyncio.run(with_hub(body, monkeypatch))


def test_file_list_cache_offline_and_local_fallback(env, monkeypatch):
    rw, _ = env

    async def body(hub):
        a = await hf.fetch_file_list_with_cache(ModelId(REPO))
        b = await hf.fetch_file_list_with_cache(ModelId(REPO))
        assert hub.calls["tree"] == 1 and [f.path for f in a] == [f.path for f in b] and len(a) == 5
        with pytest.raises(FileNotFoundError):
            await hf.fetch_file_list_with_cache(ModelId("org/unknown"), skip_internet=True)
        d = rw / "org--local"
        d.mkdir()
        (d / "config.json").write_text("{}")
        (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "m-1.safetensors", "b": "m-2.safetensors"}}))
        (d / "m-1.safetensors").write_bytes(b"x")
        got = await hf.fetch_file_list_with_cache(ModelId("org/local"), skip_internet=True)
        assert {f.path: f.size for f in got}["m-2.safetensors"] is None
        assert not store.is_model_directory_complete(d)
        (d / "m-2.safetensors").write_bytes(b"y")
        assert store.is_model_directory_complete(d)
    asyncio.run(with_hub(body, monkeypatch))


def test_helpers():
    assert hf.trim_etag('W/"abc-gzip"') == "abc" and hf.trim_etag('"abc"') == "abc"
    assert hf.parse_retry_after({"Retry-After": "7"}) == 7.0 and hf.parse_retry_after({"RateLimit": '"api";r=0;t=42'}) == 42.0
    assert hf.parse_retry_after({}) is None
    got = list(hf.filter_repo_objects(["a.json", "original/x.pth", "w/model.safetensors", "metal/k.metallib"],
                                      allow_patterns=["*"], ignore_patterns=["original/*", "metal/"]))
    assert got == ["a.json", "w/model.safetensors"]
    wm = {"model.layers.0.a": "f0", "model.layers.1.a": "f1", "model.layers.2.a": "f2", "model.norm": "f3"}
    pats = hf.allow_patterns_for_layers(wm, 1, 2)
    assert "f1" in pats and "f3" in pats and "f0" not in pats and "f2" not in pats and "*.json" in pats


def _coordinator(offline=False):
    cmd_s, cmd_r = channel()
    ev_s, ev_r = channel()
    node = NodeId("me")
    dc = DownloadCoordinator(node, SingletonShardDownloader(ResumableShardDownloader(offline=offline)), cmd_r, ev_s, offline=offline)
    return dc, cmd_s, ev_r, node


def test_coordinator_start_complete_delete_and_read_only(env, monkeypatch):
    rw, ro = env

    async def body(hub):
        dc, cmd_s, ev_r, node = _coordinator()
        shard = full_shard(card())
        async with anyio.create_task_group() as tg:
            tg.start_soon(dc.run)
            await cmd_s.send(ForwarderDownloadCommand(origin="x", command=StartDownload(target_node_id=NodeId("other"), shard_metadata=shard)))
            await cmd_s.send(ForwarderDownloadCommand(origin="x", command=StartDownload(target_node_id=node, shard_metadata=shard)))
            with anyio.fail_after(20):
                while not isinstance(dc.download_status.get(ModelId(REPO)), DownloadCompleted):
                    await anyio.sleep(0.02)
            kinds = [type(e.download_progress).__name__ for e in ev_r.collect() if isinstance(e, NodeDownloadProgress)
                     and e.download_progress.shard_metadata.model_card.model_id == REPO]
            assert kinds[0] == "DownloadPending" and "DownloadOngoing" in kinds and kinds[-1] == "DownloadCompleted"
            done = dc.download_status[ModelId(REPO)]
            assert done.model_directory == str(rw / "org--tiny") and not done.read_only
            # idempotent
            gets = hub.calls["get"]
            await cmd_s.send(ForwarderDownloadCommand(origin="x", command=StartDownload(target_node_id=node, shard_metadata=shard)))
            await anyio.sleep(0.1)
            assert hub.calls["get"] == gets
            # delete resets to pending and removes the files
            await cmd_s.send(ForwarderDownloadCommand(origin="x", command=DeleteDownload(target_node_id=node, model_id=ModelId(REPO))))
            with anyio.fail_after(30):
                while ModelId(REPO) in dc.download_status:
                    await anyio.sleep(0.02)
            assert not (rw / "org--tiny").exists()
            assert isinstance(ev_r.collect()[-1].download_progress, DownloadPending)
            # a read-only copy is found without any download and is never deleted
            rod = ro / "org--ro"
            rod.mkdir()
            (rod / "config.json").write_text("{}")
            (rod / "model.safetensors").write_bytes(b"w")
            ro_shard = full_shard(card("org/ro"))
            gets = hub.calls["get"]
            await cmd_s.send(ForwarderDownloadCommand(origin="x", command=StartDownload(target_node_id=node, shard_metadata=ro_shard)))
            with anyio.fail_after(30):
                while not isinstance(dc.download_status.get(ModelId("org/ro")), DownloadCompleted):
                    await anyio.sleep(0.02)
            assert dc.download_status[ModelId("org/ro")].read_only and hub.calls["get"] == gets
            await cmd_s.send(ForwarderDownloadCommand(origin="x", command=DeleteDownload(target_node_id=node, model_id=ModelId("org/ro"))))
            await anyio.sleep(0.1)
            assert rod.exists() and ModelId("org/ro") in dc.download_status
            tg.cancel_scope.cancel()
    asyncio.run(with_hub(body, monkeypatch))


def test_coordinator_offline_fails_and_hub_error_becomes_failed(env, monkeypatch):
    async def body(hub):
        dc, cmd_s, ev_r, node = _coordinator(offline=True)
        shard = full_shard(card())
        async with anyio.create_task_group() as tg:
            tg.start_soon(dc.run)
            await cmd_s.send(ForwarderDownloadCommand(origin="x", command=StartDownload(target_node_id=node, shard_metadata=shard)))
            with anyio.fail_after(30):
                while not isinstance(dc.download_status.get(ModelId(REPO)), DownloadFailed):
                    await anyio.sleep(0.02)
            assert "offline mode" in dc.download_status[ModelId(REPO)].error_message and hub.calls["tree"] == 0
            tg.cancel_scope.cancel()
        dc, cmd_s, ev_r, node = _coordinator()
        hub.auth = 403
        async with anyio.create_task_group() as tg:
            tg.start_soon(dc.run)
            await cmd_s.send(ForwarderDownloadCommand(origin="x", command=StartDownload(target_node_id=node, shard_metadata=shard)))
            with anyio.fail_after(30):
                while not isinstance(dc.download_status.get(ModelId(REPO)), DownloadFailed):
                    await anyio.sleep(0.02)
            assert "Access denied" in dc.download_status[ModelId(REPO)].error_message
            tg.cancel_scope.cancel()
    asyncio.run(with_hub(body, monkeypatch))
