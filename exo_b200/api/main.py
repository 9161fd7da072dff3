"""The HTTP API of a node: OpenAI / Claude / Responses / Ollama dialects, cluster control, state.

Route table and semantics follow the reference server (``src/exo/api/main.py:343-409`` and the
handlers below it): the API keeps its own fold of the global event stream, sends commands to the
master and routes ``ChunkGenerated`` events into per-command queues; a request that is
disconnected sends ``TaskCancelled`` and every request ends with ``TaskFinished``; while an
election is in progress commands are held back until the new master is known.  Served by uvicorn
on one asyncio loop shared with the rest of the node.
"""
from __future__ import annotations

import base64
import contextlib
import hashlib
import json
import time
from collections.abc import AsyncIterator
from datetime import datetime, timezone
from http import HTTPStatus
from pathlib import Path
from typing import Annotated, Any, Literal

import anyio
from fastapi import FastAPI, File, Form, HTTPException, Query, Request, UploadFile
from fastapi.middleware.cors import CORSMiddleware
from fastapi.responses import FileResponse, JSONResponse, Response, StreamingResponse
from fastapi.staticfiles import StaticFiles

from ..master.image_store import ImageStore
from ..master.placement import memory_delta_by_node, place_instance
from ..shared import constants, tracing
from ..shared.base import CommandId, InstanceId, InstanceLinkId, Memory, ModelId, NodeId, SystemId
from ..shared.cards import ModelCard, ModelTask, card_cache, card_from_local_dir, load_card
from ..shared.election import ElectionMessage
from ..shared.events import ChunkGenerated, IndexedEvent, InstanceDeleted, State, TracesMerged, apply
from ..shared.messages import (AddCustomModelCard, CancelDownload, Command, CreateInstance, DeleteCustomModelCard,
                               DeleteDownload, DeleteInstance, DeleteInstanceLink, ForwarderCommand,
                               ForwarderDownloadCommand, ImageEdits, ImageEditsCommand, ImageGeneration,
                               ImageGenerationCommand, PlaceInstance, SendInputChunk, SetInstanceLink, StartDownload,
                               TaskCancelled, TaskFinished, TextGeneration, TextGenerationCommand,
                               TextGenerationTaskParams)
from ..shared.wire import (DownloadCompleted, ErrorChunk, ImageChunk, Instance, InstanceLink, InstanceMeta,
                           InputImageChunk, Sharding)
from ..utils.async_process import TaskGroup
from ..utils.buffers import DiskEventLog
from ..utils.channels import ChannelClosed, Receiver, Sender, channel
from ..utils.power_sampler import PowerSampler
from . import types as T
from .dialects import claude, common, ollama, openai_chat, responses
from .dialects.common import GenerationError, TextChunk, Turn, collect, drive, with_sse_keepalive

API_EVENT_LOG_DIR = constants.EXO_EVENT_LOG_DIR / "api"
ONBOARDING_FILE = constants.EXO_CONFIG_HOME / "onboarding_complete"
GENERATION_TASKS = (TextGeneration, ImageGeneration, ImageEdits)


def _sse_response(gen: AsyncIterator[str], media_type: str = "text/event-stream") -> StreamingResponse:
    return StreamingResponse(gen, media_type=media_type, headers=common.SSE_HEADERS)


def _ensure_seed(p: T.AdvancedImageParams | None) -> T.AdvancedImageParams:
    """Every rank of an image instance must draw the same noise: fix the seed at the API."""
    import random
    p = p or T.AdvancedImageParams()
    return p if p.seed is not None else p.model_copy(update={"seed": random.randint(0, 2 ** 32 - 1)})


class API:
    def __init__(self, node_id: NodeId, *, port: int, event_receiver: Receiver[IndexedEvent],
                 command_sender: Sender[ForwarderCommand], download_command_sender: Sender[ForwarderDownloadCommand],
                 election_receiver: Receiver[ElectionMessage], host: str = "0.0.0.0",
                 event_log_dir: Path | None = None):
        self.node_id, self.port, self.host = node_id, port, host
        self.state = State()
        self._event_log_dir = event_log_dir or API_EVENT_LOG_DIR
        self._event_log = DiskEventLog(self._event_log_dir)
        self._system_id = SystemId()
        self.command_sender, self.download_command_sender = command_sender, download_command_sender
        self.event_receiver, self.election_receiver = event_receiver, election_receiver
        self.last_completed_election = 0
        self.paused = False
        self.paused_ev = anyio.Event()
        self._sent_image_hashes: set[str] = set()
        self._text_queues: dict[CommandId, Sender[TextChunk]] = {}
        self._image_queues: dict[CommandId, Sender[ImageChunk | ErrorChunk]] = {}
        self._text_recv: dict[CommandId, Receiver[TextChunk]] = {}
        self._image_recv: dict[CommandId, Receiver[ImageChunk | ErrorChunk]] = {}
        self._image_store = ImageStore(constants.EXO_IMAGE_CACHE_DIR)
        self._tg = TaskGroup()
        self.server = None
        self.app = FastAPI(title="exo")
        self.app.exception_handler(HTTPException)(self._http_error)
        self.app.add_middleware(CORSMiddleware, allow_origins=["*"], allow_credentials=True, allow_methods=["*"], allow_headers=["*"])
        self._routes()
        if constants.DASHBOARD_DIR.is_dir():
            self.app.mount("/", StaticFiles(directory=constants.DASHBOARD_DIR, html=True), name="dashboard")

    # ---- election pauses ----
    def reset(self, result_clock: int, event_receiver: Receiver[IndexedEvent]) -> None:
        self._event_log.close()
        self._event_log = DiskEventLog(self._event_log_dir)
        self.state = State()
        self._system_id = SystemId()
        self._text_queues, self._image_queues = {}, {}
        self._sent_image_hashes = set()
        self.unpause(result_clock)
        self.event_receiver.close()
        self.event_receiver = event_receiver
        self._tg.start_soon(self._apply_state)

    def unpause(self, result_clock: int) -> None:
        self.last_completed_election = result_clock
        self.paused = False
        self.paused_ev.set()
        self.paused_ev = anyio.Event()

    async def _pause_on_new_election(self) -> None:
        with self.election_receiver as msgs:
            async for m in msgs:
                if m.clock > self.last_completed_election:
                    self.paused = True

    async def _http_error(self, _req: Request, exc: HTTPException) -> JSONResponse:
        err = T.ErrorResponse(error=T.ErrorInfo(message=str(exc.detail), type=HTTPStatus(exc.status_code).phrase, code=exc.status_code))
        return JSONResponse(err.model_dump(), status_code=exc.status_code)

    def _routes(self) -> None:
        a = self.app
        a.get("/node_id")(lambda: self.node_id)
        a.post("/instance")(self.create_instance)
        a.post("/place_instance")(self.place_instance)
        a.get("/instance/placement")(self.get_placement)
        a.get("/instance/previews")(self.get_placement_previews)
        a.get("/instance/await", response_model=None)(self.await_instance)
        a.get("/instance/{instance_id}")(self.get_instance)
        a.delete("/instance/{instance_id}")(self.delete_instance)
        a.get("/v1/instance-links")(self.list_instance_links)
        a.post("/v1/instance-links")(self.create_instance_link)
        a.put("/v1/instance-links/{link_id}")(self.update_instance_link)
        a.delete("/v1/instance-links/{link_id}")(self.delete_instance_link)
        a.get("/v1/feature-flags")(self.get_feature_flags)
        a.get("/models")(self.get_models)
        a.get("/v1/models")(self.get_models)
        a.post("/models/add")(self.add_custom_model)
        a.delete("/models/custom/{model_id:path}")(self.delete_custom_model)
        a.get("/models/search")(self.search_models)
        a.post("/v1/chat/completions", response_model=None)(self.chat_completions)
        a.post("/bench/chat/completions", response_model=None)(self.bench_chat_completions)
        a.post("/v1/images/generations", response_model=None)(self.image_generations)
        a.post("/bench/images/generations")(self.bench_image_generations)
        a.post("/v1/images/edits", response_model=None)(self.image_edits)
        a.post("/bench/images/edits")(self.bench_image_edits)
        a.get("/images")(self.list_images)
        a.get("/images/{image_id}")(self.get_image)
        a.post("/v1/messages", response_model=None)(self.claude_messages)
        a.post("/v1/responses", response_model=None)(self.openai_responses)
        a.post("/v1/cancel/{command_id}")(self.cancel_command)
        a.get("/ollama/")(self._ollama_root)
        a.head("/ollama/")(self._ollama_root)
        a.post("/ollama/v1/chat/completions", response_model=None)(self.chat_completions)
        for p in ("/ollama/api/chat", "/ollama/api/api/chat", "/ollama/api/v1/chat"):
            a.post(p, response_model=None)(self.ollama_chat)
        a.post("/ollama/api/generate", response_model=None)(self.ollama_generate)
        for p in ("/ollama/api/tags", "/ollama/api/api/tags", "/ollama/api/v1/tags"):
            a.get(p)(self.ollama_tags)
        a.post("/ollama/api/show")(self.ollama_show)
        a.get("/ollama/api/ps")(self.ollama_ps)
        a.get("/ollama/api/version")(self.ollama_version)
        a.get("/state")(self.get_state)
        a.get("/state/{path:path}")(self.get_state)
        a.get("/events")(self.stream_events)
        a.post("/download/start")(self.start_download)
        a.delete("/download/{node_id}/{model_id:path}")(self.delete_download)
        a.post("/download/cancel")(self.cancel_download)
        a.get("/v1/traces")(self.list_traces)
        a.post("/v1/traces/delete")(self.delete_traces)
        a.get("/v1/traces/{task_id}")(self.get_trace)
        a.get("/v1/traces/{task_id}/stats")(self.get_trace_stats)
        a.get("/v1/traces/{task_id}/raw")(self.get_trace_raw)
        a.get("/onboarding")(self.get_onboarding)
        a.post("/onboarding")(self.complete_onboarding)

    # ---- plumbing ----
    async def _send(self, command: Command) -> None:
        while self.paused:
            await self.paused_ev.wait()
        await self.command_sender.send(ForwarderCommand(origin=self._system_id, command=command))

    async def _send_download(self, command) -> None:
        await self.download_command_sender.send(ForwarderDownloadCommand(origin=self._system_id, command=command))

    def _card(self, model_id: str) -> ModelCard:
        c = self.state.custom_model_cards.get(ModelId(model_id))
        return c if c is not None else load_card(model_id)

    def _gpu_index(self) -> dict[NodeId, int]:
        return {n: v.gpu_index for n, v in self.state.node_nvlink.items()}

    def _placements(self, card: ModelCard, sharding: Sharding, meta: InstanceMeta, min_nodes: int,
                    required: set[NodeId] | None = None) -> dict[InstanceId, Instance]:
        st = self.state
        return place_instance(PlaceInstance(model_card=card, sharding=sharding, instance_meta=meta, min_nodes=min_nodes),
                              st.topology, st.instances, st.node_memory, st.node_backends, required_nodes=required,
                              download_status=st.downloads, gpu_index=self._gpu_index(), node_nvlink=st.node_nvlink)

    # ---- state ----
    def get_state(self, path: str = ""):
        if path == "":
            return JSONResponse(json.loads(self.state.model_dump_json()))
        try:
            x: Any = json.loads(self.state.model_dump_json())
            for attr in path.split("/"):
                if attr != "":
                    x = x[int(attr)] if isinstance(x, list) else x[attr]
            return JSONResponse(x)
        except Exception as e:
            raise HTTPException(404, f"unable to find path '{path.replace('/', '.')}' in state json") from e

    def stream_events(self) -> StreamingResponse:
        def gen():
            yield "["
            for i, rec in enumerate(self._event_log.read_all()):
                yield ("," if i else "") + (rec if isinstance(rec, str) else json.dumps(rec))
            yield "]"
        return StreamingResponse(gen(), media_type="application/json")

    # ---- instances ----
    async def place_instance(self, payload: T.PlaceInstanceParams) -> T.CreateInstanceResponse:
        try:
            card = self._card(payload.model_id)
        except KeyError as e:
            raise HTTPException(404, str(e)) from e
        cmd = PlaceInstance(model_card=card, sharding=payload.sharding, instance_meta=payload.instance_meta, min_nodes=payload.min_nodes)
        await self._send(cmd)
        return T.CreateInstanceResponse(message="Command received.", command_id=cmd.command_id, model_card=card)

    def _total_available_memory(self) -> Memory:
        return sum((m.ram_available for m in self.state.node_memory.values()), Memory())

    async def create_instance(self, payload: T.CreateInstanceParams) -> T.CreateInstanceResponse:
        card = self._card(payload.instance.shard_assignments.model_id)
        need, have = card.storage_size, self._total_available_memory()
        if need.in_bytes > have.in_bytes:
            raise HTTPException(400, f"Insufficient memory to create instance. Required: {need.in_gb:.1f}GB, Available: {have.in_gb:.1f}GB")
        cmd = CreateInstance(instance=payload.instance)
        await self._send(cmd)
        return T.CreateInstanceResponse(message="Command received.", command_id=cmd.command_id, model_card=card)

    def _one_new(self, placements: dict[InstanceId, Instance]) -> Instance | None:
        new = [i for k, i in placements.items() if k not in self.state.instances]
        return new[0] if len(new) == 1 else None

    async def get_placement(self, model_id: ModelId, sharding: Sharding = Sharding.Pipeline,
                            instance_meta: InstanceMeta = InstanceMeta.Nvlink, min_nodes: int = 1) -> Instance:
        try:
            placements = self._placements(self._card(model_id), sharding, instance_meta, min_nodes)
        except (ValueError, KeyError) as e:
            raise HTTPException(400, str(e)) from e
        inst = self._one_new(placements)
        if inst is None:
            raise HTTPException(500, "Expected exactly one new instance from placement")
        return inst

    async def get_placement_previews(self, model_id: ModelId,
                                     node_ids: Annotated[list[NodeId] | None, Query()] = None) -> T.PlacementPreviewResponse:
        nodes = list(self.state.topology.list_nodes())
        if not nodes:
            return T.PlacementPreviewResponse(previews=[])
        try:
            card = self._card(model_id)
        except Exception as e:
            raise HTTPException(400, f"Failed to load model card: {e}") from e
        required = set(node_ids) if node_ids else None
        seen: set[tuple[Sharding, InstanceMeta, int]] = set()
        previews: list[T.PlacementPreview] = []

        def add(key, **kw) -> None:
            if key not in seen:
                seen.add(key)
                previews.append(T.PlacementPreview(model_id=card.model_id, sharding=key[0], instance_meta=key[1], **kw))
        for sharding in (Sharding.Pipeline, Sharding.Tensor):
            meta = InstanceMeta.Nvlink
            for n in range(1, len(nodes) + 1):
                try:
                    inst = self._one_new(self._placements(card, sharding, meta, n, required))
                except ValueError as e:
                    add((sharding, meta, 0), error=str(e))
                    continue
                if inst is None:
                    add((sharding, meta, 0), error="Expected exactly one new instance from placement")
                    continue
                add((sharding, meta, len(inst.shard_assignments.node_to_runner)), instance=inst,
                    memory_delta_by_node=memory_delta_by_node(inst) or None)
        return T.PlacementPreviewResponse(previews=previews)

    def get_instance(self, instance_id: InstanceId) -> Instance:
        if instance_id not in self.state.instances:
            raise HTTPException(404, "Instance not found")
        return self.state.instances[instance_id]

    async def await_instance(self, model_id: ModelId, timeout_seconds: float = Query(default=0.0, ge=0.0, le=300.0)) -> StreamingResponse:
        async def gen() -> AsyncIterator[str]:
            deadline = None if timeout_seconds == 0 else anyio.current_time() + timeout_seconds
            while True:
                for inst in self.state.instances.values():
                    if inst.shard_assignments.model_id == model_id:
                        yield common.sse(T.AwaitInstanceReadyMessage(instance=inst).model_dump_json())
                        return
                if deadline is not None and anyio.current_time() >= deadline:
                    yield common.sse(T.AwaitInstanceTimeoutMessage(message=f"No instance found for model {model_id}").model_dump_json())
                    return
                await anyio.sleep(0.1)
        return _sse_response(with_sse_keepalive(gen()))

    async def delete_instance(self, instance_id: InstanceId) -> T.DeleteInstanceResponse:
        if instance_id not in self.state.instances:
            raise HTTPException(404, "Instance not found")
        cmd = DeleteInstance(instance_id=instance_id)
        await self._send(cmd)
        return T.DeleteInstanceResponse(message="Command received.", command_id=cmd.command_id, instance_id=instance_id)

    # ---- instance links (disaggregated prefill) ----
    async def get_feature_flags(self) -> dict[str, bool]:
        return {"disaggregation": constants.ENABLE_DISAGGREGATION}

    @staticmethod
    def _need_disaggregation() -> None:
        if not constants.ENABLE_DISAGGREGATION:
            raise HTTPException(404, "Disaggregation is not enabled (set ENABLE_DISAGGREGATION=true)")

    async def list_instance_links(self) -> list[InstanceLink]:
        return list(self.state.instance_links.values()) if constants.ENABLE_DISAGGREGATION else []

    async def _set_link(self, link_id: InstanceLinkId, body: T.InstanceLinkBody) -> T.InstanceLinkResponse:
        cmd = SetInstanceLink(link_id=link_id, prefill_instances=list(body.prefill_instances), decode_instances=list(body.decode_instances))
        await self._send(cmd)
        return T.InstanceLinkResponse(message="Command received.", command_id=cmd.command_id)

    async def create_instance_link(self, body: T.InstanceLinkBody) -> T.InstanceLinkResponse:
        self._need_disaggregation()
        return await self._set_link(InstanceLinkId(), body)

    async def update_instance_link(self, link_id: InstanceLinkId, body: T.InstanceLinkBody) -> T.InstanceLinkResponse:
        self._need_disaggregation()
        return await self._set_link(link_id, body)

    async def delete_instance_link(self, link_id: InstanceLinkId) -> T.InstanceLinkResponse:
        self._need_disaggregation()
        cmd = DeleteInstanceLink(link_id=link_id)
        await self._send(cmd)
        return T.InstanceLinkResponse(message="Command received.", command_id=cmd.command_id)

    # ---- text generation ----
    async def cancel_command(self, command_id: CommandId) -> T.CancelCommandResponse:
        q = self._text_queues.get(command_id) or self._image_queues.get(command_id)
        if q is None:
            raise HTTPException(404, "Command not found or already completed")
        await self._send(TaskCancelled(cancelled_command_id=command_id))
        q.close()
        return T.CancelCommandResponse(message="Command cancelled.", command_id=command_id)

    async def _chunks(self, command_id: CommandId) -> AsyncIterator[TextChunk]:
        """The chunk stream of one command; cancels the task if the consumer goes away."""
        assert command_id in self._text_queues, "open the queue before sending the command"
        recv: Receiver[TextChunk] = self._text_recv.pop(command_id)
        try:
            with recv as chunks:
                async for ch in chunks:
                    yield ch
                    if getattr(ch, "finish_reason", None) is not None:
                        break
        except (anyio.get_cancelled_exc_class(), GeneratorExit):
            with anyio.CancelScope(shield=True):
                await self.command_sender.send(ForwarderCommand(origin=self._system_id, command=TaskCancelled(cancelled_command_id=command_id)))
            raise
        finally:
            with anyio.CancelScope(shield=True):
                with contextlib.suppress(ChannelClosed):
                    await self.command_sender.send(ForwarderCommand(origin=self._system_id, command=TaskFinished(finished_command_id=command_id)))
            self._text_queues.pop(command_id, None)

    def _open_text_queue(self, command_id: CommandId) -> None:
        self._text_queues[command_id], self._text_recv[command_id] = channel()

    async def _validate_model(self, model_id: str) -> ModelId:
        if not any(i.shard_assignments.model_id == model_id for i in self.state.instances.values()):
            raise HTTPException(404, f"No instance found for model {model_id}")
        return ModelId(model_id)

    async def _submit_text(self, params: TextGenerationTaskParams) -> TextGenerationCommand:
        """Send the command; images travel first, chunked, and only once per content hash."""
        params = params.model_copy(update={"model": await self._validate_model(params.model)}).with_card_sampling_defaults()
        images = params.images
        if images:
            hashes = [hashlib.sha256(i.encode("ascii")).hexdigest() for i in images]
            params = params.model_copy(update={"images": [], "image_hashes": dict(enumerate(hashes))})
        cmd = TextGenerationCommand(task_params=params)
        self._open_text_queue(cmd.command_id)
        if images:
            fresh = [(i, img) for i, (img, h) in enumerate(zip(images, hashes)) if h not in self._sent_image_hashes]
            self._sent_image_hashes.update(hashes)
            pieces = [(i, img[o:o + constants.EXO_MAX_CHUNK_SIZE]) for i, img in fresh for o in range(0, len(img), constants.EXO_MAX_CHUNK_SIZE)]
            for k, (i, data) in enumerate(pieces):
                await self._send(SendInputChunk(chunk=InputImageChunk(model=params.model, command_id=cmd.command_id, data=data,
                                                                      chunk_index=k, total_chunks=len(pieces), image_index=i)))
        await self._send(cmd)
        return cmd

    async def _json_body(self, cid: CommandId, render, model: str = "") -> AsyncIterator[str]:
        # a generator (not a plain return) so a client disconnect cancels the generation
        try:
            yield render(await collect(cid, self._chunks(cid), model))
        except GenerationError as e:
            yield T.ErrorResponse(error=T.ErrorInfo(message=str(e), type="InternalServerError", code=500)).model_dump_json()

    async def _serve_text(self, params: TextGenerationTaskParams, stream: bool, encoder, render, media: str = "text/event-stream",
                          keepalive: bool = True) -> StreamingResponse:
        cmd = await self._submit_text(params)
        cid, model = cmd.command_id, str(cmd.task_params.model)
        if stream:
            gen = drive(cid, self._chunks(cid), encoder, model)
            return _sse_response(with_sse_keepalive(gen) if keepalive else gen, media)
        return StreamingResponse(self._json_body(cid, render, model), media_type="application/json")

    async def chat_completions(self, payload: T.ChatCompletionRequest) -> StreamingResponse:
        params = await openai_chat.to_params(payload)
        return await self._serve_text(params, payload.stream, openai_chat.ChatStreamEncoder(), openai_chat.render)

    async def bench_chat_completions(self, payload: T.BenchChatCompletionRequest):
        params = (await openai_chat.to_params(payload)).model_copy(update={"stream": False, "bench": True, "use_prefix_cache": payload.use_prefix_cache})
        if payload.stream:
            return await self._serve_text(params, True, openai_chat.ChatStreamEncoder(), openai_chat.render)
        cmd = await self._submit_text(params)
        sampler = PowerSampler(lambda: self.state.node_system)
        turn: Turn | None = None

        async def observed() -> AsyncIterator[TextChunk]:
            async for ch in self._chunks(cmd.command_id):
                if not isinstance(ch, common.PrefillProgressChunk):
                    sampler.mark_prefill_done()
                yield ch
        async with anyio.create_task_group() as tg:
            tg.start_soon(sampler.run)
            try:
                turn = await collect(cmd.command_id, observed(), str(cmd.task_params.model))
            except GenerationError as e:
                raise HTTPException(500, str(e)) from e
            finally:
                tg.cancel_scope.cancel()
        return openai_chat.render_bench(turn, sampler.result())

    async def claude_messages(self, payload: claude.MessagesRequest) -> StreamingResponse:
        params = await claude.to_params(payload)
        return await self._serve_text(params, payload.stream, claude.ClaudeStreamEncoder(), claude.render)

    async def openai_responses(self, payload: responses.ResponsesRequest) -> StreamingResponse:
        params = await responses.to_params(payload)
        return await self._serve_text(params, payload.stream, responses.ResponsesStreamEncoder(), responses.render)

    # ---- ollama ----
    async def _ollama_root(self) -> Response:
        return Response("Ollama is running", media_type="text/plain")

    async def ollama_chat(self, request: Request) -> StreamingResponse:
        payload = ollama.ChatRequest.model_validate_json(await request.body())   # clients send no content-type
        return await self._serve_text(ollama.chat_to_params(payload), payload.stream, ollama.OllamaChatEncoder(),
                                      ollama.render_chat, "application/x-ndjson", keepalive=False)

    async def ollama_generate(self, request: Request) -> StreamingResponse:
        payload = ollama.GenerateRequest.model_validate_json(await request.body())
        return await self._serve_text(ollama.generate_to_params(payload), payload.stream, ollama.OllamaGenerateEncoder(),
                                      ollama.render_generate, "application/x-ndjson", keepalive=False)

    def _downloaded_ids(self) -> set[str]:
        return {str(d.shard_metadata.model_card.model_id) for ds in self.state.downloads.values() for d in ds
                if isinstance(d, DownloadCompleted)}

    async def ollama_tags(self) -> ollama.TagsResponse:
        have = self._downloaded_ids()
        now = time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())
        return ollama.TagsResponse(models=[
            ollama.ModelTag(name=str(c.model_id), model=str(c.model_id), modified_at=now, size=c.storage_size.in_bytes,
                            digest="sha256:000000000000",
                            details=ollama.ModelDetails(family=c.family or None, quantization_level=c.quantization or None))
            for c in self._all_cards() if str(c.model_id) in have])

    async def ollama_show(self, request: Request) -> ollama.ShowResponse:
        payload = ollama.ShowRequest.model_validate_json(await request.body())
        name = payload.name or payload.model
        if not name:
            raise HTTPException(400, "name or model is required")
        try:
            card = self._card(name)
        except Exception as e:
            raise HTTPException(404, f"Model not found: {name}") from e
        caps = (["completion", "tools"] if ModelTask.TextGeneration in card.tasks else []) + (["vision"] if card.vision else [])
        arch = card.family or "unknown"
        info: dict[str, Any] = {"general.architecture": arch, "general.basename": card.base_model or str(card.model_id)}
        if card.context_length > 0:
            info[f"{arch}.context_length"] = card.context_length
        return ollama.ShowResponse(modelfile=f"FROM {card.model_id}", template="{{ .Prompt }}", model_info=info, capabilities=caps,
                                   details=ollama.ModelDetails(family=card.family or None, quantization_level=card.quantization or None))

    async def ollama_ps(self) -> ollama.PsResponse:
        ids = dict.fromkeys(str(i.shard_assignments.model_id) for i in self.state.instances.values())
        return ollama.PsResponse(models=[ollama.PsModel(name=m, model=m, size=0) for m in ids])

    async def ollama_version(self) -> dict[str, str]:
        return {"version": "1.0.0"}

    # ---- models ----
    def _all_cards(self) -> list[ModelCard]:
        cards = {c.model_id: c for c in card_cache.list_all()}
        cards.update(self.state.custom_model_cards)
        return list(cards.values())

    @staticmethod
    def _model_entry(c: ModelCard) -> T.ModelListModel:
        return T.ModelListModel(id=c.model_id, hugging_face_id=c.model_id, name=c.model_id.short(), description="", tags=[],
                                storage_size_megabytes=c.storage_size.in_mb, supports_tensor=c.supports_tensor,
                                tasks=[t.value for t in c.tasks], is_custom=c.is_custom, family=c.family, quantization=c.quantization,
                                base_model=c.base_model, capabilities=c.capabilities, reasoning_dialect=c.reasoning_dialect,
                                context_length=c.context_length)

    async def get_models(self, status: str | None = Query(default=None)) -> T.ModelList:
        cards = self._all_cards()
        if status == "downloaded":
            have = self._downloaded_ids()
            cards = [c for c in cards if str(c.model_id) in have]
        return T.ModelList(data=[self._model_entry(c) for c in cards])

    async def add_custom_model(self, payload: T.AddCustomModelParams) -> T.ModelListModel:
        from ..download.cards import fetch_card
        try:
            card = await fetch_card(payload.model_id)
        except Exception as e:
            raise HTTPException(400, f"Failed to fetch model: {e}") from e
        await self._send(AddCustomModelCard(model_card=card))
        card_cache.cards[card.model_id] = card    # visible to the next GET /models without waiting for the event
        return self._model_entry(card)

    async def delete_custom_model(self, model_id: ModelId) -> JSONResponse:
        card = self.state.custom_model_cards.get(model_id) or card_cache.get(model_id)
        if card is None or not card.is_custom:
            raise HTTPException(404, "Custom model card not found")
        await self._send(DeleteCustomModelCard(model_id=model_id))
        return JSONResponse({"message": "Model card deleted", "model_id": str(model_id)})

    async def search_models(self, query: str = "", limit: int = 20) -> list[T.HuggingFaceSearchResult]:
        from ..download.cards import search_hub
        try:
            return await search_hub(query, limit)
        except Exception as e:
            raise HTTPException(502, f"HuggingFace search failed: {e}") from e

    # ---- images ----
    def _image_url(self, request: Request, image_id: str) -> str:
        return f"{str(request.base_url).rstrip('/')}/images/{image_id}"

    async def get_image(self, image_id: str) -> FileResponse:
        it = self._image_store.get(image_id)
        if it is None:
            raise HTTPException(404, "Image not found or expired")
        return FileResponse(it.path, media_type=it.content_type)

    async def list_images(self, request: Request) -> T.ImageListResponse:
        return T.ImageListResponse(data=[T.ImageListItem(image_id=i.image_id, url=self._image_url(request, i.image_id),
                                                         content_type=i.content_type, expires_at=i.expires_at)
                                         for i in self._image_store.list()])

    async def _image_events(self, command_id: CommandId) -> AsyncIterator[tuple[ImageChunk, str]]:
        """Reassembled images of one command: yields ``(last chunk of the image, full base64)``."""
        recv = self._image_recv.pop(command_id)
        parts: dict[tuple[int, bool, int | None], dict[int, str]] = {}
        try:
            with recv as chunks:
                async for ch in chunks:
                    if isinstance(ch, ErrorChunk) or ch.finish_reason == "error":
                        raise GenerationError(getattr(ch, "error_message", None) or "Internal server error")
                    key = (ch.image_index, ch.is_partial, ch.partial_index)
                    got = parts.setdefault(key, {})
                    got[ch.chunk_index] = ch.data
                    if len(got) == ch.total_chunks:
                        del parts[key]
                        yield ch, "".join(got[i] for i in range(len(got)))
        except (anyio.get_cancelled_exc_class(), GeneratorExit):
            with anyio.CancelScope(shield=True):
                await self.command_sender.send(ForwarderCommand(origin=self._system_id, command=TaskCancelled(cancelled_command_id=command_id)))
            raise
        finally:
            with anyio.CancelScope(shield=True):
                with contextlib.suppress(ChannelClosed):
                    await self.command_sender.send(ForwarderCommand(origin=self._system_id, command=TaskFinished(finished_command_id=command_id)))
            self._image_queues.pop(command_id, None)

    def _final_image(self, request: Request | None, ch: ImageChunk, b64: str, response_format: str) -> T.ImageData:
        if response_format == "url" and request is not None:
            stored = self._image_store.store(base64.b64decode(b64), ch.format or "png")
            return T.ImageData(b64_json=None, url=self._image_url(request, stored.image_id))
        return T.ImageData(b64_json=b64 if response_format == "b64_json" else None, url=None)

    async def _image_stream(self, request: Request, command_id: CommandId, n: int, response_format: str) -> AsyncIterator[str]:
        done = 0
        try:
            async for ch, b64 in self._image_events(command_id):
                if ch.is_partial:
                    ev = {"type": "partial", "image_index": ch.image_index, "partial_index": ch.partial_index,
                          "total_partials": ch.total_partials, "format": str(ch.format),
                          "data": {"b64_json": b64 if response_format == "b64_json" else None}}
                    yield common.sse(json.dumps(ev))
                    continue
                img = self._final_image(request, ch, b64, response_format)
                yield common.sse(json.dumps({"type": "final", "image_index": ch.image_index, "format": str(ch.format),
                                             "data": {"url": img.url} if img.url else {"b64_json": b64}}))
                done += 1
                if done >= n:
                    break
        except GenerationError as e:
            yield common.sse(T.ErrorResponse(error=T.ErrorInfo(message=str(e), type="InternalServerError", code=500)).model_dump_json())
        yield common.sse("[DONE]")

    async def _collect_images(self, request: Request | None, command_id: CommandId, n: int, response_format: str):
        finals: dict[int, T.ImageData] = {}
        stats = None
        try:
            async for ch, b64 in self._image_events(command_id):
                if ch.is_partial:
                    continue
                finals[ch.image_index] = self._final_image(request, ch, b64, response_format)
                stats = ch.stats or stats
                if len(finals) >= n:
                    break
        except GenerationError as e:
            raise HTTPException(500, str(e)) from e
        return [finals[i] for i in sorted(finals)], stats

    async def _collect_images_bench(self, request, command_id, n, response_format) -> T.BenchImageGenerationResponse:
        sampler = PowerSampler(lambda: self.state.node_system)
        async with anyio.create_task_group() as tg:
            tg.start_soon(sampler.run)
            try:
                images, stats = await self._collect_images(request, command_id, n, response_format)
            finally:
                tg.cancel_scope.cancel()
        return T.BenchImageGenerationResponse(data=images, generation_stats=stats, power_usage=sampler.result())

    def _open_image_queue(self, command_id: CommandId) -> None:
        self._image_queues[command_id], self._image_recv[command_id] = channel()

    async def _submit_image_generation(self, payload: T.ImageGenerationTaskParams) -> ImageGenerationCommand:
        payload = payload.model_copy(update={"model": await self._validate_model(payload.model),
                                             "advanced_params": _ensure_seed(payload.advanced_params)})
        cmd = ImageGenerationCommand(task_params=payload)
        self._open_image_queue(cmd.command_id)
        await self._send(cmd)
        return cmd

    async def image_generations(self, request: Request, payload: T.ImageGenerationTaskParams):
        cmd = await self._submit_image_generation(payload)
        n, fmt = payload.n or 1, payload.response_format or "b64_json"
        if payload.stream and payload.partial_images and payload.partial_images > 0:
            return StreamingResponse(self._image_stream(request, cmd.command_id, n, fmt), media_type="text/event-stream")
        images, _ = await self._collect_images(request, cmd.command_id, n, fmt)
        return T.ImageGenerationResponse(data=images)

    async def bench_image_generations(self, request: Request, payload: T.BenchImageGenerationTaskParams) -> T.BenchImageGenerationResponse:
        cmd = await self._submit_image_generation(payload.model_copy(update={"stream": False, "partial_images": 0, "bench": True}))
        return await self._collect_images_bench(request, cmd.command_id, payload.n or 1, payload.response_format or "b64_json")

    async def _submit_image_edit(self, image: UploadFile, *, prompt: str, model: str, n: int, size: str | None, response_format: str,
                                 input_fidelity: str, stream: bool, partial_images: int, bench: bool, quality: str, output_format: str,
                                 advanced_params: str | None) -> ImageEditsCommand:
        adv = None
        if advanced_params:
            with contextlib.suppress(Exception):
                adv = T.AdvancedImageParams.model_validate_json(advanced_params)
        mid = await self._validate_model(model)
        data = base64.b64encode(await image.read()).decode("utf-8")
        pieces = [data[o:o + constants.EXO_MAX_CHUNK_SIZE] for o in range(0, len(data), constants.EXO_MAX_CHUNK_SIZE)]
        cmd = ImageEditsCommand(task_params=T.ImageEditsTaskParams(
            image_data="", total_input_chunks=len(pieces), prompt=prompt, model=mid, n=n, size=T.normalize_image_size(size),
            response_format=response_format, image_strength=0.7 if input_fidelity == "high" else 0.3, stream=stream,
            partial_images=partial_images, bench=bench, quality=quality, output_format=output_format, advanced_params=_ensure_seed(adv)))
        self._open_image_queue(cmd.command_id)
        for k, piece in enumerate(pieces):
            await self._send(SendInputChunk(chunk=InputImageChunk(model=mid, command_id=cmd.command_id, data=piece, chunk_index=k,
                                                                  total_chunks=len(pieces))))
        await self._send(cmd)
        return cmd

    async def image_edits(self, request: Request, image: UploadFile = File(...), prompt: str = Form(...), model: str = Form(...),
                          n: int = Form(1), size: str | None = Form(None), response_format: Literal["url", "b64_json"] = Form("b64_json"),
                          input_fidelity: Literal["low", "high"] = Form("low"), stream: str = Form("false"),
                          partial_images: str = Form("0"), quality: Literal["high", "medium", "low"] = Form("medium"),
                          output_format: Literal["png", "jpeg", "webp"] = Form("png"), advanced_params: str | None = Form(None)):
        want_stream = stream.lower() in ("true", "1", "yes")
        partials = int(partial_images) if partial_images.isdigit() else 0
        cmd = await self._submit_image_edit(image, prompt=prompt, model=model, n=n, size=size, response_format=response_format,
                                            input_fidelity=input_fidelity, stream=want_stream, partial_images=partials, bench=False,
                                            quality=quality, output_format=output_format, advanced_params=advanced_params)
        if want_stream and partials > 0:
            return StreamingResponse(self._image_stream(request, cmd.command_id, n, response_format), media_type="text/event-stream")
        images, _ = await self._collect_images(request, cmd.command_id, n, response_format)
        return T.ImageGenerationResponse(data=images)

    async def bench_image_edits(self, request: Request, image: UploadFile = File(...), prompt: str = Form(...), model: str = Form(...),
                                n: int = Form(1), size: str | None = Form(None),
                                response_format: Literal["url", "b64_json"] = Form("b64_json"),
                                input_fidelity: Literal["low", "high"] = Form("low"),
                                quality: Literal["high", "medium", "low"] = Form("medium"),
                                output_format: Literal["png", "jpeg", "webp"] = Form("png"),
                                advanced_params: str | None = Form(None)) -> T.BenchImageGenerationResponse:
        cmd = await self._submit_image_edit(image, prompt=prompt, model=model, n=n, size=size, response_format=response_format,
                                            input_fidelity=input_fidelity, stream=False, partial_images=0, bench=True,
                                            quality=quality, output_format=output_format, advanced_params=advanced_params)
        return await self._collect_images_bench(request, cmd.command_id, n, response_format)

    # ---- downloads ----
    async def start_download(self, payload: T.StartDownloadParams) -> T.StartDownloadResponse:
        cmd = StartDownload(target_node_id=payload.target_node_id, shard_metadata=payload.shard_metadata)
        await self._send_download(cmd)
        return T.StartDownloadResponse(command_id=cmd.command_id)

    async def delete_download(self, node_id: NodeId, model_id: ModelId) -> T.DeleteDownloadResponse:
        cmd = DeleteDownload(target_node_id=node_id, model_id=ModelId(model_id))
        await self._send_download(cmd)
        return T.DeleteDownloadResponse(command_id=cmd.command_id)

    async def cancel_download(self, payload: T.CancelDownloadParams) -> T.CancelDownloadResponse:
        cmd = CancelDownload(target_node_id=payload.target_node_id, model_id=payload.model_id)
        await self._send_download(cmd)
        return T.CancelDownloadResponse(command_id=cmd.command_id)

    # ---- traces ----
    @staticmethod
    def _trace_path(task_id: str) -> Path:
        root = constants.EXO_TRACING_CACHE_DIR
        p = root / f"trace_{task_id}.json"
        if not p.resolve().is_relative_to(root.resolve()):
            raise HTTPException(400, f"Invalid task ID: {task_id}")
        return p

    def _existing_trace(self, task_id: str) -> Path:
        p = self._trace_path(task_id)
        if not p.exists():
            raise HTTPException(404, f"Trace not found: {task_id}")
        return p

    async def list_traces(self) -> T.TraceListResponse:
        files = sorted(constants.EXO_TRACING_CACHE_DIR.glob("trace_*.json"), key=lambda p: p.stat().st_mtime, reverse=True)
        return T.TraceListResponse(traces=[T.TraceListItem(
            task_id=f.stem.removeprefix("trace_"), file_size=f.stat().st_size,
            created_at=datetime.fromtimestamp(f.stat().st_mtime, tz=timezone.utc).isoformat()) for f in files])

    async def get_trace(self, task_id: str) -> T.TraceResponse:
        evs = tracing.load_trace_file(self._existing_trace(task_id))
        return T.TraceResponse(task_id=task_id, traces=[T.TraceEventResponse(name=e.name, start_us=e.start_us, duration_us=e.duration_us,
                                                                             rank=e.rank, category=e.category) for e in evs])

    async def get_trace_stats(self, task_id: str) -> T.TraceStatsResponse:
        st = tracing.compute_stats(tracing.load_trace_file(self._existing_trace(task_id)))

        def cat(c) -> T.TraceCategoryStats:
            return T.TraceCategoryStats(total_us=c.total_us, count=c.count, min_us=c.min_us, max_us=c.max_us, avg_us=c.avg_us)
        return T.TraceStatsResponse(task_id=task_id, total_wall_time_us=st.total_wall_time_us,
                                    by_category={k: cat(v) for k, v in st.by_category.items()},
                                    by_rank={r: T.TraceRankStats(by_category={k: cat(v) for k, v in d.items()}) for r, d in st.by_rank.items()})

    async def get_trace_raw(self, task_id: str) -> FileResponse:
        return FileResponse(self._existing_trace(task_id), media_type="application/json", filename=f"trace_{task_id}.json")

    async def delete_traces(self, request: T.DeleteTracesRequest) -> T.DeleteTracesResponse:
        deleted, missing = [], []
        for tid in request.task_ids:
            p = self._trace_path(tid)
            if p.exists():
                p.unlink()
                deleted.append(tid)
            else:
                missing.append(tid)
        return T.DeleteTracesResponse(deleted=deleted, not_found=missing)

    def _save_merged_trace(self, ev: TracesMerged) -> None:
        events = [tracing.TraceEvent(name=t.name, start_us=t.start_us, duration_us=t.duration_us, rank=t.rank, category=t.category)
                  for t in ev.traces]
        constants.EXO_TRACING_CACHE_DIR.mkdir(parents=True, exist_ok=True)
        tracing.export_trace(events, constants.EXO_TRACING_CACHE_DIR / f"trace_{ev.task_id}.json")

    # ---- onboarding ----
    async def get_onboarding(self) -> JSONResponse:
        return JSONResponse({"completed": ONBOARDING_FILE.exists()})

    async def complete_onboarding(self) -> JSONResponse:
        ONBOARDING_FILE.parent.mkdir(parents=True, exist_ok=True)
        ONBOARDING_FILE.write_text("true")
        return JSONResponse({"completed": True})

    # ---- event fold and serving ----
    async def _apply_state(self) -> None:
        with self.event_receiver as events:
            async for ie in events:
                self._event_log.append(ie.event.model_dump_json())
                self.state = apply(self.state, ie)
                ev = ie.event
                if isinstance(ev, ChunkGenerated):
                    queues = self._image_queues if isinstance(ev.chunk, ImageChunk) else self._text_queues
                    q = queues.get(ev.command_id)
                    if q is None and isinstance(ev.chunk, ErrorChunk):
                        q = self._image_queues.get(ev.command_id)
                    if q is not None:
                        try:
                            await q.send(ev.chunk)
                        except ChannelClosed:
                            queues.pop(ev.command_id, None)
                elif isinstance(ev, InstanceDeleted):
                    self._close_streams_for_instance(ev.instance_id)
                elif isinstance(ev, TracesMerged):
                    self._save_merged_trace(ev)

    def _close_streams_for_instance(self, instance_id: InstanceId) -> None:
        for task in self.state.tasks.values():
            if task.instance_id == instance_id and isinstance(task, GENERATION_TASKS):
                for queues in (self._text_queues, self._image_queues):
                    if (q := queues.pop(task.command_id, None)) is not None:
                        q.close()

    async def _cleanup_images(self) -> None:
        while True:
            await anyio.sleep(300)
            self._image_store.cleanup()

    async def _serve(self) -> None:
        import uvicorn
        cfg = uvicorn.Config(self.app, host=self.host, port=self.port, log_level="warning", access_log=False,
                             timeout_graceful_shutdown=2, lifespan="off")
        self.server = uvicorn.Server(cfg)
        self.server.install_signal_handlers = lambda: None   # the node owns SIGINT/SIGTERM
        try:
            await self.server.serve()
        finally:
            self.server.should_exit = True

    async def run(self) -> None:
        try:
            async with self._tg as tg:
                tg.start_soon(self._apply_state)
                tg.start_soon(self._pause_on_new_election)
                tg.start_soon(self._cleanup_images)
                tg.start_soon(self._serve)
                try:
                    await anyio.sleep_forever()
                finally:
                    for q in (*self._text_queues.values(), *self._image_queues.values()):
                        q.close()
                    if self.server is not None:
                        self.server.should_exit = True
        finally:
            self._event_log.close()
            self.command_sender.close()
            self.event_receiver.close()

    def shutdown(self) -> None:
        self._tg.cancel_tasks()
