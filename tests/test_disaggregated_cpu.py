"""Prefill/decode disaggregation on CPU: wire protocol, server error paths, KV hand-over between two engines."""
import io
import socket
import threading

import pytest
import torch

from exo_b200.models.config import preset
from exo_b200.models.weights import RandomSource, ShardSpec, build_weights
from exo_b200.shared import constants
from exo_b200.shared.base import InstanceId, ModelId
from exo_b200.shared.messages import InputMessage, TextGeneration, TextGenerationTaskParams
from exo_b200.shared.wire import TokenChunk
from exo_b200.worker.disaggregated import protocol as P
from exo_b200.worker.disaggregated.server import PrefillServer, RemotePrefillError, remote_prefill_fetch
from exo_b200.worker.engines.base import Finished


def test_frames_and_messages_roundtrip():
    buf = io.BytesIO()
    P.write_request(buf, P.PrefillRequest(request_id="r", model_id="m", token_ids=[1, 2, 3], start_pos=1))
    P.write_header(buf, P.Header(request_id="r", model_id="m", num_layers=2, dtype="bfloat16", start_pos=1))
    P.write_message(buf, P.KVChunk(layer_idx=1, num_tokens=2, n_heads=3, head_dim=4, dtype="bfloat16", keys=b"k" * 48, values=b"v" * 48))
    P.write_message(buf, P.ArraysState(layer_idx=0, arrays=[P.TensorBlob("float32", (2, 2), b"\0" * 16)]))
    P.write_message(buf, P.Done(total_tokens=2))
    P.write_message(buf, P.ErrorMessage(code=503, message="busy"))
    raw = buf.getvalue()
    assert raw[:4] == (len(raw.split(b"\x84", 1)[0]) and raw[:4])      # 4-byte big-endian length prefix
    assert int.from_bytes(raw[:4], "big") > 0
    buf.seek(0)
    req = P.read_request(buf)
    assert req.token_ids == [1, 2, 3] and req.start_pos == 1
    assert P.read_header(buf).num_layers == 2
    kc = P.read_message(buf)
    assert isinstance(kc, P.KVChunk) and kc.shape == (2, 3, 4) and kc.keys == b"k" * 48
    st = P.read_message(buf)
    assert isinstance(st, P.ArraysState) and st.arrays[0].shape == (2, 2)
    assert P.read_message(buf).total_tokens == 2
    assert P.read_message(buf).code == 503
    assert P.read_message(buf) is None
    with pytest.raises(ConnectionError):
        P.read_frame(io.BytesIO(b"\x00\x00\x00\x10abc"))
    with pytest.raises(P.ProtocolError):
        bad = io.BytesIO()
        P.write_frame(bad, b"\xc1")
        bad.seek(0)
        P.read_message(bad)


def test_server_reports_errors_in_band():
    def resolve(job, wfile):
        if job.request_id == "boom":
            raise RuntimeError("engine exploded")
        return False
    srv = PrefillServer(resolve, "127.0.0.1", 0)
    try:
        with pytest.raises(RemotePrefillError) as e:
            remote_prefill_fetch(f"127.0.0.1:{srv.port}", P.PrefillRequest(request_id="boom", token_ids=[1]))
        assert e.value.code == 500 and "exploded" in str(e.value)
        with pytest.raises(RemotePrefillError) as e:
            remote_prefill_fetch(f"127.0.0.1:{srv.port}", P.PrefillRequest(request_id="nobody", token_ids=[1]))
        assert e.value.code == 503
        with socket.create_connection(("127.0.0.1", srv.port)) as s:       # garbage instead of a request
            f = s.makefile("rwb")
            P.write_frame(f, b"\xc1\xc1")
            assert P.read_header(f).num_layers == 0
            assert P.read_message(f).code == 400
    finally:
        srv.stop()


def _serving_engine(model_id="tiny", name="tiny-llama"):
    from exo_b200.engine.engine import Engine
    from exo_b200.worker.engines.b200.builder import ServingEngine
    from exo_b200.worker.engines.b200.tokenizer import ByteTokenizer
    cfg = preset(name)
    cfg.vocab = 512
    cfg.dtype = "fp32"
    w = build_weights(cfg, ShardSpec(), RandomSource(seed=0, dtype=torch.float32))
    te = Engine(cfg, w, n_blocks=256, prefill_chunk=64)
    return ServingEngine(cfg, te, ByteTokenizer(512), model_id, "llama", (257,))


def _task(prompt, endpoint=None):
    return TextGeneration(instance_id=InstanceId("i"), command_id="c", task_params=TextGenerationTaskParams(
        model=ModelId("tiny"), input=[InputMessage(role="user", content=prompt)], temperature=0.0, max_output_tokens=6,
        bench=True, prefill_endpoint=endpoint))


def _run(engine, task, pump=None):
    engine.submit(task)
    toks = []
    for _ in range(100000):
        if pump is not None:
            pump()
        for _tid, item in engine.step():
            if isinstance(item, TokenChunk):
                toks.append(item.token_id)
            if isinstance(item, Finished):
                return toks
    raise AssertionError("generation did not finish")


@pytest.mark.parametrize("name", ["tiny-llama", "tiny-mla", "tiny-qwen3-next", "tiny-nemotron-h", "tiny-gemma4"])
def test_kv_handover_between_prefill_and_decode_engines(monkeypatch, name):
    """Dense model: the prompt's KV rows travel.  Models with recurrent layers (gated delta rule, Mamba-2): the attention layers'
    KV rows and, once per layer, the recurrent layers' state after exactly the handed-over tokens, installed into a seat of
    the decode engine."""
    monkeypatch.setattr(constants, "REMOTE_PREFILL_MIN_TOKENS", 16)
    prompt = "the quick brown fox jumps over the lazy dog " * 5       # ~220 byte tokens, several 64-token chunks
    _engine = _serving_engine
    globals()["_serving_engine"] = lambda model_id="tiny": _engine(model_id, name)
    try:
        _handover(prompt, name)
    finally:
        globals()["_serving_engine"] = _engine


def _handover(prompt, name):
    want = _run(_serving_engine(), _task(prompt))

    prefill, decode = _serving_engine(), _serving_engine()
    port = prefill.enable_prefill_server("127.0.0.1")
    stop = threading.Event()

    def prefill_loop():         # the prefill instance's runner loop
        while not stop.is_set():
            if prefill.has_work:
                prefill.step()
            else:
                stop.wait(0.002)
    t = threading.Thread(target=prefill_loop, daemon=True)
    t.start()
    try:
        steps_before = decode.te.n_steps
        got = _run(decode, _task(prompt, endpoint=f"127.0.0.1:{port}"))
        assert got == want
        assert decode.remote_prefills == 1
        # the decode engine computed only the prompt's tail + the new tokens: far fewer steps than a local prefill
        assert decode.te.n_steps - steps_before <= 1 + 6
        if name not in ("tiny-llama", "tiny-mla", "tiny-gemma4"):
            assert decode.te.sched._free_seats and len(decode.te.sched._free_seats) == decode.te.sched.max_seqs     # the seat came back
            # a second request re-uses seats on both sides
            assert _run(decode, _task(prompt + "again", endpoint=f"127.0.0.1:{port}")) == _run(_serving_engine(), _task(prompt + "again"))
            assert decode.remote_prefills == 2
        # an unreachable endpoint falls back to local prefill, same tokens
        again = _serving_engine()
        assert _run(again, _task(prompt, endpoint="127.0.0.1:9")) == want and again.remote_prefills == 0
    finally:
        stop.set()
        t.join(timeout=5)
        prefill.close()
