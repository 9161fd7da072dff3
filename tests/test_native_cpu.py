"""Native runtime: bus pub/sub + liveliness + namespace isolation, pidfile, NVML absence."""
import multiprocessing as mp
import os
import time

import anyio
import pytest

native = pytest.importorskip("exo_b200.native._exo_native")


def _drain(bus, want, timeout=5.0):
    out, t0 = [], time.time()
    while time.time() - t0 < timeout:
        ev = bus.try_recv()
        if ev is None:
            time.sleep(0.01)
            continue
        out.append(ev)
        if want(out):
            break
    return out


def test_identity_rules_and_namespace_hash():
    assert native.valid_identity("1a2b") and not native.valid_identity("0abc") and not native.valid_identity("xyz")
    assert not native.valid_identity("1" * 33)
    assert native.namespace_hash("a") != native.namespace_hash("b")


def test_pubsub_remote_only_ordering_and_liveliness():
    a = native.Bus("a1", "ns", 0, 0)
    b = native.Bus("b2", "ns", 0, 0)
    b.subscribe("t")
    a.subscribe("t")
    assert a.connect("127.0.0.1", b.listen_port)
    evs = _drain(b, lambda o: any(e[0] == "connection" for e in o))
    assert ("connection", "a1", True) in evs
    _drain(a, lambda o: any(e[0] == "connection" for e in o))
    time.sleep(0.1)  # let SUB frames land
    for i in range(200):
        assert a.publish("t", b"m%d" % i) == 1
    assert a.publish("other", b"x") == 0
    msgs = [e for e in _drain(b, lambda o: sum(e[0] == "message" for e in o) >= 200) if e[0] == "message"]
    assert [m[2] for m in msgs] == [b"m%d" % i for i in range(200)]
    assert a.try_recv() is None  # publisher does not hear itself
    a.close()
    evs = _drain(b, lambda o: any(e[0] == "connection" and not e[2] for e in o))
    assert ("connection", "a1", False) in evs
    b.close()


def test_namespace_isolation():
    a = native.Bus("a1", "cluster-one", 0, 0)
    b = native.Bus("b2", "cluster-two", 0, 0)
    a.connect("127.0.0.1", b.listen_port)
    time.sleep(0.5)
    assert a.peers() == [] and b.peers() == []
    a.close(); b.close()


def _peer_proc(port, q):
    from exo_b200.native import _exo_native as n
    bus = n.Bus("c3", "ns", 0, 0)
    bus.subscribe("t")
    bus.connect("127.0.0.1", port)
    q.put("up")
    time.sleep(60)


def test_peer_process_death_is_reported():
    a = native.Bus("a1", "ns", 0, 0)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_peer_proc, args=(a.listen_port, q), daemon=True)
    p.start()
    assert q.get(timeout=30) == "up"
    assert ("connection", "c3", True) in _drain(a, lambda o: any(e[0] == "connection" for e in o), 10)
    os.kill(p.pid, 9)
    assert ("connection", "c3", False) in _drain(a, lambda o: any(e[0] == "connection" and not e[2] for e in o), 10)
    a.close()


def test_router_over_native_transport():
    from exo_b200.native.bus import NativeTransport
    from exo_b200.routing.router import COMMANDS, make_router
    from exo_b200.shared.base import NodeId, SystemId
    from exo_b200.shared.messages import ForwarderCommand, TestCommand

    async def main():
        ta, tb = NativeTransport("a1", "ns"), NativeTransport("b2", "ns")
        ra, rb = make_router(NodeId("a1"), ta), make_router(NodeId("b2"), tb)
        got = rb.receiver(COMMANDS)
        send = ra.sender(COMMANDS)
        async with anyio.create_task_group() as tg:
            tg.start_soon(ra.run)
            tg.start_soon(rb.run)
            await anyio.sleep(0.1)
            ta.connect("127.0.0.1", tb.listen_port)
            await anyio.sleep(0.3)
            cmd = ForwarderCommand(origin=SystemId("s"), command=TestCommand())
            await send.send(cmd)
            with anyio.fail_after(5):
                assert await got.receive() == cmd
            ra.shutdown(); rb.shutdown()
            tg.cancel_scope.cancel()
    anyio.run(main)


def test_pidfile_lock(tmp_path):
    p = str(tmp_path / "exo.pid")
    f = native.Pidfile(p)
    f.write()
    assert int(open(p).read()) == os.getpid() and f.as_raw_fd() > 0
    with pytest.raises(Exception, match=f"AlreadyRunning:{os.getpid()}"):
        native.Pidfile(p)
    f.close()
    assert not os.path.exists(p)
    native.Pidfile(p).close()


def test_nvml_enumerate_without_driver_is_empty_not_fatal():
    gpus, err = native.nvml_enumerate()
    assert isinstance(gpus, list) and (gpus or err)


def test_discovery_answers_hello_with_whatsup_in_the_wire_format_and_ignores_other_namespaces():
    """Packet-level discovery (reference wire format, ``rust/networking/src/discovery.rs:313-336``): a Hello
    ``{magic "EXO", kind 1, nonce[8], namespace[8]}`` from the same namespace is answered with a WhatsUp
    ``{magic, kind 2, nonce echoed, id[16] right-aligned, port little-endian}``; another namespace gets nothing."""
    import socket
    import struct
    import time
    with socket.socket(socket.AF_INET6, socket.SOCK_DGRAM) as probe:
        probe.bind(("::", 0))
        disc_port = probe.getsockname()[1]
    bus = native.Bus("ab12", "disc-test", 0, disc_port)
    try:
        time.sleep(0.2)
        with socket.socket(socket.AF_INET6, socket.SOCK_DGRAM) as s:
            s.settimeout(3)
            nonce = b"nonce-01"
            hello = b"EXO" + bytes([1]) + nonce + struct.pack("<Q", native.namespace_hash("disc-test"))
            s.sendto(hello, ("::1", disc_port))
            pkt, _ = s.recvfrom(64)
            assert len(pkt) == 30 and pkt[:3] == b"EXO" and pkt[3] == 2
            assert pkt[4:12] == nonce
            assert pkt[12:28].hex() == "ab12".rjust(32, "0")
            assert pkt[28] | (pkt[29] << 8) == bus.listen_port
            other = b"EXO" + bytes([1]) + b"nonce-02" + struct.pack("<Q", native.namespace_hash("someone-else"))
            s.sendto(other, ("::1", disc_port))
            s.settimeout(0.5)
            try:
                s.recvfrom(64)
                raise AssertionError("a Hello from another namespace must not be answered")
            except socket.timeout:
                pass
            # a truncated packet and a wrong magic are dropped without a reply either
            s.sendto(b"EX", ("::1", disc_port))
            s.sendto(b"XXX" + bytes([1]) + bytes(16), ("::1", disc_port))
            try:
                s.recvfrom(64)
                raise AssertionError("malformed discovery packets must be ignored")
            except socket.timeout:
                pass
    finally:
        bus.close()
