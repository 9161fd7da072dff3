"""One exo node: router, event router, election, master, worker, download coordinator, API.

Composition and election handling follow the reference (``src/exo/main.py:36-504``): every node
starts with its own master and session; when an election result names a new master the event
router is rebuilt for the new session, the master is promoted or demoted, the worker and the
download coordinator are restarted against the fresh event stream and the API is reset; a result
that confirms the current master only un-pauses the API.  A node is bound to one GPU
(``--gpu`` / ``EXO_GPU_INDEX``); ``--all-gpus`` starts one node process per visible GPU on this
box, the first of them serving the API, all of them joined through ``--peers`` on loopback.
"""
from __future__ import annotations

import argparse
import multiprocessing as mp
import os
import resource
import signal
import subprocess
import sys
import uuid
from dataclasses import dataclass
from pathlib import Path

import anyio

from . import __version__
from .download.coordinator import DownloadCoordinator
from .download.shard_downloader import NoopShardDownloader, exo_shard_downloader
from .master.main import Master
from .routing import router as topics
from .routing.event_router import EventRouter
from .routing.router import Router, make_router
from .shared import constants
from .shared.base import NodeId, SessionId
from .shared.election import Election, ElectionResult
from .shared.logging import logger, logger_cleanup, logger_setup
from .utils.async_process import TaskGroup
from .utils.channels import Receiver, channel
from .utils.info_gatherer import InfoGatherer
from .worker.main import Worker


@dataclass(frozen=True)
class Args:
    verbosity: int = 0
    force_master: bool = False
    spawn_api: bool = True
    api_port: int = 52415
    no_worker: bool = False
    no_downloads: bool = False
    offline: bool = False
    no_batch: bool = False
    legacy_daemon: bool = False
    namespace: str = __version__
    bus_port: int = 52414
    discovery_port: int = 52413
    peers: tuple[str, ...] = ()
    gpu: int | None = None
    all_gpus: bool = False
    seed_models: str | None = None

    @classmethod
    def parse(cls, argv: list[str] | None = None) -> "Args":
        p = argparse.ArgumentParser(prog="exo")
        p.add_argument("-q", "--quiet", action="store_const", const=-1, dest="verbosity", default=0)
        p.add_argument("-v", "--verbose", action="count", dest="verbosity", default=0)
        p.add_argument("-m", "--force-master", action="store_true")
        p.add_argument("--no-api", action="store_false", dest="spawn_api")
        p.add_argument("--api-port", type=int, default=52415)
        p.add_argument("--no-worker", action="store_true")
        p.add_argument("--no-downloads", action="store_true", help="this node will not download models")
        p.add_argument("--offline", action="store_true", default=os.getenv("EXO_OFFLINE", "false").lower() == "true",
                       help="air-gapped mode: no internet checks, only models already on disk")
        p.add_argument("--no-batch", action="store_true", help="one request at a time instead of continuous batching")
        p.add_argument("--legacy-daemon", action="store_true", help="detach and run in the background")
        p.add_argument("--namespace", default=os.getenv("EXO_NAMESPACE", __version__),
                       help="nodes with different namespaces do not connect")
        p.add_argument("--bus-port", "--zenoh-port", type=int, default=52414, dest="bus_port", help="TCP port of the node bus (0 = any)")
        p.add_argument("--discovery-port", type=int, default=52413, help="UDP multicast discovery port (0 = off)")
        p.add_argument("--peers", type=lambda s: tuple(x for x in s.split(",") if x), default=(), help="host:port,... to dial at start")
        p.add_argument("--gpu", type=int, default=None, help="GPU index this node owns (default: EXO_GPU_INDEX or 0)")
        p.add_argument("--all-gpus", action="store_true", help="start one node per GPU of this box")
        p.add_argument("--seed-models", default=None, help="directory of pre-packaged models to move into the models dir")
        ns = p.parse_args(argv)
        return cls(**vars(ns))


def node_identity(gpu: int | None) -> NodeId:
    """Persistent per-(box, GPU) identity: 32 hex digits without a leading zero."""
    name = constants.EXO_NODE_ZID if gpu is None else constants.EXO_NODE_ZID.with_name(f"{constants.EXO_NODE_ZID.name}.gpu{gpu}")
    try:
        v = name.read_text().strip()
        if v:
            return NodeId(v)
    except OSError:
        pass
    v = uuid.uuid4().hex
    if v[0] == "0":
        v = "1" + v[1:]
    try:
        name.parent.mkdir(parents=True, exist_ok=True)
        name.write_text(v)
    except OSError:
        pass
    return NodeId(v)


def make_transport(node_id: NodeId, args: Args):
    from .native.bus import NativeTransport
    t = NativeTransport(str(node_id), args.namespace, args.bus_port, args.discovery_port)
    for peer in args.peers:
        host, _, port = peer.rpartition(":")
        t.connect(host or "127.0.0.1", int(port))
    return t


class Node:
    def __init__(self, args: Args, node_id: NodeId, router: Router):
        self.args, self.node_id, self.router = args, node_id, router
        self.session = SessionId(master_node_id=node_id, election_clock=0)
        self.event_router = self._event_router(self.session)
        self.download_coordinator = None if args.no_downloads else self._coordinator()
        self.api = None
        if args.spawn_api:
            from .api.main import API
            self.api = API(node_id, port=args.api_port, event_receiver=self.event_router.receiver(),
                           command_sender=router.sender(topics.COMMANDS),
                           download_command_sender=router.sender(topics.DOWNLOAD_COMMANDS),
                           election_receiver=router.receiver(topics.ELECTION_MESSAGES),
                           event_log_dir=constants.EXO_EVENT_LOG_DIR / f"api-{node_id[:8]}")
        self.worker = None if args.no_worker else self._worker()
        self.master: Master | None = self._master(self.session)
        er_send, self.election_results = channel()
        self.election = Election(node_id, seniority=1_000_000 if args.force_master else 0,
                                 election_message_sender=router.sender(topics.ELECTION_MESSAGES),
                                 election_message_receiver=router.receiver(topics.ELECTION_MESSAGES),
                                 connection_message_receiver=router.receiver(topics.CONNECTION_MESSAGES),
                                 command_receiver=router.receiver(topics.COMMANDS), election_result_sender=er_send)
        self._tg = TaskGroup()
        self._stopping = False

    # ---- factories (also used when a new master is elected) ----
    def _event_router(self, session: SessionId) -> EventRouter:
        return EventRouter(session, self.router.sender(topics.COMMANDS), self.router.receiver(topics.GLOBAL_EVENTS),
                           self.router.sender(topics.LOCAL_EVENTS))

    def _coordinator(self) -> DownloadCoordinator:
        return DownloadCoordinator(self.node_id, exo_shard_downloader(offline=self.args.offline),
                                   self.router.receiver(topics.DOWNLOAD_COMMANDS), self.event_router.sender(),
                                   offline=self.args.offline)

    def _worker(self) -> Worker:
        return Worker(self.node_id, event_receiver=self.event_router.receiver(), event_sender=self.event_router.sender(),
                      command_sender=self.router.sender(topics.COMMANDS),
                      download_command_sender=self.router.sender(topics.DOWNLOAD_COMMANDS), api_port=self.args.api_port,
                      info_gatherer=InfoGatherer(None, gpu_index=self.args.gpu))

    def _master(self, session: SessionId) -> Master:
        return Master(self.node_id, session, command_receiver=self.router.receiver(topics.COMMANDS),
                      local_event_receiver=self.router.receiver(topics.LOCAL_EVENTS),
                      global_event_sender=self.router.sender(topics.GLOBAL_EVENTS),
                      log_dir=constants.EXO_EVENT_LOG_DIR / f"master-{self.node_id[:8]}")   # nodes of one box share the data dir

    # ---- lifecycle ----
    async def run(self) -> None:
        async with self._tg as tg:
            for sig in (signal.SIGINT, signal.SIGTERM):
                try:
                    signal.signal(sig, lambda *_: self.shutdown())
                except ValueError:      # not the main thread (tests)
                    pass
            tg.start_soon(self.router.run)
            tg.start_soon(self.event_router.run)
            tg.start_soon(self.election.run)
            if self.download_coordinator:
                tg.start_soon(self.download_coordinator.run)
            if self.worker:
                tg.start_soon(self.worker.run)
            if self.master:
                tg.start_soon(self.master.run)
            if self.api:
                tg.start_soon(self.api.run)
            tg.start_soon(self._elect_loop)

    def shutdown(self) -> None:
        if self._stopping:
            sys.exit(1)     # second signal: do not wait for a clean stop
        self._stopping = True
        self._tg.cancel_tasks()

    async def _elect_loop(self) -> None:
        with self.election_results as results:
            async for res in results:
                await self.on_election_result(res)

    async def on_election_result(self, res: ElectionResult) -> None:
        me = res.session_id.master_node_id == self.node_id
        if res.is_new_master:
            await anyio.lowlevel.checkpoint()
            self.event_router.shutdown()
            self.event_router = self._event_router(res.session_id)
        if me and self.master is None:
            logger.info("elected master: promoting self")
            self.master = self._master(res.session_id)
            self._tg.start_soon(self.master.run)
        elif not me and self.master is not None:
            logger.info(f"{res.session_id.master_node_id} elected master: demoting self")
            self.master.shutdown()
            self.master = None
        elif me and res.is_new_master and self.master is not None:
            # same node, new session (e.g. the cluster re-formed around us): restart the master on the new session
            self.master.shutdown()
            self.master = self._master(res.session_id)
            self._tg.start_soon(self.master.run)
        self.session = res.session_id
        if not res.is_new_master:
            if self.api:
                self.api.unpause(res.won_clock)
            return
        if self.download_coordinator:
            await self.download_coordinator.shutdown()
            self.download_coordinator = self._coordinator()
            self._tg.start_soon(self.download_coordinator.run)
        if self.worker:
            await self.worker.shutdown()
            self.worker = self._worker()
            self._tg.start_soon(self.worker.run)
        if self.api:
            self.api.reset(res.won_clock, self.event_router.receiver())
        self._tg.start_soon(self.event_router.run)


def _spawn_per_gpu(args: Args, argv: list[str]) -> int:
    """``--all-gpus``: this process becomes a launcher for one node per GPU."""
    from .utils.info_gatherer import nvml_probe
    gpus = [g.index for g in nvml_probe()] or [0]
    base = [a for a in argv if a != "--all-gpus"]
    procs: list[subprocess.Popen] = []
    first_bus = args.bus_port or 52414
    for i, g in enumerate(gpus):
        cmd = [sys.executable, "-m", "exo_b200", *base, "--gpu", str(g), "--bus-port", str(first_bus + i), "--discovery-port", "0"]
        if i > 0:
            cmd += ["--no-api", "--peers", f"127.0.0.1:{first_bus}"]
        procs.append(subprocess.Popen(cmd, env={**os.environ, "EXO_GPU_INDEX": str(g)}))

    def stop(*_):
        for p in procs:
            p.terminate()
    signal.signal(signal.SIGINT, stop)
    signal.signal(signal.SIGTERM, stop)
    rc = 0
    for p in procs:
        rc = p.wait() or rc
    return rc


def main_inner(args: Args) -> None:
    soft, hard = resource.getrlimit(resource.RLIMIT_NOFILE)
    try:
        resource.setrlimit(resource.RLIMIT_NOFILE, (min(max(soft, 65535), hard), hard))
    except (ValueError, OSError):
        pass
    mp.set_start_method("spawn", force=True)
    logger_setup(constants.EXO_LOG, args.verbosity)
    logger.info(f"pid = {os.getpid()}")
    if args.offline:
        logger.info("OFFLINE mode: no internet checks, local models only")
    if args.no_batch:
        os.environ["EXO_NO_BATCH"] = "1"
    if args.gpu is not None:
        os.environ["EXO_GPU_INDEX"] = str(args.gpu)
    constants.EXO_DEFAULT_MODELS_DIR.mkdir(parents=True, exist_ok=True)
    if args.seed_models:
        from .download.store import seed_models
        seed_models(args.seed_models)
    gpu = args.gpu if args.gpu is not None else (int(os.environ["EXO_GPU_INDEX"]) if os.environ.get("EXO_GPU_INDEX") else None)
    node_id = node_identity(gpu)

    async def amain() -> None:
        router = make_router(node_id, make_transport(node_id, args))
        node = Node(args, node_id, router)
        logger.info(f"starting node {node_id} (gpu {gpu})")
        await node.run()
    try:
        anyio.run(amain)
    except BaseException as e:  # noqa: BLE001
        if not isinstance(e, (KeyboardInterrupt, SystemExit)):
            logger.critical("exo terminated due to an unhandled exception", exc_info=e)
        raise
    finally:
        logger.info("exo shutdown complete")
        logger_cleanup()


def daemonize() -> None:
    """Classic double fork; stdio goes to /dev/null (the log file keeps the record)."""
    if os.fork() > 0:
        os._exit(0)
    os.setsid()
    if os.fork() > 0:
        os._exit(0)
    sys.stdout.flush()
    sys.stderr.flush()
    with open(os.devnull, "rb", 0) as r, open(os.devnull, "ab", 0) as w:
        os.dup2(r.fileno(), 0)
        os.dup2(w.fileno(), 1)
        os.dup2(w.fileno(), 2)


def main(argv: list[str] | None = None) -> None:
    argv = list(sys.argv[1:] if argv is None else argv)
    args = Args.parse(argv)          # --help and bad flags must not need the pid lock
    if args.all_gpus:
        raise SystemExit(_spawn_per_gpu(args, argv))
    from .native.bus import load_native
    native = load_native()
    gpu_tag = "" if args.gpu is None else f".gpu{args.gpu}"
    pid_path = Path(str(constants.EXO_PID_FILE) + gpu_tag)
    pid_path.parent.mkdir(parents=True, exist_ok=True)
    try:
        pidfile = native.Pidfile(str(pid_path))
    except RuntimeError as e:
        print(f"exo is already running ({e})", file=sys.stderr)
        raise SystemExit(1) from e
    try:
        if args.legacy_daemon:
            daemonize()     # the flock travels with the descriptor across fork
        pidfile.write()
        main_inner(args)
    finally:
        pidfile.close()


if __name__ == "__main__":
    main()
