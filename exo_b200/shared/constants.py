"""Directories, environment switches and tunables.

Environment variable names and default locations are the reference's
(``src/exo/shared/constants.py:8-108``) so an existing installation's models, custom cards,
event logs and traces are found where they already are.  Added for this engine:
``EXO_KV_BLOCK_SIZE``, ``EXO_COLLECTIVE_TIMEOUT_US``, ``EXO_KERNEL_CHECKS``, ``EXO_GPU_MEMORY_FRACTION``.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path


def _flag(name: str, default: str = "false") -> bool:
    return os.getenv(name, default).lower() == "true"


def _xdg(env: str, fallback: str) -> Path:
    home = os.environ.get("EXO_HOME")
    if home is not None:
        return Path.home() / home
    if sys.platform != "linux":
        return Path.home() / ".exo"
    v = os.environ.get(env)
    return Path(v) / "exo" if v is not None else Path.home() / fallback / "exo"


def _colon_dirs(env: str) -> tuple[Path, ...]:
    raw = os.environ.get(env)
    return tuple(Path(p).expanduser() for p in raw.split(":") if p) if raw else ()


EXO_CONFIG_HOME = _xdg("XDG_CONFIG_HOME", ".config")
EXO_DATA_HOME = _xdg("XDG_DATA_HOME", ".local/share")
EXO_CACHE_HOME = _xdg("XDG_CACHE_HOME", ".cache")

_default_models = os.environ.get("EXO_DEFAULT_MODELS_DIR")
EXO_DEFAULT_MODELS_DIR = Path(_default_models).expanduser() if _default_models else EXO_DATA_HOME / "models"
EXO_MODELS_READ_ONLY_DIRS: tuple[Path, ...] = _colon_dirs("EXO_MODELS_READ_ONLY_DIRS")
EXO_MODELS_DIRS: tuple[Path, ...] = tuple(d for d in (EXO_DEFAULT_MODELS_DIR, *_colon_dirs("EXO_MODELS_DIRS"))
                                          if d not in frozenset(EXO_MODELS_READ_ONLY_DIRS))


def models_dirs() -> tuple[Path, ...]:
    """Every directory a checkpoint may be found in (writable first, then read-only)."""
    return (*EXO_MODELS_DIRS, *EXO_MODELS_READ_ONLY_DIRS)


PACKAGE_DIR = Path(__file__).resolve().parent.parent
_res = os.environ.get("EXO_RESOURCES_DIR")
RESOURCES_DIR = Path.home() / _res if _res else PACKAGE_DIR / "resources"
_dash = os.environ.get("EXO_DASHBOARD_DIR")
DASHBOARD_DIR = Path.home() / _dash if _dash else PACKAGE_DIR / "resources" / "dashboard"


def builtin_card_dirs() -> tuple[Path, ...]:
    return (RESOURCES_DIR / "inference_model_cards", RESOURCES_DIR / "image_model_cards")


EXO_LOG_DIR = EXO_CACHE_HOME / "exo_log"
EXO_LOG = EXO_LOG_DIR / "exo.log"
EXO_RUNNER_LOG_DIR = EXO_LOG_DIR / "runner_log"
EXO_RUNNER_STDOUT_LOG = EXO_RUNNER_LOG_DIR / "stdout.log"
EXO_RUNNER_STDERR_LOG = EXO_RUNNER_LOG_DIR / "stderr.log"
EXO_PID_FILE = EXO_CACHE_HOME / "exo.pid"
EXO_NODE_ZID = EXO_CACHE_HOME / "node_zid"
EXO_CONFIG_FILE = EXO_CONFIG_HOME / "config.toml"

TOPIC_LOCAL_EVENTS = "worker_events"
TOPIC_GLOBAL_EVENTS = "global_events"
TOPIC_ELECTION = "election_message"
TOPIC_COMMANDS = "commands"
TOPIC_DOWNLOAD_COMMANDS = "download_commands"
TOPIC_CONNECTIONS = "connection_messages"

EXO_MAX_CHUNK_SIZE = 512 * 1024
EXO_CUSTOM_MODEL_CARDS_DIR = EXO_DATA_HOME / "custom_model_cards"
EXO_EVENT_LOG_DIR = EXO_DATA_HOME / "event_log"
EXO_IMAGE_CACHE_DIR = EXO_CACHE_HOME / "images"
EXO_TRACING_CACHE_DIR = EXO_CACHE_HOME / "traces"

EXO_ENABLE_IMAGE_MODELS = _flag("EXO_ENABLE_IMAGE_MODELS")
EXO_OFFLINE = _flag("EXO_OFFLINE")
EXO_TRACING_ENABLED = _flag("EXO_TRACING_ENABLED")
ENABLE_DISAGGREGATION = _flag("ENABLE_DISAGGREGATION")
EXO_MAX_CONCURRENT_REQUESTS = int(os.getenv("EXO_MAX_CONCURRENT_REQUESTS", "8"))
EXO_MAX_INSTANCE_RETRIES = 5

# engine
EXO_KV_BLOCK_SIZE = int(os.getenv("EXO_KV_BLOCK_SIZE", "16"))
EXO_COLLECTIVE_TIMEOUT_US = int(os.getenv("EXO_COLLECTIVE_TIMEOUT_US", "2000000"))
EXO_GPU_MEMORY_FRACTION = float(os.getenv("EXO_GPU_MEMORY_FRACTION", "0.90"))
MAX_TOKENS = 32168
DEFAULT_TOP_LOGPROBS = 5
PREFILL_CHUNK = 4096
REMOTE_PREFILL_MIN_TOKENS = int(os.getenv("EXO_REMOTE_PREFILL_MIN_TOKENS", "1000"))   # shorter prompts are prefilled locally

DEFAULT_API_PORT = 52415
DEFAULT_BUS_PORT = 52414
DEFAULT_DISCOVERY_PORT = 52413
