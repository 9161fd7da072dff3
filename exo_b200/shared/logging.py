"""Process-wide logging: console at the chosen verbosity, a rotating file with everything.

Plays the part of the reference's loguru setup (``src/exo/shared/logging.py``): ``-q`` shows
warnings only, default shows info, ``-v`` debug; the log file always records debug, rotates at
a size cap and keeps a few generations; uvicorn's loggers are routed through the same handlers.
"""
from __future__ import annotations

import logging
import logging.handlers
import sys
from pathlib import Path

logger = logging.getLogger("exo")
_handlers: list[logging.Handler] = []
FORMAT = "%(asctime)s.%(msecs)03d | %(levelname)-7s | %(name)s:%(lineno)d - %(message)s"


def logger_setup(log_file: Path | None, verbosity: int = 0) -> None:
    logger_cleanup()
    level = logging.WARNING if verbosity < 0 else logging.INFO if verbosity == 0 else logging.DEBUG
    console = logging.StreamHandler(sys.stderr)
    console.setLevel(level)
    console.setFormatter(logging.Formatter(FORMAT, datefmt="%H:%M:%S"))
    _handlers.append(console)
    if log_file is not None:
        try:
            log_file.parent.mkdir(parents=True, exist_ok=True)
            fh = logging.handlers.RotatingFileHandler(log_file, maxBytes=50 << 20, backupCount=5)
            fh.setLevel(logging.DEBUG)
            fh.setFormatter(logging.Formatter(FORMAT, datefmt="%Y-%m-%d %H:%M:%S"))
            _handlers.append(fh)
        except OSError:
            pass
    root = logging.getLogger()
    root.setLevel(logging.DEBUG)
    for h in _handlers:
        root.addHandler(h)
    for name in ("uvicorn", "uvicorn.error", "uvicorn.access"):
        lg = logging.getLogger(name)
        lg.handlers.clear()
        lg.propagate = True


def logger_cleanup() -> None:
    root = logging.getLogger()
    for h in _handlers:
        root.removeHandler(h)
        try:
            h.flush()
            h.close()
        except Exception:  # noqa: BLE001
            pass
    _handlers.clear()
