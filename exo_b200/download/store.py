"""Where checkpoints live on disk: search, completeness, choosing a directory, deleting, seeding.

Directory policy of the reference (``src/exo/download/download_utils.py:152-275, 278-357``):
read-only roots are searched before writable ones; a directory counts as a model only when a
``*.safetensors.index.json`` is present and every weight file that index names exists (partial
``*.partial`` files do not count); downloads go to the first writable root with enough free
space, preferring one that already holds part of the model; deletion never touches read-only
roots.  Added here: a single-file checkpoint (``model.safetensors`` without an index) is also
complete, since small models ship that way.
"""
from __future__ import annotations

import json
import os
import shutil
from pathlib import Path

from pydantic import BaseModel

from ..shared import constants
from ..shared.base import ModelId
from ..shared.cards import ModelCard


class FileListEntry(BaseModel):
    type: str = "file"          # "file" | "directory"
    path: str
    size: int | None = None


class InsufficientDiskSpaceError(Exception):
    """No writable model directory has enough free space."""


def _roots_ro() -> tuple[Path, ...]:
    return constants.EXO_MODELS_READ_ONLY_DIRS


def _roots_rw() -> tuple[Path, ...]:
    return constants.EXO_MODELS_DIRS


def scan_model_directory(model_dir: Path, recursive: bool = True) -> list[FileListEntry] | None:
    """Files present, plus the weight files the index promises (size ``None`` when missing).
    ``None`` when the directory has no index and no single-file checkpoint."""
    index_files = list(model_dir.glob("**/*.safetensors.index.json"))
    single = [p for p in model_dir.glob("*.safetensors")] if not index_files else []
    if not index_files and not single:
        return None
    entries: dict[str, FileListEntry] = {}
    walker = os.walk(model_dir) if recursive else [(str(model_dir), [], [p.name for p in model_dir.iterdir() if p.is_file()])]
    for dirpath, _dirs, files in walker:
        for fn in files:
            if fn.endswith(".partial"):
                continue
            full = Path(dirpath) / fn
            rel = str(full.relative_to(model_dir))
            entries[rel] = FileListEntry(path=rel, size=full.stat().st_size)
    for idx in index_files:
        try:
            weight_map = json.loads(idx.read_text()).get("weight_map", {})
        except (OSError, json.JSONDecodeError):
            continue
        rel_dir = idx.parent.relative_to(model_dir)
        for fn in set(weight_map.values()):
            rel = str(rel_dir / fn) if rel_dir != Path(".") else fn
            entries.setdefault(rel, FileListEntry(path=rel, size=None))
    return list(entries.values())


def is_model_directory_complete(model_dir: Path, card: ModelCard | None = None) -> bool:
    files = scan_model_directory(model_dir)
    if files is None or any(f.size is None for f in files):
        return False
    if not (model_dir / "config.json").exists() and not any(f.path.endswith("model_index.json") for f in files):
        return False
    if card is not None and card.vision is not None and card.vision.weights_repo != str(card.model_id):
        vis = ModelId(card.vision.weights_repo).normalize()
        return any((d / vis).is_dir() and is_model_directory_complete(d / vis) for d in (*_roots_ro(), *_roots_rw()))
    return True


def resolve_existing_model(model_id: ModelId, card: ModelCard | None = None) -> Path | None:
    """A complete copy of the model in any models root (read-only roots first), or a local path."""
    if os.path.isdir(str(model_id)) and is_model_directory_complete(Path(str(model_id)), card):
        return Path(str(model_id))
    norm = ModelId(model_id).normalize()
    for root in (*_roots_ro(), *_roots_rw()):
        cand = root / norm
        if cand.is_dir() and is_model_directory_complete(cand, card):
            return cand
    return None


def is_read_only_model_dir(model_dir: Path) -> bool:
    return any(Path(model_dir).is_relative_to(d) for d in _roots_ro())


def build_model_path(model_id: ModelId) -> Path:
    return resolve_existing_model(model_id) or constants.EXO_DEFAULT_MODELS_DIR / ModelId(model_id).normalize()


def cache_dir(model_id: ModelId) -> Path:
    d = constants.EXO_DEFAULT_MODELS_DIR / "caches" / ModelId(model_id).normalize()
    d.mkdir(parents=True, exist_ok=True)
    return d


def downloaded_size(path: Path) -> int:
    if path.exists():
        return path.stat().st_size
    partial = path.with_suffix(path.suffix + ".partial")
    return partial.stat().st_size if partial.exists() else 0


def select_download_dir(required_bytes: int) -> Path:
    for root in _roots_rw():
        if not root.exists():
            continue
        try:
            if shutil.disk_usage(root).free >= required_bytes:
                return root
        except OSError:
            continue
    raise InsufficientDiskSpaceError(f"No writable model directory has {required_bytes / 1024 ** 3:.1f} GiB free. "
                                     f"Checked: {[str(d) for d in _roots_rw()]}")


def select_download_dir_for(model_id: ModelId, files: list[FileListEntry], total: int) -> Path:
    """Prefer a root that already holds part of this model (only the remainder must fit)."""
    norm = ModelId(model_id).normalize()
    for root in _roots_rw():
        sub = root / norm
        if not root.exists() or not sub.is_dir():
            continue
        have = sum(downloaded_size(sub / f.path) for f in files)
        try:
            if shutil.disk_usage(root).free >= max(total - have, 0):
                return root
        except OSError:
            continue
    constants.EXO_DEFAULT_MODELS_DIR.mkdir(parents=True, exist_ok=True)
    return select_download_dir(total)


def delete_model(model_id: ModelId) -> bool:
    norm = ModelId(model_id).normalize()
    deleted = False
    for root in _roots_rw():
        d = root / norm
        if d.exists():
            shutil.rmtree(d)
            deleted = True
    c = constants.EXO_DEFAULT_MODELS_DIR / "caches" / norm
    if c.exists():
        shutil.rmtree(c)
    return deleted


def seed_models(seed_dir: str | Path) -> list[Path]:
    """Move pre-packaged model directories (``org--name``) into the default models root."""
    dest = constants.EXO_DEFAULT_MODELS_DIR
    dest.mkdir(parents=True, exist_ok=True)
    moved = []
    src = Path(seed_dir)
    if not src.is_dir():
        return moved
    for p in src.iterdir():
        if p.is_dir() and "--" in p.name and not (dest / p.name).exists():
            try:
                shutil.move(str(p), str(dest / p.name))
                moved.append(dest / p.name)
            except OSError:
                continue
    return moved
