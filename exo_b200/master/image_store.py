"""TTL store for generated images served back at ``/images/{id}``.

Files live under the image cache directory for one hour (reference ``src/exo/master/image_store.py``:
TTL 1 h, listing with expiry, lazy clean-up on every access).
"""
from __future__ import annotations

import time
import uuid
from dataclasses import dataclass
from pathlib import Path

from ..shared import constants

_MIME = {"png": "image/png", "jpeg": "image/jpeg", "jpg": "image/jpeg", "webp": "image/webp"}


@dataclass(frozen=True)
class StoredImage:
    image_id: str
    path: Path
    content_type: str
    expires_at: float


class ImageStore:
    def __init__(self, directory: Path | None = None, ttl_seconds: float = 3600.0):
        self.dir = directory or constants.EXO_IMAGE_CACHE_DIR
        self.dir.mkdir(parents=True, exist_ok=True)
        self.ttl = ttl_seconds
        self.items: dict[str, StoredImage] = {}

    def store(self, data: bytes, fmt: str = "png") -> StoredImage:
        self.cleanup()
        iid = uuid.uuid4().hex
        p = self.dir / f"{iid}.{fmt}"
        p.write_bytes(data)
        it = StoredImage(iid, p, _MIME.get(fmt, "application/octet-stream"), time.time() + self.ttl)
        self.items[iid] = it
        return it

    def get(self, image_id: str) -> StoredImage | None:
        self.cleanup()
        return self.items.get(image_id)

    def list(self) -> list[StoredImage]:
        self.cleanup()
        return sorted(self.items.values(), key=lambda i: i.expires_at)

    def cleanup(self) -> None:
        now = time.time()
        for iid, it in list(self.items.items()):
            if it.expires_at <= now:
                it.path.unlink(missing_ok=True)
                del self.items[iid]
