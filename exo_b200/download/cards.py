"""Model cards from the hub: derive a card for an arbitrary repo, and search.

The reference derives a custom card by fetching ``config.json`` and the safetensors index
(``src/exo/shared/models/model_cards.py`` ``fetch_from_hf``) and searches the hub through
``huggingface_hub.list_models`` (``src/exo/api/main.py:1870-1908``).  Here both go through the
node's own hub client: the two small files land in the model's cache directory, and search is one
GET on ``/api/models``.
"""
from __future__ import annotations

import json

from ..api.types import HuggingFaceSearchResult
from ..shared.base import Memory, ModelId
from ..shared.cards import ModelCard, card_cache, card_from_local_dir
from . import hf
from .store import cache_dir, resolve_existing_model


async def fetch_card(model_id: str) -> ModelCard:
    mid = ModelId(model_id)
    known = card_cache.get(mid)
    if known is not None:
        return known
    local = resolve_existing_model(mid)
    if local is not None:
        return card_from_local_dir(mid, local)
    d = cache_dir(mid)
    await hf.download_file_with_retry(str(mid), "main", "config.json", d)
    size = 0
    try:
        await hf.download_file_with_retry(str(mid), "main", "model.safetensors.index.json", d)
    except FileNotFoundError:
        # single-file checkpoint: take the size from the listing
        files = await hf.fetch_file_list_with_cache(mid)
        size = sum(f.size or 0 for f in files if f.path.endswith(".safetensors"))
    card = card_from_local_dir(mid, d)
    if size:
        card = card.model_copy(update={"storage_size": Memory.from_bytes(size)})
    return card


async def search_hub(query: str = "", limit: int = 20) -> list[HuggingFaceSearchResult]:
    params = {"sort": "downloads", "direction": "-1", "limit": str(limit), "filter": "safetensors"}
    if query:
        params["search"] = query
    async with hf.session("short") as s, s.get(f"{hf.hf_endpoint()}/api/models", params=params, headers=hf.auth_headers()) as r:
        if r.status != 200:
            raise RuntimeError(f"hub answered {r.status}")
        rows = json.loads(await r.read())
    return [HuggingFaceSearchResult(id=m.get("id") or m.get("modelId", ""), author=m.get("author") or "",
                                    downloads=m.get("downloads") or 0, likes=m.get("likes") or 0,
                                    last_modified=str(m.get("lastModified") or ""), tags=list(m.get("tags") or []))
            for m in rows]
