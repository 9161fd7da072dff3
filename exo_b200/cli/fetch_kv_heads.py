"""Refresh ``num_key_value_heads`` (and context length) in the bundled model cards from each
model's ``config.json`` on the hub.

Counterpart of the reference's ``scripts/fetch_kv_heads.py``: tensor-parallel placement needs the
KV-head count to be divisible by the group size, so cards must carry the right number.

    python -m exo_b200.cli.fetch_kv_heads [--dry-run] [--only <substring>]
"""
from __future__ import annotations

import argparse
import asyncio
import json
import sys

from ..download import hf
from ..download.store import cache_dir
from ..shared import constants
from ..shared.cards import ModelCard


async def kv_heads_of(model_id: str) -> tuple[int | None, int]:
    d = cache_dir(model_id)
    await hf.download_file_with_retry(model_id, "main", "config.json", d)
    cfg = json.loads((d / "config.json").read_text())
    tc = cfg.get("text_config") if isinstance(cfg.get("text_config"), dict) else cfg
    return tc.get("num_key_value_heads") or tc.get("num_attention_heads"), int(tc.get("max_position_embeddings") or 0)


async def run(dry: bool, only: str) -> int:
    changed = 0
    for d in constants.builtin_card_dirs():
        for path in sorted(d.glob("*.toml")):
            card = ModelCard.load_from_path(path)
            if only and only not in str(card.model_id):
                continue
            try:
                kv, ctx = await kv_heads_of(str(card.model_id))
            except Exception as e:  # noqa: BLE001 - report and go on with the other cards
                print(f"{card.model_id}: {e}", file=sys.stderr)
                continue
            upd = {}
            if kv and kv != card.num_key_value_heads:
                upd["num_key_value_heads"] = kv
            if ctx and ctx != card.context_length:
                upd["context_length"] = ctx
            if upd:
                changed += 1
                print(f"{card.model_id}: {upd}")
                if not dry:
                    card.model_copy(update=upd).save(path)
    print(f"{changed} card(s) {'would change' if dry else 'updated'}")
    return 0


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--only", default="")
    a = ap.parse_args(argv)
    return asyncio.run(run(a.dry_run, a.only))


if __name__ == "__main__":
    raise SystemExit(main())
