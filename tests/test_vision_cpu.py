"""Image inputs: tower / processor / prompt splice, and the engine's embedding splice against token equivalence."""
import base64
import io

import numpy as np
import torch

from exo_b200.engine.engine import Engine
from exo_b200.engine.kv import SamplingParams
from exo_b200.models.config import preset
from exo_b200.models.weights import RandomSource, ShardSpec, build_weights
from exo_b200.worker.engines.b200.vision import ImageFeatures, VisionConfig, VisionProcessor, VisionTower, preprocess, splice

GREEDY = dict(temperature=0.0, ignore_eos=True)


def png(h: int, w: int, seed: int = 0) -> str:
    from PIL import Image
    rng = np.random.default_rng(seed)
    buf = io.BytesIO()
    Image.fromarray((rng.random((h, w, 3)) * 255).astype("uint8")).save(buf, format="PNG")
    return base64.b64encode(buf.getvalue()).decode()


def test_tower_grid_and_feature_cache():
    cfg = VisionConfig(width=64, depth=2, heads=2, out_hidden=48, max_tokens=40)
    tower = VisionTower(cfg, "cpu")
    px = preprocess(base64.b64decode(png(200, 300)), cfg)
    assert px.shape[0] == 3 and px.shape[1] % cfg.cell == 0 and px.shape[2] % cfg.cell == 0
    n = (px.shape[1] // cfg.cell) * (px.shape[2] // cfg.cell)
    assert cfg.min_tokens <= n <= cfg.max_tokens
    rows = tower(px)
    assert rows.shape == (n, 48) and torch.isfinite(rows).all()
    # wide and tall images keep their aspect in the grid
    wide = preprocess(base64.b64decode(png(60, 600)), cfg)
    assert wide.shape[2] > wide.shape[1]
    vp = VisionProcessor(tower, cache_entries=2)
    a = vp.features(png(64, 64, 1))
    b = vp.features("data:image/png;base64," + png(64, 64, 1))
    assert vp.hits == 1 and a.digest == b.digest and torch.equal(a.rows, b.rows)
    vp.features(png(64, 64, 2)), vp.features(png(64, 64, 3))
    assert len(vp.cache) == 2 and a.digest not in vp.cache            # least recently used entry dropped
    assert not torch.equal(vp.features(png(64, 64, 2)).rows, a.rows)


def test_splice_placeholders_and_front_insertion():
    f1, f2 = ImageFeatures(b"a" * 32, torch.zeros(3, 8)), ImageFeatures(b"b" * 32, torch.ones(5, 8))
    ids, emb, med = splice([1, 9, 4, 9, 6], 9, [f1, f2], fill_id=9)
    assert ids == [1, 9, 9, 9, 4, 9, 9, 9, 9, 9, 6]
    assert [(p, r.shape[0]) for p, r in emb] == [(1, 3), (5, 5)] and med == [(1, 4, f1.digest), (5, 10, f2.digest)]
    # one placeholder, two images: the second goes to the front, after the first token, and everything shifts
    ids, emb, med = splice([1, 9, 4], 9, [f1, f2], fill_id=0)
    assert ids == [1] + [0] * 5 + [0] * 3 + [4]
    assert [(p, r.shape[0]) for p, r in emb] == [(1, 5), (6, 3)]
    assert med == [(1, 6, f2.digest), (6, 9, f1.digest)]
    # no placeholder token at all
    ids, emb, med = splice([1, 4], None, [f1], fill_id=0)
    assert ids == [1, 0, 0, 0, 4] and emb[0][0] == 1


def test_engine_embedding_splice_equals_the_tokens_it_stands_for():
    """Rows given as ``embeds`` replace the token embeddings: feeding the embedding rows of tokens X over placeholder
    positions gives exactly the run of the prompt that has X there — also when the prompt is prefilled in chunks that
    cut through the region, and the prefix cache tells two images on the same placeholders apart."""
    cfg = preset("tiny-llama")
    w = build_weights(cfg, ShardSpec(), RandomSource(seed=0))
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(5, cfg.vocab, (40,), generator=g).tolist()
    stand_in = torch.randint(5, cfg.vocab, (11,), generator=g).tolist()
    start = 7
    real = prompt[:start] + stand_in + prompt[start + len(stand_in):]
    holes = prompt[:start] + [0] * len(stand_in) + prompt[start + len(stand_in):]
    rows = w.embed[torch.tensor(stand_in)]
    want = Engine(cfg, w, n_blocks=64).generate(real, SamplingParams(max_tokens=6, **GREEDY))
    for chunk in (4096, 16, 5):
        eng = Engine(cfg, w, n_blocks=64, prefill_chunk=chunk)
        rid = eng.submit(holes, SamplingParams(max_tokens=6, **GREEDY), embeds=[(start, rows)], media=[(start, start + 11, b"x" * 32)])
        got = []
        while eng.has_work:
            got += [o.token for o in eng.step() if o.req_id == rid and o.token is not None]
        assert got == want, (chunk, got, want)
    # same placeholder ids, other image: no false prefix-cache hit
    eng = Engine(cfg, w, n_blocks=64)
    first = eng.generate(holes, SamplingParams(max_tokens=4, **GREEDY))          # placeholders as plain tokens
    rid = eng.submit(holes, SamplingParams(max_tokens=4, **GREEDY), embeds=[(start, rows)], media=[(start, start + 11, b"y" * 32)])
    got = []
    while eng.has_work:
        got += [o.token for o in eng.step() if o.req_id == rid and o.token is not None]
    assert got == want[:4] and got != first
