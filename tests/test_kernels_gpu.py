"""Each sm_100a kernel against the plain PyTorch fp32 definition of the same op."""
import math

import pytest
import torch

from exo_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from exo_b200.ops import cuda
    cuda.load()
    return cuda


def close(a, b, rtol=2e-2, atol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    scale = b.abs().max().item()
    assert err <= atol + rtol * scale, f"max err {err} vs scale {scale}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,cols", [(1, 4096), (5, 256), (33, 7168)])
def test_rmsnorm(K, dtype, rows, cols):
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(rows, cols, device="cuda", generator=g).to(dtype)
    r = torch.randn(rows, cols, device="cuda", generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(cols, device="cuda", generator=g)).to(dtype)
    o, h = K.rmsnorm(x, w, 1e-5, r)
    ro, rh = ref.rmsnorm(x.float(), w.float(), 1e-5, r.float())
    close(h, rh, 1e-2, 1e-2)
    close(o, ro)
    o2, _ = K.rmsnorm(x, w, 1e-5)
    close(o2, ref.rmsnorm(x.float(), w.float(), 1e-5)[0])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("N,K_", [(512, 256), (6144, 4096), (1001 * 2, 1024)])
def test_linear_small(K, dtype, M, N, K_):
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(M, K_, device="cuda", generator=g).to(dtype)
    w = (torch.randn(N, K_, device="cuda", generator=g) / math.sqrt(K_)).to(dtype)
    b = torch.randn(N, device="cuda", generator=g).to(dtype)
    r = torch.randn(M, N, device="cuda", generator=g).to(dtype)
    nw = (1 + 0.1 * torch.randn(K_, device="cuda", generator=g)).to(dtype)
    close(K.linear(x, w), ref.linear(x.float(), w.float()))
    close(K.linear(x, w, b, r), ref.linear(x.float(), w.float(), b.float(), r.float()))
    want = ref.linear(ref.rmsnorm(x.float(), nw.float(), 1e-5)[0], w.float())
    close(K.linear(x, w, None, None, nw, 1e-5), want)
    close(K.linear(x, w, None, None, nw, 1e-5, True), ref.swiglu(want))


@pytest.mark.parametrize("M", [1, 2])
@pytest.mark.parametrize("N,K_", [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336), (16032, 4096),
                                   (4096, 512), (4100, 1024), (1002 * 2, 28672)])
def test_gemv_stream(K, M, N, K_):
    g = torch.Generator(device="cuda").manual_seed(7)
    x = torch.randn(M, K_, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K_, device="cuda", generator=g) / math.sqrt(K_)).bfloat16()
    b = torch.randn(N, device="cuda", generator=g).bfloat16()
    r = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    nw = (1 + 0.1 * torch.randn(K_, device="cuda", generator=g)).bfloat16()
    assert K.load().exo_gemv_stream_supported(M, N, K_, 0) == (0 if (M == 2 and K_ > 16384) else 1)
    close(K.linear(x, w), ref.linear(x.float(), w.float()))
    close(K.linear(x, w, b, r), ref.linear(x.float(), w.float(), b.float(), r.float()))
    want = ref.linear(ref.rmsnorm(x.float(), nw.float(), 1e-5)[0], w.float())
    close(K.linear(x, w, None, None, nw, 1e-5), want)
    close(K.linear(x, w, None, None, nw, 1e-5, True), ref.swiglu(want))
    K.gemm_check()
    again = K.linear(x, w, b, r)
    assert torch.equal(again, K.linear(x, w, b, r))


@pytest.mark.parametrize("M,N,K_", [(9, 256, 64), (5, 4096, 4096), (16, 4096, 4096), (32, 6144, 4096), (48, 1024, 14336),
                                     (100, 384, 512), (128, 4096, 1024), (300, 2048, 4096), (2048, 1536, 2048), (513, 1000, 320), (257, 384, 4096),
                                     (17, 128256 // 8, 4096)])
def test_gemm_tcgen05(K, M, N, K_):
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(M, K_, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K_, device="cuda", generator=g) / math.sqrt(K_)).bfloat16()
    b = torch.randn(N, device="cuda", generator=g).bfloat16()
    r = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    got = K.gemm_bf16(x, w)
    K.gemm_check()
    close(got, ref.linear(x.float(), w.float()))
    got = K.gemm_bf16(x, w, b, r)
    K.gemm_check()
    close(got, ref.linear(x.float(), w.float(), b.float(), r.float()))
    # in-place residual (out aliases residual is not used by the binding, but repeated calls must agree)
    again = K.gemm_bf16(x, w, b, r)
    assert torch.equal(got, again)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_linear_tiled_fp32_path(K, dtype):
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(37, 200, device="cuda", generator=g).to(dtype)
    w = (torch.randn(91, 200, device="cuda", generator=g) / 14).to(dtype)
    import exo_b200.ops.cuda as c
    saved, c.gemm_impl = c.gemm_impl, None
    try:
        close(K.linear(x, w), ref.linear(x.float(), w.float()))
    finally:
        c.gemm_impl = saved


def _paged_setup(dtype, B, Hq, Hkv, D, lens, qlens, bs=16, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    max_blocks = max(-(-n // bs) for n in lens) + 1
    n_blocks = B * max_blocks + 1
    kc = torch.randn(n_blocks, bs, Hkv, D, device="cuda", generator=g).to(dtype)
    vc = torch.randn(n_blocks, bs, Hkv, D, device="cuda", generator=g).to(dtype)
    perm = torch.randperm(n_blocks - 1, device="cuda", generator=g) + 1
    bt = perm[: B * max_blocks].view(B, max_blocks).int()
    T = sum(qlens)
    q = torch.randn(T, Hq, D, device="cuda", generator=g).to(dtype)
    cu = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), device="cuda", dtype=torch.int32)
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    return q, kc, vc, bt, sl, cu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (4, 2, 64), (8, 1, 128), (16, 16, 64), (16, 2, 256), (4, 2, 256), (2, 2, 256),
                                        (8, 2, 512), (4, 4, 512), (2, 1, 512)])
def test_paged_decode(K, dtype, Hq, Hkv, D):
    lens = [1, 17, 300, 2049]
    q, kc, vc, bt, sl, cu = _paged_setup(dtype, 4, Hq, Hkv, D, lens, [1] * 4)
    got = K.paged_attention(q, kc, vc, bt, sl, cu, D ** -0.5, max_q_len=1)
    want = ref.paged_attention(q.float(), kc.float(), vc.float(), bt, sl, cu, D ** -0.5)
    close(got, want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("Hq,Hkv,D", [(8, 2, 512), (2, 1, 512), (4, 2, 256)])
def test_ragged_attention_wide_heads(K, dtype, Hq, Hkv, D):
    """Prompt-shaped queries over 256- and 512-wide heads (the generic kernel: these widths are not on the tensor cores)."""
    lens, qlens = [70, 33, 5], [40, 33, 1]
    q, kc, vc, bt, sl, cu = _paged_setup(dtype, 3, Hq, Hkv, D, lens, qlens)
    got = K.paged_attention(q, kc, vc, bt, sl, cu, 1.0 / 16, max_q_len=max(qlens))
    want = ref.paged_attention(q.float(), kc.float(), vc.float(), bt, sl, cu, 1.0 / 16)
    close(got, want)


def test_rope_append_unit_norm_v_and_query_only(K):
    """The Gemma-4 forms of the fused split/norm/RoPE/append: v normalised without a weight, full-head rotation with
    zero frequencies, 512-wide heads, and a layer that reads another layer's cache (q only)."""
    g = torch.Generator(device="cuda").manual_seed(3)
    from exo_b200 import ops
    from exo_b200.models.config import RopeConfig
    for dtype, D, hq, hkv in ((torch.float32, 512, 2, 1), (torch.bfloat16, 128, 4, 2)):
        T = 9
        inv = ref.rope_inv_freq(D, RopeConfig(theta=1e6, kind="proportional", partial_rotary_factor=0.25))[0].cuda()
        qkv = torch.randn(T, (hq + 2 * hkv) * D, device="cuda", generator=g).to(dtype)
        qn, kn = (1 + 0.1 * torch.randn(2, D, device="cuda", generator=g)).to(dtype)
        pos = torch.arange(3, 3 + T, device="cuda", dtype=torch.int32)
        slots = (16 + torch.arange(T, device="cuda")).int()
        kc, vc = (torch.zeros(4, 16, hkv, D, device="cuda", dtype=dtype) for _ in range(2))
        q = K.qk_rope_append(qkv, pos, inv, 1.0, hq, hkv, D, kc, vc, slots, qn, kn, 1e-6, True)
        kc2, vc2 = kc.cpu().float() * 0, vc.cpu().float() * 0
        q2 = ops.qk_rope_append(qkv.cpu().float(), pos.cpu(), inv.cpu(), 1.0, hq, hkv, D, kc2, vc2, slots.cpu(), qn.cpu().float(),
                                kn.cpu().float(), 1e-6, True)
        close(q.cpu(), q2)
        close(kc.cpu(), kc2)
        close(vc.cpu(), vc2)
        only_q = K.qk_rope_append(qkv[:, :hq * D], pos, inv, 1.0, hq, 0, D, kc, vc, slots, qn, qn, 1e-6)
        close(only_q.cpu(), q2)


def test_geglu(K):
    g = torch.Generator(device="cuda").manual_seed(4)
    for dtype in (torch.float32, torch.bfloat16):
        x = (2 * torch.randn(33, 2 * 96, device="cuda", generator=g)).to(dtype)
        close(K.geglu(x), ref.geglu(x.float()))


def test_paged_decode_window_and_sinks(K):
    lens = [5, 200, 1000]
    q, kc, vc, bt, sl, cu = _paged_setup(torch.bfloat16, 3, 8, 2, 64, lens, [1] * 3)
    sinks = torch.randn(8, device="cuda")
    got = K.paged_attention(q, kc, vc, bt, sl, cu, 0.125, sliding_window=128, sinks=sinks, max_q_len=1)
    want = ref.paged_attention(q.float(), kc.float(), vc.float(), bt, sl, cu, 0.125, 128, sinks)
    close(got, want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_paged_ragged_prefill(K, dtype):
    lens, qlens = [40, 130, 64, 7], [40, 30, 1, 7]
    q, kc, vc, bt, sl, cu = _paged_setup(dtype, 4, 8, 2, 64, lens, qlens)
    got = K.paged_attention(q, kc, vc, bt, sl, cu, 0.125, max_q_len=40)
    want = ref.paged_attention(q.float(), kc.float(), vc.float(), bt, sl, cu, 0.125)
    close(got, want)


@pytest.mark.parametrize("window", [0, 300])
@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (4, 4), (16, 8), (8, 1)])
def test_decode_attention_tcgen05(K, Hq, Hkv, window):
    """bf16 / head_dim 128 / 16-key pages decode goes through the tensor-core split-KV kernel:
    contexts shorter than a block, longer than the 3-stage ring, not multiples of anything."""
    from exo_b200.ops import cuda as c
    lens = [1, 127, 128, 129, 1000, 5003]
    q, kc, vc, bt, sl, cu = _paged_setup(torch.bfloat16, 6, Hq, Hkv, 128, lens, [1] * 6, seed=5)
    got = K.paged_attention(q, kc, vc, bt, sl, cu, 128 ** -0.5, sliding_window=window, max_q_len=1)
    torch.cuda.synchronize()
    c.gemm_check()
    want = ref.paged_attention(q.float(), kc.float(), vc.float(), bt, sl, cu, 128 ** -0.5, window)
    close(got, want)
    again = K.paged_attention(q, kc, vc, bt, sl, cu, 128 ** -0.5, sliding_window=window, max_q_len=1)
    assert torch.equal(got, again)      # tickets were left clean and the merge order is fixed


@pytest.mark.parametrize("Hq,Hkv", [(12, 1), (24, 2)])
def test_attention_with_twelve_query_heads_per_kv_head(K, Hq, Hkv):
    """Step-3.5's sliding-window layers under tensor parallelism: 12 query heads share a KV head (not a power of two), with
    a window, in decode and in prompt-shaped steps."""
    from exo_b200.ops import cuda as c
    lens = [1, 127, 129, 1000, 3001]
    q, kc, vc, bt, sl, cu = _paged_setup(torch.bfloat16, 5, Hq, Hkv, 128, lens, [1] * 5, seed=7)
    got = K.paged_attention(q, kc, vc, bt, sl, cu, 128 ** -0.5, sliding_window=512, max_q_len=1)
    close(got, ref.paged_attention(q.float(), kc.float(), vc.float(), bt, sl, cu, 128 ** -0.5, 512))
    lens, qlens = [300, 777, 1, 700], [300, 260, 1, 517]
    q, kc, vc, bt, sl, cu = _paged_setup(torch.bfloat16, 4, Hq, Hkv, 128, lens, qlens, seed=8)
    got = K.paged_attention(q, kc, vc, bt, sl, cu, 128 ** -0.5, sliding_window=200, max_q_len=max(qlens))
    torch.cuda.synchronize()
    c.gemm_check()
    close(got, ref.paged_attention(q.float(), kc.float(), vc.float(), bt, sl, cu, 128 ** -0.5, 200))


@pytest.mark.parametrize("window", [0, 200])
@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (4, 4)])
def test_prefill_attention_tcgen05(K, Hq, Hkv, window):
    """head_dim 128 / 16-key pages take the tensor-core kernel: fresh prompts, a chunk on top of
    cached context, a decode row in the same step, lengths that are not multiples of the tiles."""
    from exo_b200.ops import cuda as c
    lens, qlens = [300, 777, 129, 1, 2048 + 5], [300, 260, 129, 1, 517]
    q, kc, vc, bt, sl, cu = _paged_setup(torch.bfloat16, 5, Hq, Hkv, 128, lens, qlens, seed=3)
    before = c.launch_count
    got = K.paged_attention(q, kc, vc, bt, sl, cu, 128 ** -0.5, sliding_window=window, max_q_len=max(qlens))
    assert c.launch_count - before == 1          # one launch: the generic path needs two
    torch.cuda.synchronize()
    c.gemm_check()
    want = ref.paged_attention(q.float(), kc.float(), vc.float(), bt, sl, cu, 128 ** -0.5, window)
    close(got, want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("D,qknorm", [(128, False), (64, True), (128, True)])
def test_qk_rope_append(K, dtype, D, qknorm):
    from exo_b200.models.config import RopeConfig
    g = torch.Generator(device="cuda").manual_seed(4)
    T, nq, nkv, bs, nb = 19, 6, 2, 16, 8
    qkv = torch.randn(T, (nq + 2 * nkv) * D, device="cuda", generator=g).to(dtype)
    pos = torch.randint(0, 5000, (T,), device="cuda", generator=g).int()
    slots = (torch.randperm(nb * bs - bs, device="cuda", generator=g)[:T] + bs).int()
    inv, ms = ref.rope_inv_freq(D, RopeConfig(theta=500000.0))
    inv = inv.cuda()
    kc = torch.zeros(nb, bs, nkv, D, device="cuda", dtype=dtype)
    vc = torch.zeros_like(kc)
    qn = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(dtype) if qknorm else None
    kn = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(dtype) if qknorm else None
    q = K.qk_rope_append(qkv, pos, inv, ms, nq, nkv, D, kc, vc, slots, qn, kn, 1e-6)
    qf, kf, vf = qkv.float().split((nq * D, nkv * D, nkv * D), -1)
    qf, kf, vf = qf.view(T, nq, D), kf.view(T, nkv, D), vf.view(T, nkv, D)
    if qknorm:
        qf, kf = ref.head_rmsnorm(qf, qn.float(), 1e-6), ref.head_rmsnorm(kf, kn.float(), 1e-6)
    qf, kf = ref.rope(qf, pos, inv, ms), ref.rope(kf, pos, inv, ms)
    close(q, qf)
    close(kc.view(-1, nkv, D)[slots.long()], kf)
    close(vc.view(-1, nkv, D)[slots.long()], vf, 1e-3, 1e-3)


def test_swiglu_embedding_argmax(K):
    g = torch.Generator(device="cuda").manual_seed(5)
    gu = torch.randn(7, 2 * 300, device="cuda", generator=g).bfloat16()
    close(K.swiglu(gu), ref.swiglu(gu.float()))
    close(K.swiglu(gu, 0.6), ref.swiglu(gu.float(), 0.6))                       # capped gate, clamped up projection
    assert float(K.swiglu(gu, 0.6).float().abs().max()) <= 0.36 + 1e-3 and float(K.swiglu(gu).float().abs().max()) > 0.5
    table = torch.randn(1000, 256, device="cuda", generator=g).bfloat16()
    ids = torch.randint(0, 1000, (33,), device="cuda", generator=g).int()
    assert torch.equal(K.embedding(table, ids), table[ids.long()])
    logits = torch.randn(9, 128256, device="cuda", generator=g).bfloat16()
    assert torch.equal(K.argmax(logits).long(), logits.float().argmax(-1))


@pytest.mark.parametrize("V", [1000, 32000, 128256])
def test_sample_matches_reference(K, V):
    g = torch.Generator(device="cuda").manual_seed(6)
    B = 16
    logits = (3 * torch.randn(B, V, device="cuda", generator=g)).float()
    temp = torch.tensor([0.0, 0.7, 1.0, 1.3] * 4, device="cuda")
    top_k = torch.tensor([0, 0, 50, 5] * 4, device="cuda", dtype=torch.int32)
    top_p = torch.tensor([1.0, 0.9, 1.0, 0.5] * 4, device="cuda")
    min_p = torch.tensor([0.0, 0.05, 0.0, 0.0] * 4, device="cuda")
    u = torch.rand(B, device="cuda", generator=g)
    got = K.sample(logits, temp, top_k, top_p, min_p, u).long()
    want = ref.sample(logits, temp, top_k, top_p, min_p, u)
    # fp ordering differences can move a draw that sits exactly on a CDF edge: allow one miss,
    # and require that every sampled token is in the reference keep set
    assert (got == want).sum().item() >= B - 1, (got, want)
    probs = torch.softmax(logits / temp.clamp_min(1e-6)[:, None], -1)
    assert (probs.gather(1, got[:, None]) > 0).all()


def _keep_set(logits, temp, top_k, top_p, min_p):
    """Boolean keep mask of the reference filter chain, fp32."""
    V = logits.shape[1]
    probs = torch.softmax(logits.float() / temp.clamp_min(1e-6)[:, None], -1)
    sp, si = probs.sort(-1, descending=True)
    k = torch.where(top_k > 0, top_k, torch.full_like(top_k, V))[:, None]
    keep = (torch.arange(V, device=logits.device)[None] < k) & ((sp.cumsum(-1) - sp) < top_p[:, None]) \
        & (sp >= min_p[:, None] * sp[:, :1])
    keep[:, 0] = True
    return torch.zeros_like(keep).scatter_(1, si, keep), probs


@pytest.mark.parametrize("shape", ["peaked", "flat", "masked"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sample_distribution_shapes(K, shape, dtype):
    """Peaked rows (what a trained model emits), nearly flat rows (random weights: the boundary bin overflows and is histogrammed
    a second time; bf16 rows, full of equal values, still end in the bisection kernel) and rows with -inf entries, over the filter settings the API exposes."""
    g = torch.Generator(device="cuda").manual_seed(11)
    B, V = 32, 128256
    if shape == "peaked":
        logits = torch.randn(B, V, device="cuda", generator=g) * 2.0
        hot = torch.randint(0, V, (B, 40), device="cuda", generator=g)
        logits.scatter_(1, hot, 12.0 + 3.0 * torch.rand(B, 40, device="cuda", generator=g))
    elif shape == "flat":
        logits = torch.randn(B, V, device="cuda", generator=g) * 0.05
    else:
        logits = torch.randn(B, V, device="cuda", generator=g) * 3.0
        logits[:, V // 2:] = float("-inf")
    logits = logits.to(dtype)
    temp = torch.tensor([0.7, 1.0, 0.3, 1.5, 0.0, 0.7, 1.0, 0.6] * 4, device="cuda")
    top_k = torch.tensor([0, 40, 0, 0, 0, 20, 1, 0] * 4, device="cuda", dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 0.95, 0.8, 1.0, 0.9, 1.0, 0.999] * 4, device="cuda")
    min_p = torch.tensor([0.05, 0.0, 0.0, 0.02, 0.0, 0.05, 0.0, 0.0] * 4, device="cuda")
    u = torch.rand(B, device="cuda", generator=g)
    got = K.sample(logits, temp, top_k, top_p, min_p, u).long()
    again = K.sample(logits, temp, top_k, top_p, min_p, u).long()
    assert torch.equal(got, again)                      # fixed-point sums: the same draw every time
    want = ref.sample(logits, temp, top_k, top_p, min_p, u)
    keep, probs = _keep_set(logits, temp, top_k, top_p, min_p)
    sampled = temp > 0
    assert torch.equal(got[~sampled], want[~sampled])
    # every draw comes from the reference keep set, bar ties at its edge (bf16 logits repeat values): the drawn token's
    # probability is then at least the smallest kept one
    floor = torch.where(keep, probs, torch.ones_like(probs)).min(-1).values
    assert (probs.gather(1, got[:, None])[:, 0] >= floor * (1 - 1e-5)).all()
    if dtype == torch.bfloat16:
        return          # bf16 logits repeat values: which of several equal tokens a rank-based top-k keeps is arbitrary
    # and it is the same token as the fp32 inverse CDF except where the draw sits on an edge of the CDF
    assert (got == want).sum().item() >= B - 3, (got, want)
    # the position of the draw in the kept CDF matches the uniform number
    kept = probs * keep
    cdf = kept.cumsum(-1) / kept.sum(-1, keepdim=True)
    hi = cdf.gather(1, got[:, None])[:, 0]
    lo = hi - (kept / kept.sum(-1, keepdim=True)).gather(1, got[:, None])[:, 0]
    ok = (u >= lo - 1e-4) & (u <= hi + 1e-4)
    assert ok[sampled].all(), (u, lo, hi)


@pytest.mark.parametrize("kind,E,k,n_group,topk_group,dtype", [
    ("softmax", 128, 8, 1, 1, torch.bfloat16), ("softmax", 60, 4, 1, 1, torch.float32),
    ("sigmoid", 256, 8, 8, 4, torch.float32), ("sigmoid", 64, 6, 1, 1, torch.bfloat16)])
def test_moe_route(K, kind, E, k, n_group, topk_group, dtype):
    g = torch.Generator(device="cuda").manual_seed(1)
    # distinct values in every row, also after rounding to bf16: the top-k has no ties to break
    logits = torch.stack([torch.randperm(E, device="cuda", generator=g) for _ in range(37)]).float().mul(6.0 / E).sub(3.0).to(dtype)
    bias = 0.1 * torch.randn(E, device="cuda", generator=g) if kind == "sigmoid" else None
    w, ids = K.moe_route(logits, k, kind, True, bias, n_group, topk_group, 2.5)
    rw, rids = ref.moe_route(logits, k, kind, True, bias, n_group, topk_group, 2.5)
    assert w.dtype == torch.float32 and ids.dtype == torch.int32
    assert torch.equal(ids.sort(-1)[0], rids.sort(-1)[0])
    assert torch.equal(ids, rids)
    close(w, rw, 1e-4, 1e-5)
    w2, _ = K.moe_route(logits, k, kind, False, bias, n_group, topk_group, 1.0)
    close(w2, ref.moe_route(logits, k, kind, False, bias, n_group, topk_group, 1.0)[0], 1e-4, 1e-5)


@pytest.mark.parametrize("T,E,k,H,F,offset,E_all", [
    (1, 8, 2, 256, 128, 0, 8), (3, 16, 4, 512, 192, 16, 64),            # grouped GEMVs
    (40, 8, 2, 256, 128, 0, 8), (300, 16, 8, 512, 384, 32, 64), (2048, 4, 2, 256, 256, 0, 4),   # grouped tcgen05 GEMMs, one-block plan
    (3000, 4, 2, 256, 256, 0, 4)])                                                                 # more than 4096 pairs: multi-kernel plan
def test_moe_experts(K, T, E, k, H, F, offset, E_all):
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    wgu = (torch.randn(E, 2 * F, H, device="cuda", generator=g) / math.sqrt(H)).bfloat16()
    wd = (torch.randn(E, H, F, device="cuda", generator=g) / math.sqrt(F)).bfloat16()
    logits = torch.randn(T, E_all, device="cuda", generator=g)
    w, ids = ref.moe_route(logits, k, "softmax", True)
    out = K.moe_experts(x, wgu, wd, w, ids, offset)
    want = ref.moe_experts(x, wgu, wd, w, ids, offset)
    assert K.load().exo_gemm_last_error() == 0
    close(out, want, 2e-2, 2e-2)
    # the same call again (plan scratch and tensor maps are reused) gives the same bits
    assert torch.equal(out, K.moe_experts(x, wgu, wd, w, ids, offset))


@pytest.mark.parametrize("act", ["gelu_tanh", "relu2"])
@pytest.mark.parametrize("T,E,k,H,F,offset,E_all", [(2, 8, 2, 256, 128, 0, 8), (3, 16, 4, 512, 192, 16, 64),
                                                     (300, 16, 8, 512, 384, 32, 64), (2048, 4, 2, 256, 320, 0, 4)])
def test_moe_experts_other_activations(K, act, T, E, k, H, F, offset, E_all):
    """GeGLU experts (Gemma-4) and non-gated relu^2 experts (Nemotron-H: one up projection of F rows) on the grouped GEMV
    and the grouped tcgen05 GEMM paths."""
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    rows = F if act == "relu2" else 2 * F
    wup = (torch.randn(E, rows, H, device="cuda", generator=g) / math.sqrt(H)).bfloat16()
    wd = (torch.randn(E, H, F, device="cuda", generator=g) / math.sqrt(F)).bfloat16()
    logits = torch.randn(T, E_all, device="cuda", generator=g)
    w, ids = ref.moe_route(logits, k, "softmax", True)
    out = K.moe_experts(x, wup, wd, w, ids, offset, None, act)
    want = ref.moe_experts(x, wup, wd, w, ids, offset, act)
    assert K.load().exo_gemm_last_error() == 0
    close(out, want, 2e-2, 2e-2)


@pytest.mark.parametrize("T,E,k,H,F,offset,E_all", [(2, 8, 2, 256, 128, 0, 8), (300, 16, 8, 512, 384, 32, 64)])
def test_moe_experts_clamped_swiglu(K, T, E, k, H, F, offset, E_all):
    """Step-3.5's clamped SwiGLU in the routed experts: grouped GEMV and grouped tcgen05 paths, bf16 and block-scaled fp8."""
    from exo_b200.ops import quant
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    wgu = (torch.randn(E, 2 * F, H, device="cuda", generator=g) / math.sqrt(H)).bfloat16()
    wd = (torch.randn(E, H, F, device="cuda", generator=g) / math.sqrt(F)).bfloat16()
    w, ids = ref.moe_route(torch.randn(T, E_all, device="cuda", generator=g), k, "softmax", True)
    lim = 0.4
    out = K.moe_experts(x, wgu, wd, w, ids, offset, None, "silu", lim)
    want = ref.moe_experts(x, wgu, wd, w, ids, offset, "silu", lim)
    assert K.load().exo_gemm_last_error() == 0
    close(out, want, 2e-2, 2e-2)
    plain = ref.moe_experts(x, wgu, wd, w, ids, offset)
    assert float((want.float() - plain.float()).abs().max()) > 0.05           # the limit bites at these magnitudes
    if H % 64 == 0 and F % 128 == 0:
        qgu, qd = quant.quantize(wgu, "mxfp8"), quant.quantize(wd, "mxfp8")
        out8 = K.moe_experts(x, qgu, qd, w, ids, offset, None, "silu", lim)
        want8 = ref.moe_experts(x, qgu, qd, w, ids, offset, "silu", lim)
        close(out8, want8, 3e-2, 3e-2)


@pytest.mark.parametrize("kind", ["mxfp8", "dsfp8"])
@pytest.mark.parametrize("M,N,K_", [(1, 256, 256), (5, 384, 1024), (32, 1000, 4096), (200, 512, 96), (300, 640, 2048)])
def test_gemm_fp8_weights(K, kind, M, N, K_):
    from exo_b200.ops import quant
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(M, K_, device="cuda", generator=g).bfloat16()
    # magnitudes spread over several octaves per block so that every block scale and the subnormal codes are exercised
    w = torch.randn(N, K_, device="cuda", generator=g) * torch.exp2(torch.randint(-6, 3, (N, 1), device="cuda", generator=g).float())
    wq = quant.quantize(w.bfloat16(), kind)
    bias = torch.randn(N, device="cuda", generator=g).bfloat16()
    res = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    want = ref.linear(x.float(), wq, bias.float(), res.float())
    out = K.linear(x, wq, bias, res)
    assert K.load().exo_gemm_last_error() == 0
    close(out, want, 1e-2, 1e-2)
    # the other operand form (f16 on both sides of the MMA by default, bf16 as the alternative) agrees
    old_min, K.FP8_F16_MIN_WEIGHTS = K.FP8_F16_MIN_WEIGHTS, 0          # small test shapes take the f16 form too
    try:
        other = K.linear(x, wq, bias, res)
    finally:
        K.FP8_F16_MIN_WEIGHTS = old_min
    assert K.load().exo_gemm_last_error() == 0
    close(other, want, 1e-2, 1e-2)
    # against the unquantised weights the error is the fp8 rounding (2^-4 relative per weight, averaged down by the sum)
    close(K.linear(x, wq), ref.linear(x.float(), w.bfloat16().float()), 5e-2, 5e-2)
    sw = K.linear(x, quant.quantize(w[: N // 2 * 2].bfloat16(), kind), swiglu_out=True)
    close(sw, ref.swiglu(ref.linear(x, quant.quantize(w[: N // 2 * 2].bfloat16(), kind))), 3e-2, 3e-2)


@pytest.mark.parametrize("kind", ["mxfp8", "dsfp8"])
@pytest.mark.parametrize("T,E,k,H,F,offset,E_all", [
    (2, 8, 2, 256, 128, 0, 8), (300, 16, 8, 512, 384, 32, 64), (2500, 4, 2, 256, 256, 0, 4),
    # a handful of tokens take the streaming GEMV pair: an expert-parallel shard (most pairs live elsewhere), reduction
    # lengths that are not a multiple of the 16-tile unroll, every expert local
    (1, 8, 8, 7168, 2048, 8, 64), (4, 8, 8, 7168, 2048, 8, 64), (3, 16, 4, 2048, 512, 0, 16), (4, 4, 2, 1088, 384, 0, 4)])
def test_moe_experts_fp8(K, kind, T, E, k, H, F, offset, E_all):
    from exo_b200.ops import quant
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    wgu = quant.quantize((torch.randn(E, 2 * F, H, device="cuda", generator=g) / math.sqrt(H)).bfloat16(), kind)
    wd = quant.quantize((torch.randn(E, H, F, device="cuda", generator=g) / math.sqrt(F)).bfloat16(), kind)
    logits = torch.randn(T, E_all, device="cuda", generator=g)
    w, ids = ref.moe_route(logits, k, "softmax", True)
    want = ref.moe_experts(x, wgu, wd, w, ids, offset)
    for f16 in (True, False):       # f16 operands on both sides of the MMAs (default) and the bf16 form
        K.fp8_f16_operands = f16
        try:
            out = K.moe_experts(x, wgu, wd, w, ids, offset)
        finally:
            K.fp8_f16_operands = True
        assert K.load().exo_gemm_last_error() == 0
        close(out, want, 2e-2, 2e-2)


@pytest.mark.parametrize("M,F,K_", [(256, 512, 256), (700, 1792, 1024), (2048, 1000, 512)])
def test_gemm_tcgen05_fused_swiglu(K, M, F, K_):
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(M, K_, device="cuda", generator=g).bfloat16()
    w = (torch.randn(2 * F, K_, device="cuda", generator=g) / math.sqrt(K_)).bfloat16()
    got = K.gemm_bf16(x, w, swiglu_out=True)
    K.gemm_check()
    assert got.shape == (M, F)
    close(got, ref.swiglu(ref.linear(x, w)), 2e-2, 2e-2)
    K.use_fused_swiglu = False
    try:
        unfused = K.gemm_bf16(x, w, swiglu_out=True)
    finally:
        K.use_fused_swiglu = True
    close(got, unfused, 1e-2, 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hk,hv,dk,dv,lens", [
    (2, 4, 32, 32, [5, 1, 70]),          # toy heads; a sequence longer than one chunk of the chunked definition
    (2, 2, 64, 64, [1, 1, 1, 1]),        # decode-shaped: one token per sequence
    (4, 8, 128, 128, [130, 1, 17]),      # Qwen3-Next head sizes (512-thread CTAs)
])
def test_gated_delta_rule(K, dtype, hk, hv, dk, dv, lens):
    """Convolution + recurrence + gated norm against the fp32 definition, over two consecutive steps: the second step
    continues every sequence from the state the first one left in its seat (one sequence restarts from position 0)."""
    g = torch.Generator(device="cuda").manual_seed(1)
    B, C, taps, seats_n = len(lens), 2 * hk * dk + hv * dv, 4, 8
    W = C + hv * dv + 2 * hv
    conv_w = torch.randn(C, taps, device="cuda", generator=g) * 0.5
    a_log = torch.randn(hv, device="cuda", generator=g) * 0.5
    dt_bias = torch.randn(hv, device="cuda", generator=g) * 0.5
    norm_w = (1 + 0.1 * torch.randn(dv, device="cuda", generator=g)).to(dtype)
    seats = torch.tensor([3, 1, 5, 2][:B], dtype=torch.int32, device="cuda")
    conv_k = torch.randn(seats_n, C, taps - 1, device="cuda", generator=g).to(dtype)          # stale content of the seats
    rec_k = torch.randn(seats_n, hv, dk, dv, device="cuda", generator=g)
    conv_r, rec_r = conv_k.clone(), rec_k.clone()
    start = [0] * B
    for step, step_lens in enumerate((lens, [3] * B)):
        T = sum(step_lens)
        cu = torch.tensor([0] + list(torch.tensor(step_lens).cumsum(0)), dtype=torch.int32, device="cuda")
        if step == 1:
            start[0] = 0                                                                      # seat reused by a new sequence
        pos = torch.cat([torch.arange(s, s + n) for s, n in zip(start, step_lens)]).to(torch.int32).cuda()
        proj = torch.randn(T, W, device="cuda", generator=g).to(dtype)
        got = K.gated_delta(proj, conv_w, a_log, dt_bias, norm_w, 1e-6, conv_k, rec_k, seats, cu, pos, hk, hv, dk, dv)
        want = ref.gated_delta(proj.float(), conv_w, a_log, dt_bias, norm_w.float(), 1e-6, conv_r, rec_r, seats, cu, pos,
                               hk, hv, dk, dv)
        tol = 3e-2 if dtype == torch.bfloat16 else 2e-3
        close(got, want, tol, tol)
        used = seats.long()
        close(rec_k[used], rec_r[used], tol, tol)
        close(conv_k[used], conv_r[used], 1e-2, 1e-2)
        start = [s + n for s, n in zip(start, step_lens)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("groups,heads,d_state,head_dim,lens", [(2, 8, 32, 32, [5, 1, 70]), (1, 4, 128, 64, [40, 1, 1, 1]),
                                                                 (8, 16, 128, 64, [130, 17])])
def test_mamba2(K, dtype, groups, heads, d_state, head_dim, lens):
    """Mamba-2 mixer (convolution with bias, state-space recurrence, skip, grouped gated norm) against the fp32 definition
    over two consecutive steps; the second continues from the seats' state."""
    g = torch.Generator(device="cuda").manual_seed(2)
    B, taps, seats_n = len(lens), 4, 8
    width, gn = heads * head_dim, groups * d_state
    C = 2 * gn + width
    W = C + width + 2 * heads
    conv_w = torch.randn(C, taps, device="cuda", generator=g) * 0.5
    conv_b = torch.randn(C, device="cuda", generator=g) * 0.2
    a_log, dt_bias = torch.randn(heads, device="cuda", generator=g) * 0.5, torch.randn(heads, device="cuda", generator=g) * 0.5
    skip = 1 + 0.2 * torch.randn(heads, device="cuda", generator=g)
    norm_w = (1 + 0.1 * torch.randn(width, device="cuda", generator=g)).to(dtype)
    seats = torch.tensor([3, 1, 5, 2][:B], dtype=torch.int32, device="cuda")
    conv_k = torch.randn(seats_n, C, taps - 1, device="cuda", generator=g).to(dtype)
    ssm_k = torch.randn(seats_n, heads, d_state, head_dim, device="cuda", generator=g)
    conv_r, ssm_r = conv_k.clone(), ssm_k.clone()
    start = [0] * B
    for step_lens in (lens, [3] * B):
        T = sum(step_lens)
        cu = torch.tensor([0] + list(torch.tensor(step_lens).cumsum(0)), dtype=torch.int32, device="cuda")
        pos = torch.cat([torch.arange(s, s + n) for s, n in zip(start, step_lens)]).to(torch.int32).cuda()
        proj = torch.randn(T, W, device="cuda", generator=g).to(dtype)
        proj[:, -heads:] = proj[:, -2 * heads:-heads]                                          # the time step sits in both slots
        got = K.mamba2(proj, conv_w, conv_b, a_log, dt_bias, skip, norm_w, 1e-5, conv_k, ssm_k, seats, cu, pos, groups, heads,
                       d_state, head_dim)
        want = ref.mamba2(proj.float(), conv_w, conv_b, a_log, dt_bias, skip, norm_w.float(), 1e-5, conv_r, ssm_r, seats, cu, pos,
                          groups, heads, d_state, head_dim)
        tol = 3e-2 if dtype == torch.bfloat16 else 2e-3
        close(got, want, tol, tol)
        close(ssm_k[seats.long()], ssm_r[seats.long()], tol, tol)
        start = [s + n for s, n in zip(start, step_lens)]


def test_sigmoid_gate_and_scaled_add(K):
    g = torch.Generator(device="cuda").manual_seed(2)
    for dtype in (torch.float32, torch.bfloat16):
        wide = torch.randn(37, 3 * 96, device="cuda", generator=g).to(dtype)
        x = torch.randn(37, 96, device="cuda", generator=g).to(dtype)
        close(K.sigmoid_gate(x, wide[:, 192:]), x.float() * torch.sigmoid(wide[:, 192:].float()))
        y = torch.randn(37, 96, device="cuda", generator=g).to(dtype)
        logit = torch.randn(37, 1, device="cuda", generator=g).to(dtype)
        close(K.scaled_add(y, x, logit), y.float() + x.float() * torch.sigmoid(logit.float()))
