"""The peer-memory collectives on ONE GPU: the peer is a second local arena whose flags the test sets by hand.

Kernels that wait on one another are never launched side by side on one device; here the "peer" has no
kernel at all: its partial is written by the host and its arrival flag is either pre-set (the normal
case) or left unset (the wait must run out, the kernel must return, and the status word must say so).
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

BAR_IN, BAR_OUT = 2048 // 4, 2112 // 4      # int32 word offsets of the barrier flags in the arena header


def _setup(n_ranks, rank, rows, hidden):
    from exo_b200.ops import cuda as K
    from exo_b200.parallel.fused import arena_layout, bind
    lib = bind(K.load())
    K.ensure_gemm_init(torch.device("cuda", 0))
    L = arena_layout(lib, n_ranks, rows, hidden, 64, 8)
    arenas = [torch.zeros(L["total"], dtype=torch.uint8, device="cuda") for _ in range(n_ranks)]
    arr = (C.c_void_p * n_ranks)(*[a.data_ptr() for a in arenas])
    rc = lib.exo_comm_init(arr, None, n_ranks, rank, L["slot"], L["gather_off"], L["x_off"], L["x_bytes"], L["h_off"],
                           L["n_off"], L["ll_off"], L["ll_slot"])
    assert rc == 0
    return lib, K, L, arenas


def _region(arena, L, which, parity, rows, cols):
    off = {0: L["x_off"], 1: L["h_off"], 2: L["n_off"]}[which] + parity * L["x_bytes"]
    return arena[off:off + rows * cols * 2].view(torch.bfloat16).view(rows, cols)


def _flags(arena):
    return arena[:4096].view(torch.int32)


def _ref(parts, res, w, eps):
    h = (sum(p.float() for p in parts) + res.float()).bfloat16()
    hf = h.float()
    x = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return h, x.bfloat16()


@pytest.mark.parametrize("rows,cols", [(3, 4096), (32, 4096), (200, 1024), (17, 7168), (64, 8192)])
def test_one_shot_reduce_norm_against_fp32_reference(rows, cols):
    lib, K, L, (A, B) = _setup(2, 0, 256, 8192)
    g = torch.Generator(device="cuda").manual_seed(rows * 31 + cols)
    st = torch.cuda.current_stream().cuda_stream
    for it in range(4):                                  # both parities, twice: the flags must come back clean
        parity = it & 1
        xa = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
        xb = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
        res = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
        w = (1 + 0.1 * torch.randn(cols, device="cuda", generator=g)).bfloat16()
        _region(A, L, 0, parity, rows, cols).copy_(xa)
        _region(B, L, 0, parity, rows, cols).copy_(xb)
        _flags(A)[BAR_IN + parity * 8 + 1] = 1          # the peer's "partial ready"
        h = torch.empty(rows, cols, dtype=torch.bfloat16, device="cuda")
        x = torch.empty_like(h)
        with_norm = it != 3
        rc = lib.exo_reduce_norm_bf16(res.data_ptr(), w.data_ptr() if with_norm else None, 1e-5, h.data_ptr(),
                                      x.data_ptr() if with_norm else None, rows, cols, parity, 0, 1, st)
        assert rc == 0
        torch.cuda.synchronize()
        want_h, want_x = _ref([xa, xb], res, w, 1e-5)
        assert torch.equal(h, want_h)                    # fp32 sum in rank order, one rounding: exact
        if with_norm:
            assert (x.float() - want_x.float()).abs().max() <= 0.02 * want_x.float().abs().max()
        f = _flags(A)
        assert int(f[BAR_IN + parity * 8].item()) == 0 and int(f[BAR_IN + parity * 8 + 1].item()) == 0
        assert int(_flags(B)[BAR_IN + parity * 8].item()) == it // 2 + 1     # our signal reached the peer's arena
    K.check_status()
    lib.exo_comm_reset()


def test_two_shot_reduce_norm_writes_this_ranks_rows_into_every_arena():
    rows, cols = 1000, 4096
    lib, K, L, (A, B) = _setup(2, 0, 1024, 4096)
    g = torch.Generator(device="cuda").manual_seed(5)
    xa = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    xb = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    res = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(cols, device="cuda", generator=g)).bfloat16()
    parity = 1
    _region(A, L, 0, parity, rows, cols).copy_(xa)
    _region(B, L, 0, parity, rows, cols).copy_(xb)
    _flags(A)[BAR_IN + parity * 8 + 1] = 1
    _flags(A)[BAR_OUT + parity * 8 + 1] = 1              # the peer's "rows broadcast": number of the reduction on this parity
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.exo_reduce_norm_bf16(res.data_ptr(), w.data_ptr(), 1e-5, None, None, rows, cols, parity, 1, 1, st)
    assert rc == 0
    torch.cuda.synchronize()
    want_h, want_x = _ref([xa, xb], res, w, 1e-5)
    mine = (rows + 1) // 2                               # rank 0 owns the first half of the rows
    for arena in (A, B):
        h = _region(arena, L, 1, parity, rows, cols)
        x = _region(arena, L, 2, parity, rows, cols)
        assert torch.equal(h[:mine], want_h[:mine])
        assert (x[:mine].float() - want_x[:mine].float()).abs().max() <= 0.02 * want_x.float().abs().max()
        assert float(h[mine:].float().abs().max()) == 0.0   # the peer's rows are the peer's to write
    # sharded form: the residual stream's rows stay in a private tensor, only the normalised rows are broadcast
    parity = 0
    _region(A, L, 0, parity, rows, cols).copy_(xa)
    _region(B, L, 0, parity, rows, cols).copy_(xb)
    _flags(A)[BAR_IN + parity * 8 + 1] = 1
    _flags(A)[BAR_OUT + parity * 8 + 1] = 1
    h_priv = torch.zeros(rows, cols, dtype=torch.bfloat16, device="cuda")
    assert lib.exo_reduce_norm_bf16(res.data_ptr(), w.data_ptr(), 1e-5, h_priv.data_ptr(), None, rows, cols, parity, 1, 0, st) == 0
    torch.cuda.synchronize()
    assert torch.equal(h_priv[:mine], want_h[:mine]) and float(h_priv[mine:].float().abs().max()) == 0.0
    for arena in (A, B):
        assert float(_region(arena, L, 1, parity, rows, cols).float().abs().max()) == 0.0      # hbuf untouched
        x = _region(arena, L, 2, parity, rows, cols)
        assert (x[:mine].float() - want_x[:mine].float()).abs().max() <= 0.02 * want_x.float().abs().max()
    # ... and gathered on request: this rank's rows go to every arena's hbuf
    GATHER = 2240 // 4
    _flags(A)[GATHER + 1] = 1
    assert lib.exo_gather_rows_bf16(h_priv.data_ptr(), rows, cols, parity, st) == 0
    torch.cuda.synchronize()
    for arena in (A, B):
        assert torch.equal(_region(arena, L, 1, parity, rows, cols)[:mine], want_h[:mine])
    K.check_status()
    lib.exo_comm_reset()


def test_a_wait_that_runs_out_returns_sets_the_status_word_and_leaves_the_context_usable():
    from exo_b200.ops.cuda import DeviceWaitTimeout
    rows, cols = 8, 4096
    lib, K, L, (A, B) = _setup(2, 0, 256, 4096)
    lib.exo_set_collective_timeout_us(20000)             # 20 ms instead of the serving default
    try:
        x = torch.randn(rows, cols, device="cuda").bfloat16()
        h = torch.empty_like(x)
        st = torch.cuda.current_stream().cuda_stream
        _region(A, L, 0, 0, rows, cols).copy_(x)
        # nobody raises the peer's flag: the kernel must give up after ~20 ms and return normally
        assert lib.exo_reduce_norm_bf16(None, None, 0.0, h.data_ptr(), None, rows, cols, 0, 0, 1, st) == 0
        torch.cuda.synchronize()
        with pytest.raises(DeviceWaitTimeout):
            K.check_status()
        K.check_status()                                 # the word was cleared by the raise
        # the older push-style all-reduce kernel takes the same path
        out = torch.empty_like(x)
        assert lib.exo_allreduce_bf16(x.data_ptr(), None, out.data_ptr(), x.numel(), 0, st) == 0
        torch.cuda.synchronize()
        assert lib.exo_comm_status() == 4
        # a healthy collective right afterwards: the peer's flag is there, the result is exact
        _region(B, L, 0, 0, rows, cols).copy_(x)
        _flags(A)[BAR_IN + 1] = 1
        assert lib.exo_reduce_norm_bf16(None, None, 0.0, h.data_ptr(), None, rows, cols, 0, 0, 1, st) == 0
        torch.cuda.synchronize()
        K.check_status()
        assert torch.equal(h, (x.float() * 2).bfloat16())
        # and an ordinary kernel still runs on this context
        y = K.rmsnorm(x, torch.ones(cols, device="cuda", dtype=torch.bfloat16), 1e-5)[0]
        assert torch.isfinite(y.float()).all()
    finally:
        lib.exo_set_collective_timeout_us(2000000)
        lib.exo_comm_reset()


def _ll_slot(arena, L, n_ranks, parity, src, n_values):
    off = L["ll_off"] + (parity * n_ranks + src) * L["ll_slot"]
    return arena[off:off + n_values * 4].view(torch.int32).view(-1, 2)      # [words, (two bf16, sequence number)]


@pytest.mark.parametrize("M", [1, 2])
def test_flag_in_data_handover_between_streaming_projections(M):
    """Row-parallel GEMV pushes (data, sequence) words; the next RMSNorm + GEMV polls them in its prologue."""
    from exo_b200.ops import reference as ref
    H, Kr, N2 = 4096, 1024, 6144
    lib, K, L, (A, B) = _setup(2, 0, 256, H)
    K.ensure_stream_init(torch.device("cuda", 0))
    g = torch.Generator(device="cuda").manual_seed(11 + M)
    st = torch.cuda.current_stream().cuda_stream
    w_o = (torch.randn(H, Kr, device="cuda", generator=g) / 32).bfloat16()
    w_up = (torch.randn(N2, H, device="cuda", generator=g) / 64).bfloat16()
    norm_w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).bfloat16()
    for it in range(4):                                   # both parities twice: the epoch must advance each time
        parity, seq = it & 1, it // 2 + 1
        x = torch.randn(M, Kr, device="cuda", generator=g).bfloat16()
        res = torch.randn(M, H, device="cuda", generator=g).bfloat16()
        peer = torch.randn(M, H, device="cuda", generator=g).bfloat16()       # what rank 1's projection would have sent
        words = _ll_slot(A, L, 2, parity, 1, M * H)
        words[:, 0] = peer.view(torch.int32).view(-1)
        words[:, 1] = seq
        assert lib.exo_gemv_stream_tp(x.data_ptr(), w_o.data_ptr(), None, None, None, 0.0, M, H, Kr, 0, 1, parity,
                                      None, None, st) == 0
        h_out = torch.empty(M, H, dtype=torch.bfloat16, device="cuda")
        y = torch.empty(M, N2, dtype=torch.bfloat16, device="cuda")
        assert lib.exo_gemv_stream_tp(None, w_up.data_ptr(), None, y.data_ptr(), norm_w.data_ptr(), 1e-5, M, N2, H, 0, 2,
                                      parity, res.data_ptr(), h_out.data_ptr(), st) == 0
        torch.cuda.synchronize()
        mine = ref.linear(x.float(), w_o.float()).bfloat16()
        # our words reached both arenas with this hand-over's sequence number
        for arena in (A, B):
            got = _ll_slot(arena, L, 2, parity, 0, M * H)
            assert bool((got[:, 1] == seq).all())
            sent = got[:, 0].contiguous().view(torch.bfloat16).view(M, H)
            assert (sent.float() - mine.float()).abs().max() <= 0.02 * mine.float().abs().max()
        sent = _ll_slot(A, L, 2, parity, 0, M * H)[:, 0].contiguous().view(torch.bfloat16).view(M, H)
        want_h = (res.float() + sent.float() + peer.float()).bfloat16()
        assert torch.equal(h_out, want_h)
        want_y = ref.linear(ref.rmsnorm(want_h.float(), norm_w.float(), 1e-5)[0], w_up.float())
        assert (y.float() - want_y).abs().max() <= 0.02 * want_y.abs().max()
    K.check_status()
    # a hand-over nobody pushed: the consumer gives up within the budget and says so
    lib.exo_set_collective_timeout_us(20000)
    try:
        assert lib.exo_tp_ll_finish(None, h_out.data_ptr(), M * H, 0, st) == 0
        torch.cuda.synchronize()
        assert lib.exo_comm_status() == 4
    finally:
        lib.exo_set_collective_timeout_us(2000000)
        lib.exo_comm_reset()


@pytest.mark.parametrize("M,Kr", [(5, 2048), (32, 2048), (64, 1792), (33, 128), (64, 256)])
def test_gemm_epilogue_handover_and_reduce_norm_kernel(M, Kr):
    """Decode-batch row-parallel GEMM whose epilogue sends (data, sequence) words (split-K and single-pass tiles),
    consumed by the reduce + RMSNorm kernel."""
    from exo_b200.ops import reference as ref
    H = 4096
    lib, K, L, (A, B) = _setup(2, 0, 256, H)
    g = torch.Generator(device="cuda").manual_seed(M * 7 + Kr)
    st = torch.cuda.current_stream().cuda_stream
    w_o = (torch.randn(H, Kr, device="cuda", generator=g) / 32).bfloat16()
    norm_w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).bfloat16()
    for it in range(4):
        parity, seq = it & 1, it // 2 + 1
        x = torch.randn(M, Kr, device="cuda", generator=g).bfloat16()
        res = torch.randn(M, H, device="cuda", generator=g).bfloat16()
        peer = torch.randn(M, H, device="cuda", generator=g).bfloat16()
        words = _ll_slot(A, L, 2, parity, 1, M * H)
        words[:, 0] = peer.view(torch.int32).view(-1)
        words[:, 1] = seq
        splits = lib.exo_gemm_splits(M, H, Kr)
        assert lib.exo_gemm_bf16_tp(x.data_ptr(), w_o.data_ptr(), None, M, H, Kr, splits, parity, st) == 0
        h = torch.empty(M, H, dtype=torch.bfloat16, device="cuda")
        xn = torch.empty_like(h)
        with_norm = it != 2
        assert lib.exo_tp_ll_reduce_norm(res.data_ptr(), norm_w.data_ptr() if with_norm else None, 1e-5, h.data_ptr(),
                                         xn.data_ptr() if with_norm else None, M, H, parity, st) == 0
        torch.cuda.synchronize()
        sent = _ll_slot(B, L, 2, parity, 0, M * H)                 # what reached the peer's arena
        assert bool((sent[:, 1] == seq).all())
        mine = sent[:, 0].contiguous().view(torch.bfloat16).view(M, H)
        want_mine = ref.linear(x.float(), w_o.float())
        assert (mine.float() - want_mine).abs().max() <= 0.02 * want_mine.abs().max()
        want_h = (res.float() + mine.float() + peer.float()).bfloat16()
        assert torch.equal(h, want_h)
        if with_norm:
            want_x = ref.rmsnorm(want_h.float(), norm_w.float(), 1e-5)[0]
            assert (xn.float() - want_x).abs().max() <= 0.02 * want_x.abs().max()
    K.check_status()
    lib.exo_comm_reset()


@pytest.mark.parametrize("swiglu", [False, True])
def test_gated_gemm_consumes_rows_of_a_deferred_two_shot_reduction(swiglu):
    """All-gather -> GEMM: the reduction kernel leaves without waiting for the peer's rows; the projection's CTAs wait
    for the flag of the rank that owns their rows.  Here the peer's rows and its flag are put in place by hand."""
    from exo_b200.ops import reference as ref
    rows, cols, N = 1024, 4096, 2048
    lib, K, L, (A, B) = _setup(2, 0, 1024, cols)
    g = torch.Generator(device="cuda").manual_seed(9)
    st = torch.cuda.current_stream().cuda_stream
    xa = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    xb = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    res = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    nw = (1 + 0.1 * torch.randn(cols, device="cuda", generator=g)).bfloat16()
    w = (torch.randn(N, cols, device="cuda", generator=g) / 64).bfloat16()
    want_h, want_x = _ref([xa, xb], res, nw, 1e-5)
    parity, mine = 1, rows // 2
    _region(A, L, 0, parity, rows, cols).copy_(xa)
    _region(B, L, 0, parity, rows, cols).copy_(xb)
    _flags(A)[BAR_IN + parity * 8 + 1] = 1
    h_priv = torch.zeros(rows, cols, dtype=torch.bfloat16, device="cuda")
    # mode 2: residual stream sharded (bit 0 clear), no trailing wait (bit 1 set)
    assert lib.exo_reduce_norm_bf16(res.data_ptr(), nw.data_ptr(), 1e-5, h_priv.data_ptr(), None, rows, cols, parity, 1, 2, st) == 0
    torch.cuda.synchronize()
    xn = _region(A, L, 2, parity, rows, cols)
    assert int(_flags(A)[BAR_OUT + parity * 8 + 0].item()) == 1          # our rows are flagged; the flag stays up for the GEMM
    assert float(xn[mine:].float().abs().max()) == 0.0                    # the peer's rows have not arrived
    xn[mine:].copy_(want_x[mine:])                                        # ... now they have
    _flags(A)[BAR_OUT + parity * 8 + 1] = 1
    got = K.gemm_bf16(xn, w, None, None, swiglu, gate_parity=parity)
    torch.cuda.synchronize()
    K.check_status()
    full = torch.cat((xn[:mine], want_x[mine:]))
    want = ref.linear(full.float(), w.float())
    if swiglu:
        want = ref.swiglu(want.bfloat16().float())
    assert (got.float() - want).abs().max() <= 0.03 * want.abs().max()
    # a peer that never delivers: the gated GEMM gives up within the budget and says so
    lib.exo_set_collective_timeout_us(20000)
    try:
        _flags(A)[BAR_OUT + parity * 8 + 1] = 0
        K.gemm_bf16(xn, w, None, None, swiglu, gate_parity=parity)
        torch.cuda.synchronize()
        assert lib.exo_comm_status() == 4
        K.gemm_check() if False else None
        lib.exo_gemm_last_error()                                         # the MMA warp's own wait ran out too: clear it
    finally:
        lib.exo_set_collective_timeout_us(2000000)
        lib.exo_comm_reset()
