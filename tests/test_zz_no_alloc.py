"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at the moment they need attention:
a server whose HBM is already fully handed to the KV pool, a latency-critical thread that must
not hit the device-wide synchronisation of cudaMalloc/cudaFree, or a C program linking the
library without PyTorch's allocator.  For them ``exo_paged_decode_noalloc`` keeps its split-KV
scratch inside the library.  This file checks that it gives the same output as the regular entry
point (which takes a caller-supplied workspace), twice in a row because the built-in scratch is
shared between calls and keeps the previous call's contents.  It is collected last on purpose.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(B, Hq, Hkv, D, lens, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    bs = 16
    max_blocks = max(-(-n // bs) for n in lens) + 1
    n_blocks = B * max_blocks + 1
    kc = torch.randn(n_blocks, bs, Hkv, D, device="cuda", generator=g).bfloat16()
    vc = torch.randn(n_blocks, bs, Hkv, D, device="cuda", generator=g).bfloat16()
    bt = (torch.randperm(n_blocks - 1, device="cuda", generator=g) + 1)[: B * max_blocks].view(B, max_blocks).int()
    q = torch.randn(B, Hq, D, device="cuda", generator=g).bfloat16()
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    return q, kc, vc, bt, sl, max_blocks, bs


def test_noalloc_entry_point_matches_workspace_entry_point_twice():
    from exo_b200.ops import cuda as K
    from exo_b200.ops import reference as ref
    lib = K.load()
    fn = lib.exo_paged_decode_noalloc
    fn.restype = C.c_int
    p, i, f = C.c_void_p, C.c_int, C.c_float
    fn.argtypes = [p, p, p, p, p, p, f, i, i, i, i, i, i, i, i, p, i, p]
    st = torch.cuda.current_stream().cuda_stream
    for call, (lens, seed) in enumerate((([700, 33, 2049, 5], 1), ([64, 1500, 18, 901], 2))):
        B, Hq, Hkv, D = 4, 32, 8, 128
        q, kc, vc, bt, sl, max_blocks, bs = _setup(B, Hq, Hkv, D, lens, seed)
        cu = torch.arange(B + 1, device="cuda", dtype=torch.int32)
        want = K.paged_attention(q, kc, vc, bt, sl, cu, D ** -0.5, max_q_len=1)   # existing entry point
        n_splits = lib.exo_paged_decode_splits(B, Hkv, max_blocks * bs)
        got = torch.empty_like(q)
        rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), sl.data_ptr(), got.data_ptr(),
                D ** -0.5, B, Hq, Hkv, D, max_blocks, bs, n_splits, 0, None, K.BF16, st)
        assert rc == 0, f"call {call}: rc={rc}"
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs().max().item()
        scale = want.float().abs().max().item()
        assert err <= 2e-2 + 2e-2 * scale, f"call {call}: max err {err}"
        # and both agree with the plain PyTorch definition of the op
        gold = ref.paged_attention(q.float(), kc.float(), vc.float(), bt, sl, cu, D ** -0.5)
        assert (got.float() - gold).abs().max().item() <= 2e-2 + 2e-2 * gold.abs().max().item()


def test_noalloc_entry_point_rejects_oversized_problems():
    from exo_b200.ops import cuda as K
    lib = K.load()
    fn = lib.exo_paged_decode_noalloc
    fn.restype = C.c_int
    p, i, f = C.c_void_p, C.c_int, C.c_float
    fn.argtypes = [p, p, p, p, p, p, f, i, i, i, i, i, i, i, i, p, i, p]
    # B * Hq * n_splits * (D + 2) floats would exceed the 8 MiB built-in scratch: refused, nothing launched
    rc = fn(None, None, None, None, None, None, 1.0, 256, 64, 8, 128, 8, 16, 64, 0, None, K.BF16, None)
    assert rc == -7
