"""The debugging flavour behind EXO_KERNEL_CHECKS=1: guard bands behind outputs, host validation of the index
tensors that kernels dereference unchecked."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_guard_bands_stay_intact_under_the_kernels_and_catch_a_store_behind_the_end(monkeypatch):
    from exo_b200.ops import cuda as K
    monkeypatch.setattr(K, "CHECKS", True)
    K._guards.clear()
    x = torch.randn(37, 4096, device="cuda").bfloat16()
    w = torch.ones(4096, device="cuda", dtype=torch.bfloat16)
    y, _ = K.rmsnorm(x, w, 1e-5)
    wt = (torch.randn(1000, 4096, device="cuda") / 64).bfloat16()
    z = K.linear(x, wt)
    assert len(K._guards) >= 2 and z.shape == (37, 1000)
    K.verify_guards()                                   # every band is as it was written
    assert not K._guards
    out = K._empty(8, 16, dtype=torch.bfloat16, device=x.device, what="victim")
    flat, n, _ = K._guards[-1]
    flat[n + 3] = 1.0                                   # what an out-of-bounds store of a kernel would do
    with pytest.raises(K.KernelError, match="victim"):
        K.verify_guards()
    assert out.shape == (8, 16)


def test_index_tensors_are_validated_on_the_host_in_checks_mode(monkeypatch):
    from exo_b200.ops import cuda as K
    monkeypatch.setattr(K, "CHECKS", True)
    table = torch.randn(100, 64, device="cuda").bfloat16()
    ok = torch.tensor([0, 5, 99], device="cuda", dtype=torch.int32)
    assert K.embedding(table, ok).shape == (3, 64)
    with pytest.raises(K.KernelError, match="token ids"):
        K.embedding(table, torch.tensor([3, 100], device="cuda", dtype=torch.int32))
    K._guards.clear()
