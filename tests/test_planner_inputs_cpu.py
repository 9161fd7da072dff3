"""The placement planner's inputs: measured link figures replace the nominal ones where the probe has run."""
import json

from exo_b200.master.placement import choose_shape, estimate_decode_step_us, is_moe_card
from exo_b200.shared.base import Memory, ModelId
from exo_b200.shared.cards import ModelCard
from exo_b200.utils import info_gatherer, link_probe
from exo_b200.utils.info_gatherer import GpuSample, nvlink_info


def _gpu(i, n=4):
    return GpuSample(index=i, name="NVIDIA B200", uuid=f"GPU-{i}", mem_total=180 << 30, mem_free=170 << 30, power_mw=0, temp_c=0,
                     util_pct=0, p2p_ok=[1] * n, nvlink_peers_links=[0] * n, active_links=18)


def _card(name="org/Llama-3.1-70B", family="llama", gb=70):
    return ModelCard(model_id=ModelId(name), storage_size=Memory.from_mb(gb * 1024), n_layers=80, hidden_size=8192,
                     supports_tensor=True, num_key_value_heads=8, tasks=["TextGeneration"], family=family)


def test_measured_peer_bandwidth_and_latency_replace_links_times_nominal():
    nominal = nvlink_info(_gpu(0), 4)
    assert all(not p.measured and p.gbps == 18 * info_gatherer.NVLINK5_GBPS_PER_LINK for p in nominal.peers)
    probe = {"gpu": 0, "hbm_gbps": 6540.0, "peers": {"1": {"gbps": 771.5, "latency_us": 2.4}, "2": {"error": -2}}}
    got = nvlink_info(_gpu(0), 4, probe)
    by = {p.peer_gpu: p for p in got.peers}
    assert got.hbm_gbps == 6540.0
    assert by[1].measured and by[1].gbps == 771.5 and by[1].latency_us == 2.4
    assert not by[2].measured and by[2].gbps == nominal.peers[1].gbps      # failed probe: nominal figure kept
    assert not by[3].measured


def test_cost_model_takes_the_measured_figures():
    card = _card()
    slow = estimate_decode_step_us(card, 8, 1, 700.0, hbm_gbps=3000.0, link_latency_us=10.0)
    fast = estimate_decode_step_us(card, 8, 1, 700.0, hbm_gbps=6500.0, link_latency_us=2.0)
    assert slow > fast
    # decode walks pipeline stages one after the other, so with NVSwitch (uniform, low-latency links) the latency
    # model keeps a 70B model on TP8; the measured figures only move the estimate, not the ranking
    from exo_b200.shared.wire import Sharding
    assert choose_shape(card, 8, Sharding.Tensor, 700.0, 6500.0, 0.5) == (8, 1)
    t8 = estimate_decode_step_us(card, 8, 1, 700.0, 1, 6500.0, 2.0)
    t42 = estimate_decode_step_us(card, 4, 2, 700.0, 1, 6500.0, 2.0)
    assert t8 < t42


def test_moe_cards_are_recognised_by_name_or_family_not_by_a_stray_letter():
    assert is_moe_card(_card("Qwen/Qwen3-235B-A22B-Instruct-2507-FP8", "qwen"))
    assert is_moe_card(_card("deepseek-ai/DeepSeek-V3.1", "deepseek"))
    assert not is_moe_card(_card("meta-llama/Llama-3.1-70B-Instruct", "llama"))
    assert not is_moe_card(_card("Qwen/Qwen3-32B-AWQ", "qwen"))


def test_probe_result_is_cached_per_gpu(tmp_path, monkeypatch):
    from exo_b200.shared import constants
    monkeypatch.setattr(constants, "EXO_CACHE_HOME", tmp_path)
    calls = []

    class R:
        stdout = json.dumps({"gpu": 1, "hbm_gbps": 6400.0, "peers": {"0": {"gbps": 760.0, "latency_us": 2.1}}}) + "\n"

    def fake_run(cmd, **kw):
        calls.append(cmd)
        return R()
    monkeypatch.setattr(link_probe.subprocess, "run", fake_run)
    a = link_probe.measure(1, [0], "GPU-1")
    b = link_probe.measure(1, [0], "GPU-1")
    assert a == b and a["peers"]["0"]["gbps"] == 760.0 and len(calls) == 1
