"""Typed configuration with environment overrides."""
import pytest

from commbench_b200 import config as CFG


@pytest.fixture(autouse=True)
def fresh_config():
    CFG.reset_config()
    yield
    CFG.reset_config()


def test_defaults_and_environment_overrides(monkeypatch):
    c = CFG.get_config()
    assert c.ar_oneshot_max_bytes == 512 * 1024 and c.use_nvls is True and c.nvtx is False
    assert c.timeout_s == 2.0 and c.heap_bytes == 1 << 30 and c.attn_impl == 4
    assert CFG.get_config() is c                                    # process-wide object
    CFG.reset_config()
    monkeypatch.setenv("CB200_TIMEOUT_S", "0.25")
    monkeypatch.setenv("CB200_HEAP_BYTES", str(4 << 30))
    monkeypatch.setenv("CB200_USE_NVLS", "off")
    monkeypatch.setenv("CB200_NVTX", "1")
    monkeypatch.setenv("CB200_MOE_FUSED_SWIGLU", "false")
    monkeypatch.setenv("CB200_COLL_MAX_BLOCKS", "32")
    c = CFG.get_config()
    assert (c.timeout_s, c.heap_bytes, c.use_nvls, c.nvtx) == (0.25, 4 << 30, False, True)
    assert c.moe_fused_swiglu is False and c.coll_max_blocks == 32


def test_set_config_rejects_unknown_fields():
    CFG.set_config(fused_poll_ns=500, attn_impl=1)
    assert CFG.get_config().fused_poll_ns == 500 and CFG.get_config().attn_impl == 1
    with pytest.raises(KeyError):
        CFG.set_config(no_such_knob=1)


def test_every_field_is_documented_by_a_typed_default():
    import dataclasses

    for f in dataclasses.fields(CFG.Config):
        assert isinstance(f.default, (bool, int, float)), f.name
        assert CFG._coerce("1", type(f.default)) in (True, 1, 1.0)


def test_expert_placement_is_balanced_and_deterministic():
    from commbench_b200.parallel.ep import balanced_placement, imbalance

    load = [100, 90, 80, 70, 1, 1, 1, 1]
    start = list(range(8))
    new = balanced_placement(load, 4)
    assert sorted(new) == start and new == balanced_placement(load, 4)
    assert imbalance(load, start, 4) > 2.0 and imbalance(load, new, 4) < 1.2
    # every rank keeps exactly E / W slots
    assert all(len(new[r * 2:(r + 1) * 2]) == 2 for r in range(4))
    assert imbalance([0] * 8, start, 4) == 1.0


def test_ag_gemm_comm_cta_rule():
    from commbench_b200.ops.tp import AgGemm

    # largest count that keeps the compute CTAs' tile waves, within the cap
    assert AgGemm.pick_comm_ctas(8192, 14336, 512, 148, 8) == 4      # 72 pairs: 25 waves, 70: 26
    assert AgGemm.pick_comm_ctas(8192, 7168, 512, 148, 8) == 10
    assert AgGemm.pick_comm_ctas(8192, 3584, 256, 148, 8, cap=4) == 4
    assert AgGemm.pick_comm_ctas(8192, 3584, 512, 148, 8, cap=4) % 2 == 0
