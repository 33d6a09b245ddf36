"""Shape gate and policy: pure host logic.  Truth-table style of the reference's
tools/smoke_dispatch.py:16-29, with sm_100 thresholds."""
import json

from sparseflow_b200 import dispatch
from sparseflow_b200.nn.policy import SparseFlowPolicy


def test_classify_projection_matches_reference_rule():
    assert dispatch.classify_projection(4096, 11008) == "ffn_gate_up"
    assert dispatch.classify_projection(4096, 22016) == "ffn_gate_up"      # fused gate|up
    assert dispatch.classify_projection(11008, 4096) == "ffn_down"
    assert dispatch.classify_projection(4096, 4096) == "attn_proj"
    assert dispatch.classify_projection(8192, 28672) == "ffn_gate_up"
    assert dispatch.classify_projection(4096, 8192) == "attn_proj"         # exactly 2x is not "> 2x"


def test_gate_truth_table(tmp_path):
    gate = {"min_m": {"attn_proj": 1024, "ffn_gate_up": 512, "ffn_down": 1024},
            "max_m": {"attn_proj": 65536, "ffn_gate_up": 65536, "ffn_down": 65536},
            "decode_max_m": {"attn_proj": 0, "ffn_gate_up": 8, "ffn_down": 0}}
    p = tmp_path / "gate.json"
    p.write_text(json.dumps(gate))
    old = dispatch.GATE_FILE
    try:
        dispatch.reload_gate(str(p))
        cases = [
            (4096, 4096, 22016, True), (512, 4096, 22016, True), (511, 4096, 22016, False),
            (4, 4096, 22016, True), (9, 4096, 22016, False),          # decode band then the gap
            (1024, 11008, 4096, True), (1023, 11008, 4096, False), (4, 11008, 4096, False),
            (2048, 4096, 4096, True), (512, 4096, 4096, False),
            (4096, 4000, 22016, False),                                 # in_features % 64 != 0
            (4096, 4096, 22012, False),                                 # out_features % 8 != 0
            (70000, 4096, 22016, False), (0, 4096, 22016, False),
        ]
        for M, i, o_, want in cases:
            assert dispatch.should_use_sparse(M, i, o_) is want, (M, i, o_)
    finally:
        dispatch.reload_gate(old)
    assert dispatch.get_padded_M(77) == 77
    assert dispatch.pad_to_multiple(77, 32) == 96


def test_policy_substring_semantics_and_json(tmp_path):
    pol = SparseFlowPolicy(min_M_gate_up=256, max_M_gate_up=2048, min_M_down=512, max_M_down=2048,
                           min_M_qkv=512, max_M_qkv=2048, min_M_o=512, max_M_o=2048, min_M_default=512)
    assert pol.should_use_sparse("layer3.gate_proj", 256)
    assert not pol.should_use_sparse("layer3.gate_proj", 255)
    assert pol.should_use_sparse("group_thing", 300)          # contains "up": treated as gate/up
    assert not pol.should_use_sparse("down_proj", 256) and pol.should_use_sparse("down_proj", 512)
    assert not pol.should_use_sparse("down_proj", 4096)
    assert pol.should_use_sparse("q_proj", 512) and not pol.should_use_sparse("v_proj", 100)
    assert pol.should_use_sparse("o_proj", 2048) and pol.should_use_sparse("o", 600)
    assert pol.should_use_sparse("default", 512) and pol.should_use_sparse("default", 10 ** 6)
    assert not pol.should_use_sparse("gate_proj", 0)
    p = tmp_path / "policy.json"
    p.write_text(json.dumps({"ops": {"gate_proj": {"min_m": 128, "max_m": 16384}, "down_proj": {"min_m": 640},
                                       "q_proj": {"max_m": 999}, "o_proj": {"min_m": 7}, "note": "x"}}))
    pol.load_runtime_policy(str(p))
    assert (pol.min_M_gate_up, pol.max_M_gate_up, pol.min_M_down, pol.max_M_qkv, pol.min_M_o) == (128, 16384, 640, 999, 7)


def test_policy_low_band_and_defaults_follow_the_measured_table():
    pol = SparseFlowPolicy()
    assert pol.min_M_gate_up == dispatch.THRESHOLDS["ffn_gate_up"] and pol.min_M_down == dispatch.THRESHOLDS["ffn_down"]
    assert pol.min_M_qkv == pol.min_M_o == dispatch.THRESHOLDS["attn_proj"]
    assert pol.decode_max_M_down == dispatch.DECODE_MAX_M["ffn_down"]
    pol = SparseFlowPolicy(min_M_down=512, decode_max_M_down=64, min_M_qkv=2048, decode_max_M_qkv=0)
    assert pol.should_use_sparse("down_proj", 1) and pol.should_use_sparse("down_proj", 64)
    assert not pol.should_use_sparse("down_proj", 65) and not pol.should_use_sparse("down_proj", 511)
    assert pol.should_use_sparse("down_proj", 512)
    assert not pol.should_use_sparse("k_proj", 1) and pol.should_use_sparse("k_proj", 2048)


def test_op_level_gate_with_overrides(tmp_path):
    """Truth table of decide(): overrides first, then low band, then [lo, hi]; reasons agree with decisions."""
    from sparseflow_b200 import shape_gate as sg
    ranges = {"ffn_gate": sg.GateRange(lo=256, hi=65536), "ffn_down": sg.GateRange(lo=512, hi=131072, decode_hi=64)}
    ok, why = sg.decide("ffn_gate", 4, 64, ranges=ranges)
    assert ok and why == "gate:run (lo=256 <= M_eff=256 <= hi=65536)"
    ok, why = sg.decide("ffn_gate", 1, 255, ranges=ranges)
    assert not ok and why == "gate:skip (M_eff=255 < lo=256)"
    ok, why = sg.decide("ffn_gate", 1024, 65, ranges=ranges)
    assert not ok and "> hi=65536" in why
    assert sg.decide("ffn_down", 8, 8, ranges=ranges) == (True, "gate:run (M_eff=64 <= decode_hi=64)")
    assert sg.decide("ffn_down", 5, 13, ranges=ranges)[0] is False
    assert sg.decide("lm_head", 1, 4096, ranges=ranges) == (False, "no-range:default-dense")
    assert sg.decide("ffn_down", 0, 7, ranges=ranges)[0] is False
    assert sg.decide_sparse_sm89 is sg.decide_sparse_sm100
    # default ranges come from the measured table
    r = sg.default_ranges()
    assert r["ffn_gate"].lo == dispatch.THRESHOLDS["ffn_gate_up"] and r["attn_qkv"].decode_hi == dispatch.DECODE_MAX_M["attn_proj"]
    # overrides generated with the reference's rule
    results = [
        {"shape": "ffn_gate", "batch": 1, "seq_len": 128, "speedup": 1.5, "skipped": False, "acc_gate_pass": True},
        {"shape": "ffn_gate", "batch": 1, "seq_len": 128, "speedup": 1.1, "skipped": False},          # worse duplicate
        {"shape": "ffn_gate", "batch": 64, "seq_len": 64, "speedup": 1.9, "acc_gate_pass": False},
        {"shape": "ffn_down", "batch": 2, "seq_len": 512, "speedup": 1.05},
        {"shape": "ffn_down", "batch": 2, "seq_len": 16, "speedup": 3.0, "skipped": True, "shape_gate": "M too small"},
        {"shape": "attn_qkv", "batch": 1, "seq_len": 1, "speedup": None},
        {"batch": 1}, "junk",
    ]
    doc = sg.make_overrides(results, min_speedup=1.2, source_run="run.json", run_id="r1")
    ov = doc["overrides"]
    assert ov["ffn_gate|b=1|s=128"]["decision"] == "sparse" and ov["ffn_gate|b=1|s=128"]["speedup"] == 1.5
    assert ov["ffn_gate|b=64|s=64"] == {"decision": "dense", "reason": "acc_gate_fail", "speedup": 1.9, "acc_max_err_pct": None}
    assert ov["ffn_down|b=2|s=512"]["reason"] == "speedup=1.050<min"
    assert ov["ffn_down|b=2|s=16"]["reason"] == "skipped (M too small)"
    assert ov["attn_qkv|b=1|s=1"]["reason"] == "no-speedup" and len(ov) == 5
    p = tmp_path / "ov.json"
    p.write_text(json.dumps(doc))
    o = sg.ShapeOverrides(str(p))
    assert o.min_speedup == 1.2 and o.src == "run.json"
    assert sg.decide("ffn_gate", 1, 128, overrides=o, ranges=ranges) == (True, "override:sparse (speedup=1.500>=min)")
    assert sg.decide("ffn_gate", 64, 64, overrides=o, ranges=ranges) == (False, "override:dense (acc_gate_fail)")
    assert sg.decide("ffn_gate", 4, 64, overrides=o, ranges=ranges)[1].startswith("gate:run")     # no override: range gate
    assert sg.ShapeOverrides(str(tmp_path / "missing.json")).map == {}
    import pytest
    with pytest.raises(FileNotFoundError):
        sg.ShapeOverrides(str(tmp_path / "missing.json"), strict=True)
    with pytest.raises(ValueError):
        sg.make_overrides([{"batch": 1}])


def test_measured_shapes_are_decided_on_their_own_measurements(tmp_path):
    """A shape the sweep measured is decided on ITS speed-ups, not on the thresholds of its class (which the worst
    shape of the class sets); between two measured token counts both must win; unseen shapes use the class."""
    gate = {"min_speedup": 1.05,
            "min_m": {"attn_proj": 2048, "ffn_gate_up": 512, "ffn_down": 512},
            "max_m": {"attn_proj": 1 << 20, "ffn_gate_up": 1 << 20, "ffn_down": 1 << 20},
            "decode_max_m": {"attn_proj": 32, "ffn_gate_up": 128, "ffn_down": 64},
            "measurements": [
                {"class": "attn_proj", "K": 8192, "N": 8192, "M": m, "speedup": s}
                for m, s in ((16, 1.4), (128, 1.2), (512, 0.98), (1024, 1.30), (4096, 1.5))] + [
                {"class": "attn_proj", "K": 4096, "N": 4096, "M": m, "speedup": s}
                for m, s in ((16, 1.5), (128, 0.87), (1024, 0.94), (4096, 1.4))] + ["junk", {"K": 1}]}
    p = tmp_path / "gate.json"
    p.write_text(json.dumps(gate))
    old = dispatch.GATE_FILE
    try:
        dispatch.reload_gate(str(p))
        s = dispatch.should_use_sparse
        # 8192 x 8192: wins at 1024 tokens although the class threshold says 2048
        assert s(1024, 8192, 8192) and s(4096, 8192, 8192) and s(2000, 8192, 8192)
        assert not s(512, 8192, 8192) and not s(300, 8192, 8192) and not s(700, 8192, 8192)    # a loss at 512 on one side
        assert s(64, 8192, 8192) and s(1, 8192, 8192) and s(100000, 8192, 8192)                 # ends: nearest measurement
        # 4096 x 4096: its own losses at 128 .. 1024 stand
        assert s(16, 4096, 4096) and not s(64, 4096, 4096) and not s(1024, 4096, 4096) and s(4096, 4096, 4096)
        assert not s(2048, 4096, 4096)                       # between a loss (1024) and a win (4096)
        # a shape the sweep has not seen: class thresholds
        assert dispatch.measured_decision(1024, 5120, 5120) is None
        assert not s(1024, 5120, 5120) and s(2048, 5120, 5120) and s(32, 5120, 5120)
        # the op-level gate reads the reloaded table too
        from sparseflow_b200 import shape_gate as sg
        assert sg.DEFAULT_RANGES["attn_qkv"].lo == 2048 and sg.decide("attn_qkv", 1, 2048)[0]
    finally:
        dispatch.reload_gate(old)
