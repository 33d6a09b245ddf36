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
