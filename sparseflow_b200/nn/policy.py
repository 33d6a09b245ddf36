"""Per-operation policy for the sparse / dense decision, keyed by op name.

Same dataclass and methods as the reference's ``sparseflow/nn/policy.py`` (fields :13-27,
``load_runtime_policy`` :37-72, ``should_use_sparse`` :74-95), including its substring matching of
``op_name.lower()`` (any name containing "gate" or "up" is a gate/up op, and so on).  Defaults are
the B200 crossovers of the measured gate table (``gate_sm100.json``, see ``dispatch.py``) instead of
the reference's A100 numbers, and each op class has a second, low band ``M <= decode_max_M_*`` in which
the sparse path wins because it streams 0.5625x the weight bytes (0 = no such band)."""
from dataclasses import dataclass, field

from .. import dispatch as _gate


def _lo(cls):
    return field(default_factory=lambda: int(_gate.THRESHOLDS[cls]))


def _dec(cls):
    return field(default_factory=lambda: int(_gate.DECODE_MAX_M[cls]))


@dataclass
class SparseFlowPolicy:
    min_M_default: int = 1024

    # MLP thresholds (B200 crossovers against cuBLAS on the same pruned weights)
    min_M_gate_up: int = _lo("ffn_gate_up")
    min_M_down: int = _lo("ffn_down")

    # Attention projections
    min_M_qkv: int = _lo("attn_proj")
    min_M_o: int = _lo("attn_proj")

    # Low (bandwidth-bound) band, not present upstream
    decode_max_M_gate_up: int = _dec("ffn_gate_up")
    decode_max_M_down: int = _dec("ffn_down")
    decode_max_M_qkv: int = _dec("attn_proj")
    decode_max_M_o: int = _dec("attn_proj")

    # Upper bounds: none observed on B200 up to M = 16384
    max_M_gate_up: int = 1 << 20
    max_M_down: int = 1 << 20
    max_M_qkv: int = 1 << 20
    max_M_o: int = 1 << 20

    @staticmethod
    def supports_sm80() -> bool:
        """Kept for source compatibility; the kernels here need sm_100."""
        return SparseFlowPolicy.supports_sm100()

    @staticmethod
    def supports_sm100() -> bool:
        import torch
        if not torch.cuda.is_available():
            return False
        major, _ = torch.cuda.get_device_capability()
        return major == 10

    # which pair of fields an op name of a policy file sets: first match wins, in the order upstream tests them
    # (sparseflow/nn/policy.py:37-72): "gate"/"up" anywhere in the name, then "down", then q/k/v_proj, then any "o"
    _FILE_RULES = (
        (lambda n: "gate" in n or "up" in n, "gate_up"),
        (lambda n: "down" in n, "down"),
        (lambda n: "q_proj" in n or "k_proj" in n or "v_proj" in n, "qkv"),
        (lambda n: "o" in n, "o"),
    )

    def load_runtime_policy(self, path: str):
        """Thresholds from a JSON policy file: ``{"ops": {<op name>: {"min_m": .., "max_m": ..}, ..}}`` (a file without
        the ``"ops"`` level is read as that mapping itself).  Returns self."""
        import json
        with open(path, "r") as fh:
            doc = json.load(fh)
        table = doc.get("ops", doc)
        for name, limits in table.items():
            if not isinstance(limits, dict):
                continue
            lowered = name.lower()
            suffix = next((sfx for matches, sfx in self._FILE_RULES if matches(lowered)), None)
            if suffix is None:
                continue
            for key, prefix in (("min_m", "min_M_"), ("max_m", "max_M_")):
                if key in limits:
                    setattr(self, prefix + suffix, int(limits[key]))
        return self

    def should_use_sparse(self, op_name: str, M: int) -> bool:
        if M <= 0:
            return False
        op_lower = op_name.lower()
        if "gate" in op_lower or "up" in op_lower:
            return M <= self.decode_max_M_gate_up or self.min_M_gate_up <= M <= self.max_M_gate_up
        if "down" in op_lower:
            return M <= self.decode_max_M_down or self.min_M_down <= M <= self.max_M_down
        if any(x in op_lower for x in ["q_proj", "k_proj", "v_proj"]):
            return M <= self.decode_max_M_qkv or self.min_M_qkv <= M <= self.max_M_qkv
        if "o_proj" in op_lower or "o" == op_lower:
            return M <= self.decode_max_M_o or self.min_M_o <= M <= self.max_M_o
        return M >= self.min_M_default
