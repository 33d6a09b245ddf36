"""Per-operation policy for the sparse / dense decision, keyed by op name.

Same dataclass and methods as the reference's ``sparseflow/nn/policy.py`` (fields :13-27,
``load_runtime_policy`` :37-72, ``should_use_sparse`` :74-95), including its substring matching of
``op_name.lower()`` (any name containing "gate" or "up" is a gate/up op, and so on).  Defaults are
B200 numbers instead of the reference's A100 ones."""
from dataclasses import dataclass


@dataclass
class SparseFlowPolicy:
    min_M_default: int = 1024

    # MLP thresholds (B200 crossovers against cuBLAS on the same pruned weights)
    min_M_gate_up: int = 512
    min_M_down: int = 1024

    # Attention projections
    min_M_qkv: int = 1024
    min_M_o: int = 1024

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

    def load_runtime_policy(self, path: str):
        """Load min_m and max_m from a JSON policy file ({"ops": {name: {min_m, max_m}}})."""
        import json
        with open(path, "r") as f:
            data = json.load(f)

        ops = data.get("ops", data)
        for op, cfg in ops.items():
            if not isinstance(cfg, dict):
                continue
            op_lower = op.lower()
            if "gate" in op_lower or "up" in op_lower:
                if "min_m" in cfg:
                    self.min_M_gate_up = int(cfg["min_m"])
                if "max_m" in cfg:
                    self.max_M_gate_up = int(cfg["max_m"])
            elif "down" in op_lower:
                if "min_m" in cfg:
                    self.min_M_down = int(cfg["min_m"])
                if "max_m" in cfg:
                    self.max_M_down = int(cfg["max_m"])
            elif any(k in op_lower for k in ["q_proj", "k_proj", "v_proj"]):
                if "min_m" in cfg:
                    self.min_M_qkv = int(cfg["min_m"])
                if "max_m" in cfg:
                    self.max_M_qkv = int(cfg["max_m"])
            elif "o" in op_lower:
                if "min_m" in cfg:
                    self.min_M_o = int(cfg["min_m"])
                if "max_m" in cfg:
                    self.max_M_o = int(cfg["max_m"])
        return self

    def should_use_sparse(self, op_name: str, M: int) -> bool:
        if M <= 0:
            return False
        op_lower = op_name.lower()
        if "gate" in op_lower or "up" in op_lower:
            return self.min_M_gate_up <= M <= self.max_M_gate_up
        if "down" in op_lower:
            return self.min_M_down <= M <= self.max_M_down
        if any(x in op_lower for x in ["q_proj", "k_proj", "v_proj"]):
            return self.min_M_qkv <= M <= self.max_M_qkv
        if "o_proj" in op_lower or "o" == op_lower:
            return self.min_M_o <= M <= self.max_M_o
        return M >= self.min_M_default
