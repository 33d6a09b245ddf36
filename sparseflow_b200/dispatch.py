"""Shape gate: sparse or dense per GEMM call, from crossovers measured on B200.

Same interface as the reference's ``sparseflow/dispatch.py`` (``classify_projection`` :27-33,
``pad_to_multiple`` :35-37, ``should_use_sparse`` :39-53, ``get_padded_M`` :55-57); the thresholds
are re-derived for sm_100a and live in ``gate_sm100.json`` next to this file (written by
``python -m sparseflow_b200.gate_sweep`` on a B200).  Differences that follow from the new kernels:

* no M padding: TMA zero-fills ragged token tiles, so ``get_padded_M`` is the identity;
* the reference sends ``M_eff < 32`` to dense; here a decode band ``M_eff <= decode_max_m`` can be
  sparse as well (HBM-bound regime, sparse streams 0.5625x the weight bytes);
* ``in_features % 64 == 0`` stays a requirement (K tile of the tcgen05 kernel);
* a shape that the sweep measured itself is decided on ITS measurements (speed-up >= the table's
  ``min_speedup`` at the measured token counts that bracket ``M_eff``), not on the thresholds of its
  class, which are set by the worst shape of the class; shapes the sweep has not seen fall back to
  the class thresholds.  This is the per-shape override idea of ``demo/shape_gate_sm89.py:48-80``
  applied inside ``should_use_sparse``.
"""
from __future__ import annotations

import json
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
GATE_FILE = os.environ.get("SPARSEFLOW_GATE_FILE", os.path.join(_HERE, "gate_sm100.json"))

# Fallback table if the JSON is absent: conservative values from the first B200 measurements.
_DEFAULT = {
    "min_m": {"attn_proj": 1024, "ffn_gate_up": 512, "ffn_down": 1024},
    "max_m": {"attn_proj": 1 << 20, "ffn_gate_up": 1 << 20, "ffn_down": 1 << 20},
    "decode_max_m": {"attn_proj": 0, "ffn_gate_up": 0, "ffn_down": 0},
}


def _load() -> dict:
    try:
        with open(GATE_FILE) as fh:
            data = json.load(fh)
        out = {k: dict(_DEFAULT[k]) for k in _DEFAULT}
        for k in _DEFAULT:
            out[k].update({c: int(v) for c, v in data.get(k, {}).items()})
        shapes: dict = {}
        min_speedup = float(data.get("min_speedup", 1.05))
        for r in data.get("measurements", []):
            try:
                key = (int(r["K"]), int(r["N"]))
                shapes.setdefault(key, {})[int(r["M"])] = float(r["speedup"]) >= min_speedup
            except (KeyError, TypeError, ValueError):
                continue
        out["shapes"] = {k: sorted(v.items()) for k, v in shapes.items()}
        return out
    except (OSError, ValueError):
        out = {k: dict(v) for k, v in _DEFAULT.items()}
        out["shapes"] = {}
        return out


_TABLE = _load()
# Lower / upper bounds per projection class (names as in the reference).
THRESHOLDS = _TABLE["min_m"]
MAX_THRESHOLDS = _TABLE["max_m"]
DECODE_MAX_M = _TABLE["decode_max_m"]
# (in_features, out_features) -> [(measured M, sparse wins there)], ascending M
SHAPE_TABLE = _TABLE["shapes"]


def reload_gate(path: str | None = None) -> None:
    """Re-read the gate table (after a sweep wrote a new one)."""
    global GATE_FILE
    if path is not None:
        GATE_FILE = path
    t = _load()
    for dst, key in ((THRESHOLDS, "min_m"), (MAX_THRESHOLDS, "max_m"), (DECODE_MAX_M, "decode_max_m"),
                     (SHAPE_TABLE, "shapes")):
        dst.clear()
        dst.update(t[key])


def classify_projection(in_features: int, out_features: int) -> str:
    if out_features > in_features * 2:
        return "ffn_gate_up"
    elif in_features > out_features * 2:
        return "ffn_down"
    else:
        return "attn_proj"


def pad_to_multiple(x: int, multiple: int) -> int:
    """Round up to next multiple."""
    return ((x + multiple - 1) // multiple) * multiple


def measured_decision(M_eff: int, in_features: int, out_features: int):
    """True / False from this shape's own measurements, or None when the sweep has not measured it.
    Between two measured token counts both must be sparse wins; outside the measured range the nearest
    end decides."""
    pts = SHAPE_TABLE.get((in_features, out_features))
    if not pts:
        return None
    lo = hi = None
    for m, win in pts:
        if m <= M_eff:
            lo = win
        if m >= M_eff:
            hi = win
            break
    if lo is None:
        return hi
    if hi is None:
        return lo
    return lo and hi


def should_use_sparse(M_eff: int, in_features: int, out_features: int) -> bool:
    if M_eff <= 0 or in_features % 64 != 0 or out_features % 8 != 0:
        return False
    own = measured_decision(M_eff, in_features, out_features)
    if own is not None:
        return own
    proj_type = classify_projection(in_features, out_features)
    if M_eff <= DECODE_MAX_M[proj_type]:
        return True
    if M_eff < THRESHOLDS[proj_type]:
        return False
    if M_eff > MAX_THRESHOLDS[proj_type]:
        return False
    return True


def get_padded_M(M_eff: int) -> int:
    """Return the M to actually use.  No padding is needed on sm_100a."""
    return M_eff
