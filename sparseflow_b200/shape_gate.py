"""Op-level shape gate with per-shape overrides: ``decide(op, batch, seq) -> (use_sparse, reason)``.

Interface of the reference's ``demo/shape_gate_sm89.py`` (``GateRange`` :15-18, ``DEFAULT_RANGES`` :24-28,
``ShapeOverrides`` :30-47, ``decide_sparse_sm89`` :48-80) and ``demo/gate_runtime.py`` (``decide`` :32-53):
overrides keyed ``"<op>|b=<batch>|s=<seq>"`` decide first, then a range gate on ``M_eff = batch * seq``;
the reason string always agrees with the decision.  ``make_overrides`` is the decision rule of
``tools/make_shape_overrides_sm89_from_results.py:18-22,99-127`` (skipped -> dense, accuracy failure ->
dense, speed-up >= min_speedup -> sparse, else dense; best entry per shape kept).

What differs: the ranges are the B200 crossovers of ``gate_sm100.json`` (see ``dispatch.py``), and each op
has a second, low band ``M_eff <= decode_hi`` where the sparse path wins because it streams 0.5625x
the weight bytes; ``decide_sparse_sm100`` is the native name and ``decide_sparse_sm89`` / ``decide`` are kept
as aliases so that callers of the reference's demo code run unchanged.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, Iterable, Optional, Tuple

from . import dispatch


@dataclass(frozen=True)
class GateRange:
    lo: int
    hi: int
    decode_hi: int = 0      # sparse also for M_eff <= decode_hi (0 = no low band)


_OP_CLASS = {"ffn_gate": "ffn_gate_up", "ffn_gate_up": "ffn_gate_up", "ffn_up": "ffn_gate_up",
             "ffn_down": "ffn_down", "attn_qkv": "attn_proj", "attn_proj": "attn_proj", "attn_o": "attn_proj"}


def default_ranges() -> Dict[str, GateRange]:
    """Ranges per op name (the reference's three names plus their class names) from the measured table."""
    return {op: GateRange(lo=int(dispatch.THRESHOLDS[c]), hi=int(dispatch.MAX_THRESHOLDS[c]),
                          decode_hi=int(dispatch.DECODE_MAX_M[c])) for op, c in _OP_CLASS.items()}


class _LiveRanges(dict):
    """``DEFAULT_RANGES`` of the reference's module, but read from the gate table at every lookup so that
    ``dispatch.reload_gate()`` takes effect here too."""

    def get(self, op, default=None):
        return default_ranges().get(op, default)

    def __getitem__(self, op):
        return default_ranges()[op]

    def __contains__(self, op):
        return op in _OP_CLASS

    def __iter__(self):
        return iter(_OP_CLASS)

    def __len__(self):
        return len(_OP_CLASS)

    def items(self):
        return default_ranges().items()

    def keys(self):
        return default_ranges().keys()

    def values(self):
        return default_ranges().values()


DEFAULT_RANGES: Dict[str, GateRange] = _LiveRanges()


class ShapeOverrides:
    """Per-shape decision map {"<op>|b=<batch>|s=<seq>": {"decision": "dense"|"sparse", "reason": ...}}.
    A missing file gives an empty map (shape_gate_sm89.py:36-44); ``strict=True`` raises instead
    (gate_runtime.py:19-22)."""

    def __init__(self, path: Optional[str] = None, strict: bool = False):
        self.path = path
        self.map: Dict[str, Dict[str, Any]] = {}
        self.min_speedup = None
        self.src = None
        if path:
            p = Path(path)
            if p.exists():
                j = json.loads(p.read_text())
                if isinstance(j, dict):
                    self.map = j.get("overrides", {})
                    self.min_speedup = j.get("min_speedup")
                    self.src = j.get("source_run")
            elif strict:
                raise FileNotFoundError(path)

    def lookup(self, op: str, batch: int, seq: int) -> Optional[Dict[str, Any]]:
        return self.map.get(f"{op}|b={batch}|s={seq}")


def decide_sparse_sm100(op: str, batch: int, seq: int, overrides: Optional[ShapeOverrides] = None,
                        ranges: Optional[Dict[str, GateRange]] = None) -> Tuple[bool, str]:
    if overrides:
        rec = overrides.lookup(op, batch, seq)
        if rec:
            why = rec.get("reason", "override")
            if rec.get("decision", "dense") == "sparse":
                return True, f"override:sparse ({why})"
            return False, f"override:dense ({why})"
    r = (ranges if ranges is not None else DEFAULT_RANGES).get(op)
    if r is None:
        return False, "no-range:default-dense"
    m_eff = int(batch) * int(seq)
    if m_eff <= 0:
        return False, f"gate:skip (M_eff={m_eff} <= 0)"
    if m_eff <= r.decode_hi:
        return True, f"gate:run (M_eff={m_eff} <= decode_hi={r.decode_hi})"
    if m_eff < r.lo:
        return False, f"gate:skip (M_eff={m_eff} < lo={r.lo})"
    if m_eff > r.hi:
        return False, f"gate:skip (M_eff={m_eff} > hi={r.hi})"
    return True, f"gate:run (lo={r.lo} <= M_eff={m_eff} <= hi={r.hi})"


decide_sparse_sm89 = decide_sparse_sm100     # the reference's name
decide = decide_sparse_sm100                 # demo/gate_runtime.py's name


def make_overrides(results: Iterable[Dict[str, Any]], min_speedup: float = 1.20, source_run: Optional[str] = None,
                   run_id: Optional[str] = None) -> Dict[str, Any]:
    """Results [{shape, batch, seq_len, speedup, skipped, shape_gate, acc_gate_pass, acc_max_err_pct}] ->
    the overrides document ``ShapeOverrides`` reads."""
    def num(v):
        try:
            return float(v) if v is not None else None
        except (TypeError, ValueError):
            return None

    best: Dict[Tuple[str, int, int], Dict[str, Any]] = {}
    for r in results:
        if not isinstance(r, dict):
            continue
        try:
            key = (str(r["shape"]), int(r["batch"]), int(r["seq_len"]))
        except (KeyError, TypeError, ValueError):
            continue
        prev = best.get(key)
        if prev is None:
            best[key] = r
            continue
        cs, ps = bool(r.get("skipped", False)), bool(prev.get("skipped", False))
        cv, pv = num(r.get("speedup")), num(prev.get("speedup"))
        if (ps and not cs) or (ps == cs and cv is not None and (pv is None or cv > pv)):
            best[key] = r
    if not best:
        raise ValueError("no valid (shape, batch, seq_len) entries in results")
    out = {"source_run": source_run, "run_id": run_id, "min_speedup": min_speedup, "overrides": {}}
    for (shape, b, s), r in sorted(best.items()):
        sp, acc_err = num(r.get("speedup")), r.get("acc_max_err_pct")
        if bool(r.get("skipped", False)):
            dec, why = "dense", f"skipped ({r.get('shape_gate', '')})"
        elif r.get("acc_gate_pass", True) is False:
            dec, why = "dense", "acc_gate_fail"
        elif sp is None:
            dec, why = "dense", "no-speedup"
        elif sp >= min_speedup:
            dec, why = "sparse", f"speedup={sp:.3f}>=min"
        else:
            dec, why = "dense", f"speedup={sp:.3f}<min"
        out["overrides"][f"{shape}|b={b}|s={s}"] = {"decision": dec, "reason": why, "speedup": sp,
                                                    "acc_max_err_pct": acc_err}
    return out
