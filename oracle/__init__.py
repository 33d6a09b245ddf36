"""CPU oracle for the 2:4-sparse FFN path.

TEST INFRASTRUCTURE ONLY.  Nothing under ``sparseflow_b200/`` may import this
package; it is the checker the CUDA path is compared with (tests, the smoke
check and the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``).

Parity pin: ``oracle.sparse24.prune_24`` is byte-identical to the unmodified
reference scripts (``experiments/gen_dense_reference.py`` ->
``experiments/prune_24_cpu.py`` -> ``experiments/gen_pruned_ref.py``) on their
seed-0 128x128 fixture; the outputs of that run are committed under
``tests/golden/`` together with the script that produced them.
"""
from .sparse24 import (  # noqa: F401
    PAIR_TO_REF_CODE,
    prune_24,
    prune_24_loop,
    prune_24_pruned_chunked,
    hw_nibbles,
    hw_meta_tiled,
    hw_meta_tiled_to_nibbles,
    ref_codes_to_pairs,
    ref_codes_packed_bytes,
    enum_codes_kmajor,
    nibble_words_rowmajor,
    decompress,
    validate_24,
    to_f32,
    from_f32,
    gemm_ref,
    silu_mul_ref,
    ffn_ref,
    interleave_gate_up_rows,
    rel_err_metrics,
)
