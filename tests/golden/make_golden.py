#!/usr/bin/env python3
"""Regenerate the golden fixtures from the UNMODIFIED reference scripts.

Runs, in a scratch directory, the reference's own oracle pipeline
  experiments/gen_dense_reference.py  (seed 0, 128x128 fp16 A, column-major B)
  experiments/prune_24_cpu.py         (pruned dense, compressed values, code bytes)
  experiments/gen_pruned_ref.py       (fp32 matmul on the pruned A)
and copies the resulting ``.bin`` files next to this script, plus a manifest of
sha256 digests.  Needs a checkout of the reference; usage:

    python tests/golden/make_golden.py /path/to/SparseFlow

It also writes ``tie_patterns.npz``: the reference's selection rule
(``np.argsort(np.abs(vals))[-2:]``, executed here, not restated) applied to all
81 rank patterns over four slots and to special values (NaN, inf, +-0,
denormals), which pins the tie-break behaviour.
"""
import hashlib
import itertools
import json
import os
import shutil
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
FILES = ["A_dense.bin", "B_dense.bin", "A_pruned_dense.bin", "dA.bin", "dE.bin", "D_pruned_ref.bin"]


def main(ref_root: str) -> None:
    exp = os.path.join(ref_root, "experiments")
    with tempfile.TemporaryDirectory() as tmp:
        for script in ("gen_dense_reference.py", "prune_24_cpu.py", "gen_pruned_ref.py"):
            subprocess.run([sys.executable, os.path.join(exp, script)], cwd=tmp, check=True,
                           stdout=subprocess.DEVNULL)
        manifest = {"numpy": np.__version__, "files": {}}
        for f in FILES:
            shutil.copy(os.path.join(tmp, f), os.path.join(HERE, f))
            with open(os.path.join(HERE, f), "rb") as fh:
                manifest["files"][f] = hashlib.sha256(fh.read()).hexdigest()

    # Nibble-packed code bytes (two groups per byte) from the reference's artifact generator, run as is.
    with tempfile.TemporaryDirectory() as tmp:
        subprocess.run([sys.executable, os.path.join(exp, "gen_test_artifacts.py")], cwd=tmp, check=True,
                       stdout=subprocess.DEVNULL)
        with open(os.path.join(tmp, "dA.bin"), "rb") as fh:           # same seed-0 matrix: same compressed values
            assert hashlib.sha256(fh.read()).hexdigest() == manifest["files"]["dA.bin"]
        shutil.copy(os.path.join(tmp, "dE_case_0.bin"), os.path.join(HERE, "dE_case_0.bin"))
        with open(os.path.join(HERE, "dE_case_0.bin"), "rb") as fh:
            manifest["files"]["dE_case_0.bin"] = hashlib.sha256(fh.read()).hexdigest()

    # Tie / special-value patterns: the reference's selection expression run as is.
    pats = []
    for ranks in itertools.product(range(3), repeat=4):
        pats.append([np.float16(1.0 + r) * (1 if (i % 2 == 0) else -1) for i, r in enumerate(ranks)])
    nan, inf = np.float16(np.nan), np.float16(np.inf)
    den = np.float16(6e-8)
    specials = [
        [nan, 1, 2, 3], [1, nan, 2, 3], [3, 2, 1, nan], [nan, nan, 1, 2], [nan, 1, nan, 2],
        [nan, nan, nan, nan], [inf, nan, 1, 2], [inf, -inf, 1, 2], [inf, 1, -inf, nan],
        [0.0, -0.0, 0.0, -0.0], [-0.0, 0.0, 1, 0.0], [den, -den, 0.0, den], [den, 0.0, 0.0, 0.0],
        [0.0, 0.0, 0.0, 0.0], [65504, -65504, 65504, 1], [1, 1, 1, 1], [-1, 1, -1, 1],
    ]
    for s in specials:
        pats.append([np.float16(v) for v in s])
    pats = np.array(pats, dtype=np.float16)
    kept = np.zeros((len(pats), 2), np.uint8)
    for i, vals in enumerate(pats):
        idx = np.argsort(np.abs(vals))[-2:]     # experiments/prune_24_cpu.py:21
        idx.sort()                               # experiments/prune_24_cpu.py:22
        kept[i] = idx
    np.savez(os.path.join(HERE, "tie_patterns.npz"), patterns=pats.view(np.uint16), kept=kept)
    with open(os.path.join(HERE, "tie_patterns.npz"), "rb") as fh:
        manifest["files"]["tie_patterns.npz"] = hashlib.sha256(fh.read()).hexdigest()
    with open(os.path.join(HERE, "manifest.json"), "w") as fh:
        json.dump(manifest, fh, indent=1, sort_keys=True)
    print(json.dumps(manifest, indent=1, sort_keys=True))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
