"""Regenerates tests/golden/generator_vectors.json from the CPU oracle.

The reference project holds no numeric golden vectors for this path (its kernels
use constant operands and never read results back), so the fixtures pin the
build's own seeded generators: any later change to the counter-based streams
shows up as a diff here.  Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import binding as orc  # noqa: E402

cases = []
for seed, dist, mean, std, first, n in ((0, 1, 0.0, 1.0, 0, 8), (1, 0, 0.0, 1.0, 0, 8), (3, 2, 0.0, 1.0, 0, 8),
                                        (40, 2, 0.0, 0.02, 0, 8), (1, 0, 0.0, 1.0, (1 << 33) + 5, 4),
                                        (2, 1, 0.0, 1.0, 128 * 16, 4)):
    bits = orc.fill_f32(n, seed, dist, mean, std, first=first).view(np.uint32).tolist()
    cases.append(dict(seed=seed, dist=dist, mean=mean, std=std, first=first, n=n, bits=bits))
out = dict(cases=cases, i8_seed2=orc.fill_i8(32, 2).tolist(), cycle16_seed9=orc.chase_cycle(16, 9).tolist())
(Path(__file__).parent / "generator_vectors.json").write_text(json.dumps(out, indent=1) + "\n")
print("wrote", len(cases), "cases")
