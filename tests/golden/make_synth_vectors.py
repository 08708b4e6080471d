"""Writes synth_vectors.json from the CPU checker: python tests/golden/make_synth_vectors.py"""
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
from oracle import oracle as orc  # noqa: E402

cases = []
for seed, stream, start, n, sigma in [(20261125, 1, 0, 256, 0.02), (7, 300, 123456789, 512, 0.1), (99, 2, 5, 256, 1.0)]:
    x = orc.synth_normal(seed, stream, start, n, sigma)
    cases.append({
        "seed": seed, "stream": stream, "start": start, "n": n, "sigma": sigma,
        "first_bits": [format(int(v), "08x") for v in x.view(np.uint32)[:8]],
        "wire_hex": {name: orc.quantize(qt, x).tobytes().hex() for name, qt in orc.QT_NAMES.items() if qt},
    })
(HERE / "synth_vectors.json").write_text(json.dumps({"generator": "oracle/camelid_oracle.c synth_normal + quantize_block_*", "cases": cases}, indent=1))
print("wrote", HERE / "synth_vectors.json")
