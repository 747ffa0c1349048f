"""Generates tests/golden/dequant_golden.npz.

For every block format: a few seeded rows in raw GGUF layout, their dequantized f32
values as computed by the independent `gguf` Python package (gguf.quants.dequantize,
v0.19.0), a seeded activation vector, and the f64 dot products.  The CPU oracle and the
CUDA kernels are both checked against these files, so the check does not depend on the
`gguf` package (or on the mounted reference tree) being present at test time.

Run from the repository root:  python tests/golden/gen_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

entry.load_package()
from saient_quartz_b200 import synth  # noqa: E402
from gguf import quants, GGMLQuantizationType as T  # noqa: E402

K, N = 512, 6
out = {}
x = synth.make_x(K, seed=0x60D, tensor_id=1)
out["x"] = x
for t, (name, be, bb) in sorted(synth.FORMATS.items()):
    w = synth.make_weights(t, K, N, seed=0x60D, tensor_id=t)
    if name == "F32":
        deq = w.view(np.float32).copy()
    elif name == "F16":
        deq = w.view(np.float16).astype(np.float32)
    else:
        deq = quants.dequantize(w.reshape(N, -1), T[name]).reshape(-1).astype(np.float32)
    out[f"w_{name}"] = w
    out[f"deq_{name}"] = deq
    out[f"y64_{name}"] = deq.reshape(N, K).astype(np.float64) @ x.astype(np.float64)
np.savez_compressed(os.path.join(ROOT, "tests", "golden", "dequant_golden.npz"), **out)
print("wrote", len(out), "arrays")
