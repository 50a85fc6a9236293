"""Writes tests/golden/closed_form.json: known-answer vectors for the reference's closed-form
fixtures (src/ops/transformer.rs:2833-2980, 4102-4189, 1683-1728).

Weights come from the per-element closed-form formulas and outputs from a numpy restatement of the
legacy tests' `expected` (f32 left-to-right sum) -- neither uses the C oracle, so the file pins it.
Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from oracle import ref  # only the pure-Python fixture generators and closed forms are used here


def case(name, fmt, packed, value_fn, x, rows, cols, m):
    dense = np.array([[value_fn(r, c) for c in range(cols)] for r in range(rows)], dtype=np.float32)
    y = ref.closed_form_expected(value_fn, x, m, rows, cols)
    return {"name": name, "format": fmt, "rows": rows, "cols": cols, "m": m,
            "packed_u8": packed.tolist(), "x_bits": x.view(np.uint32).tolist(),
            "dense_bits": dense.view(np.uint32).ravel().tolist(),
            "y_f32seq_bits": y.view(np.uint32).ravel().tolist()}


cases = [
    case("qk_tests Q4_K (5, 512) m=3", "q4_k", ref.qk_q4k_packed(5, 512), ref.qk_q4k_value, ref.qk_input(3, 512), 5, 512, 3),
    case("qk_tests Q5_K (5, 512) m=3", "q5_k", ref.qk_q5k_packed(5, 512), ref.qk_q5k_value, ref.qk_input(3, 512), 5, 512, 3),
    case("qk_tests Q6_K (5, 512) m=2", "q6_k", ref.qk_q6k_packed(5, 512), ref.qk_q6k_value, ref.qk_input(2, 512), 5, 512, 2),
    case("q6_k_tests (6, 768) m=1", "q6_k", ref.q6_packed(6, 768), ref.q6_value, ref.q6_input(1, 768), 6, 768, 1),
    case("q8_0_tests (7, 128) m=2", "q8_0", ref.q8_packed(7, 128), ref.q8_value, ref.q8_input(2, 128), 7, 128, 2),
]
out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "closed_form.json")
with open(out, "w") as f:
    json.dump({"source": "closed-form fixtures of the reference's legacy K-quant tests", "cases": cases}, f)
print(out, os.path.getsize(out))
