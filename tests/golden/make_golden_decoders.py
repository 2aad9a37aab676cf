"""Generates tests/golden/golden_decoders.npz from the reference's OWN ggml build (oracle/_ref, variant `base`): for
every block type that the executor reads through its element decoders only (q4_1 q5_0 q5_1 q2_K q3_K q5_K q6_K), the
bytes ggml_quantize_chunk gives for seeded rows (random and edge-case rows) and the values ggml's dequantizer gives
back for them.

    python tests/golden/make_golden_decoders.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from make_golden import hard_rows  # noqa: E402
from oracle.bindings import Q2_K, Q3_K, Q4_1, Q5_0, Q5_1, Q5_K, Q6_K, Ref  # noqa: E402

TYPES = ((Q4_1, "q4_1"), (Q5_0, "q5_0"), (Q5_1, "q5_1"), (Q2_K, "q2_K"), (Q3_K, "q3_K"), (Q5_K, "q5_K"), (Q6_K, "q6_K"))


def main():
    ref = Ref("base")
    rng = np.random.default_rng(20241125)
    x = np.concatenate([(rng.standard_normal((8, 512)) * 0.02).astype(np.float32), hard_rows(rng, 8, 512),
                        rng.standard_normal((8, 512)).astype(np.float32)])
    out = {"x": x}
    for ty, nm in TYPES:
        out["quant_" + nm] = ref.quantize(ty, x)
        out["dequant_" + nm] = ref.dequantize(ty, out["quant_" + nm], 512)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_decoders.npz"), **out)
    print("wrote %d arrays" % len(out))


if __name__ == "__main__":
    main()
