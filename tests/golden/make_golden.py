"""Regenerates ``qmatmul_small.npz`` from the C oracle (``oracle/candy_oracle.c``).

    python tests/golden/make_golden.py

The reference ships no golden vector for this path, so these fixtures are outputs of the
restated algorithm on seeded inputs: they pin the oracle against regressions and give the
GPU tests fixed bytes to reproduce.  Hand-derived known answers live in the tests
themselves, not here.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle_c as oc  # noqa: E402

OUT = Path(__file__).resolve().parent / "qmatmul_small.npz"


def main():
    rng = np.random.default_rng(20240521)
    n, k, m = 24, 256, 3
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    w[1, 32:64] = 0.0                      # an all-zero block
    w[2, 0:32] = np.float32(3e-8)          # scale underflows to an f16 subnormal / zero
    w[3, 64] = np.float32(-0.5)            # a dominant negative extreme
    w[3, 65] = np.float32(0.5)             # tie in magnitude with the opposite sign, later in order
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[2, 96:128] = 0.0                     # a zero activation block (Q8_1 amax == 0 branch)
    out = {"w": w, "x": x}
    for qt, name in ((oc.Q4_0, "q4_0"), (oc.Q8_0, "q8_0")):
        for order in (0, 1):
            if qt == oc.Q8_0 and order == 1:
                continue
            tag = f"{name}_o{order}"
            blocks = oc.quantize(qt, order, w)
            out[f"{tag}_blocks"] = blocks
            out[f"{tag}_deq"] = oc.dequantize(qt, order, blocks)
            out[f"{tag}_y"] = oc.qmatmul(qt, order, x, blocks, n)
            out[f"{tag}_y_q8_1"] = oc.qmatmul(qt, order, x, blocks, n, q8_1=True)
    out["x_q8_1"] = oc.quantize_q8_1(x)
    np.savez_compressed(OUT, **out)
    print(OUT, OUT.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
