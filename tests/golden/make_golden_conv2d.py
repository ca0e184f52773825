"""Generates tests/golden/reference_conv2d.npz by running the REFERENCE's own C kernel
`hodu_cpu_conv2d_f32_fallback` (ops_conv.c, compiled into oracle/_ref by oracle/build.py) on
small seeded inputs.  Needs the reference tree; the committed .npz is what the tests read.

    python tests/golden/make_golden_conv2d.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from hodu_b200.op_metadatas import conv2d_metadata  # noqa: E402
from oracle import oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# name: batch, in_channels, out_channels, (H, W), (KH, KW), stride, padding, dilation, offsets
CASES = {
    "k3_pad1": (2, 3, 4, (9, 11), (3, 3), (1, 1), (1, 1), (1, 1), (0, 0)),
    "stride2_dilated": (1, 2, 5, (12, 10), (3, 2), (2, 1), (0, 1), (1, 2), (0, 0)),
    "pointwise": (2, 4, 3, (6, 6), (1, 1), (1, 1), (0, 0), (1, 1), (0, 0)),
    "pointwise_stride2": (1, 3, 2, (7, 8), (1, 1), (2, 2), (0, 0), (1, 1), (0, 0)),
    "k5_pad2_offsets": (1, 2, 3, (8, 8), (5, 5), (1, 1), (2, 2), (1, 1), (5, 3)),
    "wide_rows": (1, 1, 2, (4, 37), (2, 3), (1, 2), (1, 0), (1, 1), (0, 0)),
}


def main():
    ref = O.ref()
    if ref is None or not hasattr(ref.base, "hodu_cpu_conv2d_f32_fallback"):
        raise SystemExit("oracle/_ref (with ops_conv.c) is missing and the reference tree is not mounted")
    rng = np.random.Generator(np.random.Philox(key=777))
    out = {}
    for name, (b, ci, co, hw, k, s, p, d, offs) in CASES.items():
        md = conv2d_metadata(b, ci, co, hw, k, s, p, d, offs[0], offs[1])
        x = rng.standard_normal(offs[0] + b * ci * hw[0] * hw[1], dtype=np.float32)
        w = rng.standard_normal(offs[1] + co * ci * k[0] * k[1], dtype=np.float32)
        y = np.zeros(md[0], dtype=np.float32)
        ref.call("hodu_cpu_conv2d_f32_fallback", x, w, y, md)
        out[name + "__md"] = np.array(md, dtype=np.int64)
        out[name + "__in"], out[name + "__w"], out[name + "__out"] = x, w, y
    np.savez_compressed(os.path.join(HERE, "reference_conv2d.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
