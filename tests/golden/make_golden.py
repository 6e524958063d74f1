"""Generate golden vectors for the reference compressed-weight layout.

Run in a container that has the reference checkout; it imports the reference's
own packer (convert/convert_utils.py: reorder_weight, compress_weight) on
small seeded ternary matrices and stores inputs and outputs in
``ref_packer_golden.npz`` next to this script.  The tests only read the .npz.

    python tests/golden/make_golden.py /path/to/reference
"""
import os
import sys

import numpy as np
import torch


def ternary(n, k, p_zero, seed):
    rng = np.random.default_rng(seed)
    r = rng.random((n, k))
    sign = rng.integers(0, 2, size=(n, k), dtype=np.int8) * 2 - 1
    return np.where(r < p_zero, 0, sign).astype(np.int8)


CASES = [  # name, N, K, P(0), seed
    ("t64x64_p45", 64, 64, 0.45, 1),
    ("t128x192_p45", 128, 192, 0.45, 2),
    ("t64x256_p90", 64, 256, 0.90, 3),
    ("t192x64_p00", 192, 64, 0.0, 4),
    ("t64x128_p100", 64, 128, 1.0, 5),
    ("t256x320_p45", 256, 320, 0.45, 6),
]


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "convert"))
    import convert_utils as cu  # the reference's packer

    out = {}
    for name, n, k, p, seed in CASES:
        w = ternary(n, k, p, seed)
        wt = torch.from_numpy(w)
        cv, tg, tm, bm = cu.compress_weight(wt)
        out[name + "/w"] = w
        out[name + "/reordered"] = cu.reorder_weight(wt).numpy()
        out[name + "/compressed_val"] = cv.numpy().astype(np.uint32)
        out[name + "/tile_offsets"] = tg.numpy().astype(np.int32)
        out[name + "/median_offsets"] = tm.numpy().astype(np.uint16)
        out[name + "/bitmap"] = bm.numpy().astype(np.uint64)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_packer_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TERNAINFER_REFERENCE")
    if not root:
        sys.exit("usage: make_golden.py <path of the Gu-J/TernaInfer checkout>  (or set TERNAINFER_REFERENCE)")
    main(root)
