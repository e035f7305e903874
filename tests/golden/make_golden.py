"""Regenerates tests/golden/digests.json and tests/golden/tiny_tnn.npz from the
reference's own compiled objects (oracle/_ref/libtnns_ref.so, built by oracle/Makefile
from the reference sources).  Run from the repository root:

    make -C oracle && python tests/golden/make_golden.py

Each digest is the SHA-256 of the raw bytes of (packed weights, packed im2row matrix,
fp32 NCHW layer output) that the reference produces for one seeded case of
tests/cases.py.  The reference library is needed only here; the tests read the JSON.
"""
import hashlib
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from cases import act_ternary, extra_cases, make_case, reference_test_cases, wgt_ternary, TNN  # noqa: E402
from fastertnn_b200.workloads import Layer  # noqa: E402
from oracle import binding  # noqa: E402


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def golden_cases():
    return (reference_test_cases(N=2, dist="uniform", max_ops=3e9)
            + reference_test_cases(N=2, dist="alphabet", max_ops=3e9)
            + extra_cases())


def main():
    R = binding.ref()
    if R is None:
        raise SystemExit("oracle/_ref/libtnns_ref.so is missing: run `make -C oracle` where the reference sources are")
    out = {}
    for c in golden_cases():
        c = c.build()
        wp = R.pack_weights(wgt_ternary(c.type), c.w, c.w_thr)
        ap = R.pack(act_ternary(c.type), c.x, c.thr, c.kernel_hw, c.padding, c.stride)
        y = R.conv(c.type, c.x, c.thr, wp, c.kernel_hw, c.padding, c.stride, c.alpha)
        out[c.name] = {"weights": sha(wp), "packed": sha(ap), "output": sha(y), "N": c.N}
    here = Path(__file__).resolve().parent
    (here / "digests.json").write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
    # one tiny case stored in full, for debugging without any oracle
    c = make_case(TNN, Layer(70, 4, 5, 6, 3, 3, 1, 1), 2, 424242, "uniform", name="tiny")
    wp = R.pack_weights(True, c.w, c.w_thr)
    np.savez_compressed(here / "tiny_tnn.npz", x=c.x, thr=c.thr, w=c.w, w_thr=c.w_thr, packed_w=wp,
                        packed_a=R.pack(True, c.x, c.thr, c.kernel_hw, c.padding, c.stride),
                        y=R.conv(TNN, c.x, c.thr, wp, c.kernel_hw, c.padding, c.stride, c.alpha))
    print(f"wrote {len(out)} digests")


if __name__ == "__main__":
    main()
