"""Generate tests/golden/e8_golden.npz from the reference's own E8 decode.

Runs where the reference sources are mounted: `make -C oracle ref` compiles
cpp/src/neighbors/octex/detail/e8.cuh of hpdic/octex for the host (oracle/_ref/libe8_ref.so), and
this script feeds it seeded points (uniform in [-6, 6], the first 1 000 coordinates moved onto exact
half-integer ties, as the reference's own unit test does in cpp/tests/test_build.cu:94-105) and
stores the points, the decoded lattice points and the cell codes.  The fixture travels; the
reference does not.

    python tests/golden/make_e8_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle_py  # noqa: E402


def main():
    oracle_py.build(force=True)
    ref = oracle_py.ref_e8()
    if ref is None:
        raise SystemExit("oracle/_ref/libe8_ref.so is missing: the reference sources are not here")
    rng = np.random.default_rng(7)
    n, b = 4096, 4
    x = rng.uniform(-6.0, 6.0, size=(n, 8 * b)).astype(np.float32)
    flat = x.reshape(-1)
    flat[:1000] = np.round(flat[:1000] * 2.0) * 0.5
    out = {"x": x}
    for name, inv in (("inv_2p5", np.float32(1.0 / 2.5)), ("inv_1", np.float32(1.0)),
                      ("inv_0p2", np.float32(1.0 / 5.0))):
        out["codes_" + name] = oracle_py.cell_code(x, b, float(inv), which=ref)
        out["scale_" + name] = np.float32(inv)
    out["points_inv_1"] = oracle_py.e8_point(x[:512], which=ref)
    # other block counts on the same coordinates
    for bb in (1, 2, 3, 8):
        rows = (n * 8 * b) // (8 * bb)
        sub = np.ascontiguousarray(x.reshape(-1)[:rows * 8 * bb].reshape(rows, 8 * bb))
        out[f"codes_b{bb}"] = oracle_py.cell_code(sub, bb, 0.4, which=ref)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "e8_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
