"""Regenerates tests/golden/*.npz from the CPU oracle:  python tests/golden/make_golden.py

The reference ships no golden vectors and cannot be executed without TensorRT, so these fixtures
freeze the oracle's own results (which are pinned to the reference by reading, by a definition-level
dense brute force in tests/test_oracle.py and by the reference's single known voxel count). Their job
is to catch silent drift of the oracle and to give the GPU tests a second, file-based target.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)

from conftest import load_package  # noqa: E402
import make_golden_inputs as mk  # noqa: E402
from oracle import binding as oracle  # noqa: E402


def main():
    pkg = load_package()
    case = mk.small_case(pkg)
    r = oracle.front_end(case["points"], case["range"], case["voxel"], case["max_voxels"], case["layers"],
                         np.concatenate([w.ravel() for w in case["weights"]]), np.concatenate(case["scale"]),
                         np.concatenate(case["shift"]), fp16=False, bev=case["bev"])
    assert r["status"] == 0
    nz = np.flatnonzero(r["dense"])
    np.savez_compressed(os.path.join(HERE, "front_end_small.npz"), layer_rows=r["layer_rows"],
                        layer_pairs=r["layer_pairs"], coors=r["coors"], feat=r["feat"], dense_nz=nz,
                        dense_val=r["dense"].ravel()[nz])
    print("rows", r["layer_rows"], "pairs", r["layer_pairs"], "final", r["num"])
    # a small weight file in the exporter's text format (tools/gen_wts.py:85-99), written by the pure-Python
    # restatement of that loop; tests/test_formats.py reads it with the library and compares bit patterns
    from oracle import formats as oracle_formats

    oracle_formats.write_wts(os.path.join(HERE, "tiny.wts"), tiny_wts_blobs())


def tiny_wts_blobs():
    """Blobs of tests/golden/tiny.wts: seeded values plus the special bit patterns a reader can get wrong."""
    rng = np.random.default_rng(12345)
    return [
        ("backbone.middle_conv.0.weight", rng.standard_normal((3, 2, 4)).astype(np.float32)),
        ("backbone.middle_conv.1.running_var", rng.uniform(0.5, 2.0, 4).astype(np.float32)),
        ("special", np.array([0x00000000, 0x80000000, 0x7F800000, 0xFF800000, 0x7FC00001, 0x00000001, 0x7F7FFFFF],
                             np.uint32).view(np.float32)),
        ("empty", np.zeros((0,), np.float32)),
    ]


if __name__ == "__main__":
    main()
