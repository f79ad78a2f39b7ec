"""CPU tests of the oracle itself: known answers, an independent dense brute force, golden vectors."""
import os

import numpy as np
import pytest

from conftest import canonical_rulebook

# the reference checkout, when it sits beside this repository (or where SESSD_REFERENCE_ROOT points)
_REFERENCE = os.environ.get("SESSD_REFERENCE_ROOT",
                            os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference"))
KITTI0 = os.path.join(_REFERENCE, "data", "kitti_training_velodyne_reduced", "000000.bin")
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_np_round_matches_numpy_rule(oracle):
    # half-way cases go to even (voxelGenerator.cu:61-68); others round to nearest
    for x, want in [(0.5, 0), (1.5, 2), (2.5, 2), (3.5, 4), (40.0, 40), (39.6, 40), (1407.9999, 1408), (0.49, 0)]:
        assert oracle.np_round(x) == want


def test_grid_size_of_reference_geometry(oracle, pkg):
    # (70.4-0)/0.05, (40+40)/0.05, (1+3)/0.1 in fp32 -> 1408 x 1600 x 40; the conv stack then uses Z = 41
    assert oracle.grid_size(pkg.synth.POINT_RANGE, pkg.synth.VOXEL_SIZE) == (1408, 1600, 40)


@pytest.mark.skipif(not os.path.exists(KITTI0), reason="reference lidar frame not reachable")
def test_known_voxel_count_of_first_reference_frame(oracle, pkg):
    # 16825 is the only known-answer value in the reference tree (submConv3dlayer.cu:254, :618)
    pts = np.fromfile(KITTI0, dtype=np.float32).reshape(-1, 4)
    _, _, _, n, st = oracle.voxelize(pts, pkg.synth.POINT_RANGE, pkg.synth.VOXEL_SIZE, 60000)
    assert (n, st) == (16825, 0)


def test_voxelize_hand_case(oracle):
    rng, vs = (0.0, 0.0, 0.0, 4.0, 4.0, 2.0), (1.0, 1.0, 1.0)
    pts = np.array([
        [0.5, 0.5, 0.5, 1.0],    # voxel (z0,y0,x0)  row 0
        [3.5, 0.5, 1.5, 2.0],    # voxel (1,0,3)     row 1
        [0.25, 0.75, 0.1, 3.0],  # row 0 again
        [4.0, 0.5, 0.5, 9.0],    # x == max: dropped
        [-0.1, 0.5, 0.5, 9.0],   # x < min: dropped
        [0.9, 0.9, 0.9, 5.0],    # row 0
        [0.1, 0.1, 0.1, 7.0], [0.2, 0.2, 0.2, 7.0], [0.3, 0.3, 0.3, 7.0],  # row 0: points 4,5,6 of the voxel
        [0.4, 0.4, 0.4, 100.0],  # 7th point of row 0: beyond max 5, ignored
    ], np.float32)
    vox, coors, npv, n, st = oracle.voxelize(pts, rng, vs, max_voxels=8, max_pts=5)
    assert n == 2 and st == 0
    assert coors[:2].tolist() == [[0, 0, 0, 0], [0, 1, 0, 3]]
    assert npv[:2].tolist() == [5, 1]
    kept = pts[[0, 2, 5, 6, 7]]
    want = kept[0].copy()
    for r in kept[1:]:
        want = want + r
    np.testing.assert_array_equal(vox[0], want / np.float32(5))
    np.testing.assert_array_equal(vox[1], pts[1])
    assert not vox[2:].any() and not coors[2:].any()


def test_voxelize_overflow_keeps_first_voxels(oracle):
    rng, vs = (0.0, 0.0, 0.0, 8.0, 1.0, 1.0), (1.0, 1.0, 1.0)
    pts = np.array([[x + 0.5, 0.5, 0.5, float(x)] for x in [5, 1, 7, 3, 1, 0]], np.float32)
    vox, coors, npv, n, st = oracle.voxelize(pts, rng, vs, max_voxels=3)
    assert n == 3 and st == oracle.VOXEL_OVERFLOW
    assert coors[:3, 3].tolist() == [5, 1, 7] and npv[:3].tolist() == [1, 2, 1]


def _dense_conv_bruteforce(coors, feat, W, K, S, P, in_shape, out_shape, subm):
    """Definition-level dense evaluation: out[o] = sum_k in[o*s - p + k] W[k]; active set per the plugin rules."""
    Cin, Cout = W.shape[1], W.shape[2]
    dense = np.zeros(tuple(in_shape) + (Cin,), np.float64)
    act = np.zeros(tuple(in_shape), bool)
    for c, f in zip(coors, feat):
        dense[c[1], c[2], c[3]] = f
        act[c[1], c[2], c[3]] = True
    out = {}
    trip = []
    for oz in range(out_shape[0]):
        for oy in range(out_shape[1]):
            for ox in range(out_shape[2]):
                if subm and not act[oz, oy, ox]:
                    continue
                acc = np.zeros(Cout)
                hit = False
                for kz in range(K[0]):
                    for ky in range(K[1]):
                        for kx in range(K[2]):
                            iz, iy, ix = oz * S[0] - P[0] + kz, oy * S[1] - P[1] + ky, ox * S[2] - P[2] + kx
                            if 0 <= iz < in_shape[0] and 0 <= iy < in_shape[1] and 0 <= ix < in_shape[2] and act[iz, iy, ix]:
                                k = (kz * K[1] + ky) * K[2] + kx
                                acc += dense[iz, iy, ix] @ W[k].astype(np.float64)
                                hit = True
                                trip.append((k, (iz * in_shape[1] + iy) * in_shape[2] + ix,
                                             (oz * out_shape[1] + oy) * out_shape[2] + ox))
                if hit:
                    out[(oz, oy, ox)] = acc
    trip = np.array(sorted(trip), np.int64).reshape(-1, 3)
    return out, trip


CASES = [
    # subm, K, S, P, in_shape
    (True, (3, 3, 3), (1, 1, 1), (1, 1, 1), (4, 6, 5)),
    (False, (3, 3, 3), (2, 2, 2), (1, 1, 1), (5, 8, 6)),
    (False, (3, 3, 3), (2, 2, 2), (0, 1, 1), (11, 8, 6)),
    (False, (3, 1, 1), (2, 1, 1), (0, 0, 0), (5, 6, 7)),
]


@pytest.mark.parametrize("subm,K,S,P,in_shape", CASES)
def test_rulebook_and_conv_against_dense_bruteforce(oracle, subm, K, S, P, in_shape):
    rs = np.random.RandomState(7)
    out_shape = in_shape if subm else tuple((in_shape[j] + 2 * P[j] - K[j]) // S[j] + 1 for j in range(3))
    vol = int(np.prod(in_shape))
    n = vol // 3
    cells = rs.permutation(vol)[:n]
    coors = np.zeros((n, 4), np.int32)
    coors[:, 1], coors[:, 2], coors[:, 3] = cells // (in_shape[1] * in_shape[2]), (cells // in_shape[2]) % in_shape[1], cells % in_shape[2]
    Cin, Cout, maxV = 4, 16, 256
    feat = rs.randn(n, Cin).astype(np.float32)
    W = rs.randn(int(np.prod(K)), Cin, Cout).astype(np.float32)
    if subm:
        pairs, num, st = oracle.subm_rulebook(coors, n, in_shape, maxV)
        ocoors, on = coors, n
    else:
        ocoors, on, pairs, num, st = oracle.spconv_rulebook(coors, n, K, S, P, out_shape, maxV)
    assert st == 0
    want, want_trip = _dense_conv_bruteforce(coors, feat, W, K, S, P, in_shape, out_shape, subm)
    got_trip = canonical_rulebook(pairs, num, coors, ocoors[:on], in_shape, out_shape)
    np.testing.assert_array_equal(got_trip, want_trip)
    assert on == len(want)
    out = oracle.conv_apply(feat, pairs, num, W, on)
    out64 = oracle.conv_apply_f64(feat, pairs, num, W, on)
    for r in range(on):
        key = tuple(int(v) for v in ocoors[r, 1:])
        np.testing.assert_allclose(out64[r], want[key], rtol=1e-12, atol=1e-12)
        np.testing.assert_allclose(out[r], want[key], rtol=2e-5, atol=2e-5)


def test_spconv_output_numbering_is_first_seen_order(oracle):
    coors = np.array([[0, 4, 4, 4], [0, 0, 0, 0], [0, 4, 4, 5]], np.int32)
    oc, on, pairs, num, st = oracle.spconv_rulebook(coors, 3, (3, 3, 3), (2, 2, 2), (1, 1, 1), (3, 4, 4), 64)
    # input (4,4,4) (even coords, pad 1) has the single candidate (2,2,2); (0,0,0) -> (0,0,0); (4,4,5) -> x in {3,2}
    assert on == 3 and st == 0
    assert oc[0].tolist() == [0, 2, 2, 2] and oc[1].tolist() == [0, 0, 0, 0] and oc[2].tolist() == [0, 2, 2, 3]


def test_scale_shift_relu_and_fold(oracle):
    g, b, m, v = [np.array(t, np.float32) for t in ([1.5, 0.5], [0.1, -0.2], [0.3, 0.4], [0.25, 4.0])]
    sc, sh = oracle.fold_bn(g, b, m, v, 1e-5)
    np.testing.assert_allclose(sc, g / np.sqrt(v + 1e-5), rtol=1e-6)
    np.testing.assert_allclose(sh, b - m * g / np.sqrt(v + 1e-5), rtol=1e-6)
    x = np.array([[1.0, -3.0], [-1.0, 2.0]], np.float32)
    y = oracle.scale_shift_relu(x, sc, sh)
    np.testing.assert_allclose(y, np.maximum(0, x * sc + sh), rtol=1e-6)


def test_sparse2dense_layout(oracle):
    feat = np.arange(2 * 3, dtype=np.float32).reshape(2, 3) + 1
    coors = np.array([[0, 1, 2, 3], [0, 0, 0, 1]], np.int32)
    d = oracle.sparse2dense(feat, coors, 2, 3, 2, 4, 5)
    assert d.shape == (1, 6, 4, 5)
    for c in range(3):
        assert d[0, c * 2 + 1, 2, 3] == feat[0, c] and d[0, c * 2 + 0, 0, 1] == feat[1, c]
    assert np.count_nonzero(d) == 6


def test_golden_vectors(oracle, pkg):
    """The committed fixtures (tests/golden/make_golden.py) pin the oracle against silent drift."""
    g = np.load(os.path.join(GOLDEN, "front_end_small.npz"))
    import make_golden_inputs as mk

    case = mk.small_case(pkg)
    r = oracle.front_end(case["points"], case["range"], case["voxel"], case["max_voxels"], case["layers"],
                         np.concatenate([w.ravel() for w in case["weights"]]), np.concatenate(case["scale"]),
                         np.concatenate(case["shift"]), fp16=False, bev=case["bev"])
    np.testing.assert_array_equal(r["layer_rows"], g["layer_rows"])
    np.testing.assert_array_equal(r["layer_pairs"], g["layer_pairs"])
    np.testing.assert_array_equal(r["coors"], g["coors"])
    np.testing.assert_array_equal(r["feat"], g["feat"])
    nz = np.flatnonzero(r["dense"])
    np.testing.assert_array_equal(nz, g["dense_nz"])
    np.testing.assert_array_equal(r["dense"].ravel()[nz], g["dense_val"])


# ---- detection post-processing (anchor decode, score filter) -------------------------------------------

KITTI_RANGE = (0.0, -40.0, -3.0, 70.4, 40.0, 1.0)
CAR = (3.9, 1.6, 1.56)
ANGLES = (0.0, 1.57)


def test_anchor_layout_and_identity_decode(oracle):
    """Zero regression outputs give the anchors themselves (generateAnchorDecode.cu:201-247): x fastest,
    two yaws per cell, centres at half a stride from the range minimum, z = -1, (w, l, h) order."""
    H, W = 200, 176
    ap = oracle.anchor_params(KITTI_RANGE, CAR, ANGLES)
    out = oracle.anchor_decode(np.zeros((H * W * 2, 7), np.float32), ap, H, W, 2)
    f = np.float32
    sx, sy = f(f(70.4) - f(0.0)) / f(W), f(f(40.0) - f(-40.0)) / f(H)
    assert out[0].tolist() == [f(0.0) + sx / f(2), f(-40.0) + sy / f(2), -1.0, f(1.6), f(3.9), f(1.56), 0.0]
    assert out[1, 6] == f(1.57) and out[1, 0] == out[0, 0]
    assert out[2, 0] == f(0.0) + sx / f(2) + f(1) * sx                 # next cell along x
    assert out[2 * W, 1] == f(-40.0) + sy / f(2) + f(1) * sy           # next row along y
    assert out[-1, 0] == f(0.0) + sx / f(2) + f(W - 1) * sx and out[-1, 1] == f(-40.0) + sy / f(2) + f(H - 1) * sy


def test_anchor_decode_against_numpy(oracle):
    H, W = 9, 11
    rs = np.random.RandomState(3)
    t = (rs.randn(H * W * 2, 7) * 0.5).astype(np.float32)
    out = oracle.anchor_decode(t, oracle.anchor_params(KITTI_RANGE, CAR, ANGLES), H, W, 2)
    idx = np.arange(H * W * 2)
    f = np.float32
    sx, sy = f(70.4) / f(W), f(80.0) / f(H)
    ax = (f(0.0) + sx / f(2)) + ((idx % (W * 2)) // 2).astype(np.float32) * sx
    ay = (f(-40.0) + sy / f(2)) + (idx // (W * 2)).astype(np.float32) * sy
    diag = np.sqrt(f(3.9) * f(3.9) + f(1.6) * f(1.6), dtype=np.float32)
    want = np.stack([t[:, 0] * diag + ax, t[:, 1] * diag + ay, t[:, 2] * f(1.56) + f(-1.0),
                     np.exp(t[:, 3]) * f(1.6), np.exp(t[:, 4]) * f(3.9), np.exp(t[:, 5]) * f(1.56),
                     t[:, 6] + np.where(idx % 2 == 0, f(0.0), f(1.57))], axis=1).astype(np.float32)
    np.testing.assert_allclose(out, want, rtol=1e-6, atol=1e-6)


def test_filter_boxes_hand_case(oracle):
    """Six anchors, threshold 0.45 (logit of 0.45 is about -0.2007)."""
    boxes = np.arange(42, dtype=np.float32).reshape(6, 7)
    boxes[:, 6] = [0.5, -0.5, 0.5, -0.5, 0.0, 2.0]
    cls = np.array([3.0, -5.0, 0.0, -0.19, -0.21, 10.0], np.float32)     # pass: 0, 2, 3, 5
    iou = np.array([1.0, 1.0, 0.0, -1.0, 1.0, 0.5], np.float32)
    dirs = np.array([[1, 0], [0, 0], [0, 1], [0, 1], [0, 0], [2, 2]], np.float32)
    ob, oc, oi, od, valid, passed = oracle.filter_boxes(boxes, cls, iou, dirs, 2, 3, 0.45, 0.0)
    assert (valid, passed) == (3, 4)                       # anchor 5 passes too but the table holds 3 rows
    np.testing.assert_array_equal(ob[:, :6], boxes[[0, 2, 3], :6])
    np.testing.assert_array_equal(od, [0, 1, 1])
    np.testing.assert_array_equal(oi, [1.0, 0.5, 0.0])
    f = np.float32
    # anchor 0: direction 0 and yaw > 0 -> yaw + pi; anchor 2: direction 1, yaw > 0 -> kept; anchor 3:
    # direction 1 and yaw < 0 -> yaw + pi
    np.testing.assert_array_equal(ob[:, 6], [f(0.5) + f(3.1415926), f(0.5), f(-0.5) + f(3.1415926)])
    s0 = f(1) / (f(1) + np.exp(f(-3.0)))
    np.testing.assert_allclose(oc, [s0, f(0.5) * f(0.5) ** 4, 0.0], rtol=1e-6)
    np.testing.assert_array_equal(ob[:, 8], oc)
    assert not ob[:, 7].any()
    # a tie between the two directions selects the later one (>= in the reference loop)
    _, _, _, od2, _, _ = oracle.filter_boxes(boxes, cls, iou, dirs, 2, 6, 0.45, 0.0)
    assert od2[3] == 1 and od2[:4].tolist() == [0, 1, 1, 1]


def test_filter_boxes_against_numpy(oracle):
    rs = np.random.RandomState(8)
    n = 5000
    boxes = rs.randn(n, 7).astype(np.float32)
    cls = (rs.randn(n) * 2 - 2).astype(np.float32)
    iou = rs.uniform(-1, 1, n).astype(np.float32)
    dirs = rs.randn(n, 2).astype(np.float32)
    ob, oc, oi, od, valid, passed = oracle.filter_boxes(boxes, cls, iou, dirs, 2, 10000, 0.45, 0.0)
    score = (np.float32(1) / (np.float32(1) + np.exp(-cls))).astype(np.float32)
    keep = np.nonzero(score >= np.float32(0.45))[0]
    assert valid == passed == len(keep)
    q = ((iou[keep] + np.float32(1)) * np.float32(0.5)).astype(np.float32)
    np.testing.assert_array_equal(oi[:valid], q)
    np.testing.assert_allclose(oc[:valid], score[keep] * q * q * q * q, rtol=1e-6)
    best = (dirs[keep, 1] >= dirs[keep, 0]).astype(np.float32)
    np.testing.assert_array_equal(od[:valid], best)
    yaw = boxes[keep, 6]
    flip = ((best == 1) & (yaw < 0)) | ((best == 0) & (yaw > 0))
    np.testing.assert_array_equal(ob[:valid, 6], np.where(flip, yaw + np.float32(3.1415926), yaw).astype(np.float32))
    assert not ob[valid:].any() and not oc[valid:].any()


# ---- rotated NMS -------------------------------------------------------------------------------

def _box(x, y, w, l, yaw, score, z=0.0, h=1.5, label=0.0):
    return np.array([x, y, z, w, l, h, yaw, label, score], np.float32)


def test_bev_iou_hand_cases(oracle):
    a = _box(0, 0, 2, 4, 0.0, 0.9)
    assert abs(oracle.bev_iou(a, a) - 1.0) < 1e-5
    assert oracle.bev_iou(a, _box(10, 0, 2, 4, 0.0, 0.5)) == 0.0                 # disjoint
    # shifted by half the width: overlap 1 x 4 = 4, union 8 + 8 - 4
    assert abs(oracle.bev_iou(a, _box(1, 0, 2, 4, 0.0, 0.5)) - 4.0 / 12.0) < 1e-5
    # the same box turned by 90 degrees: the 2 x 2 centre square is shared
    assert abs(oracle.bev_iou(a, _box(0, 0, 2, 4, np.pi / 2, 0.5)) - 4.0 / 12.0) < 1e-4
    # a small box inside a large one: no edge crossings, only contained corners
    assert abs(oracle.bev_iou(_box(0, 0, 10, 10, 0.3, 0.9), _box(1, 1, 2, 2, 1.0, 0.5)) - 4.0 / 100.0) < 1e-4


def test_bev_iou_against_rasterised_area(oracle):
    """Independent check: area of the intersection counted on a fine grid."""
    rs = np.random.RandomState(21)
    g = (np.arange(600) + 0.5) / 600 * 12 - 6
    gx, gy = np.meshgrid(g, g)

    def inside(b):
        c, s = np.cos(-b[6]), np.sin(-b[6])
        rx, ry = (gx - b[0]) * c - (gy - b[1]) * s, (gx - b[0]) * s + (gy - b[1]) * c
        return (np.abs(rx) < b[3] / 2) & (np.abs(ry) < b[4] / 2)

    for _ in range(40):
        a = _box(rs.uniform(-1, 1), rs.uniform(-1, 1), rs.uniform(1, 3), rs.uniform(2, 5), rs.uniform(-3, 3), 0.5)
        b = _box(rs.uniform(-1, 1), rs.uniform(-1, 1), rs.uniform(1, 3), rs.uniform(2, 5), rs.uniform(-3, 3), 0.5)
        ia, ib = inside(a), inside(b)
        inter, union = (ia & ib).sum(), (ia | ib).sum()
        assert abs(oracle.bev_iou(a, b) - inter / union) < 2e-2


def test_rotated_nms_order_and_suppression(oracle):
    boxes = np.stack([
        _box(0, 0, 2, 4, 0.0, 0.50),        # 0: suppressed by 2 (same place, lower score)
        _box(20, 0, 2, 4, 0.3, 0.90),       # 1: best, kept
        _box(0.2, 0, 2, 4, 0.0, 0.80),      # 2: kept
        _box(20.1, 0.1, 2, 4, 0.3, 0.85),   # 3: suppressed by 1
        _box(-20, 5, 2, 4, 1.0, 0.10),      # 4: far away, kept last
        _box(40, 40, 2, 4, 0.0, 0.80),      # 5: same score as 2, later row: after 2
    ])
    kept, order = oracle.rotated_nms(boxes, 0.01)
    assert order.tolist() == [1, 2, 5, 4]
    np.testing.assert_array_equal(kept, boxes[[1, 2, 5, 4]])
    # touching corners only: IoU far below the 0.01 threshold, both kept
    two = np.stack([_box(0, 0, 2, 2, 0.0, 0.9), _box(1.99, 1.99, 2, 2, 0.0, 0.8)])
    assert oracle.rotated_nms(two, 0.01)[1].tolist() == [0, 1]
    assert oracle.rotated_nms(np.zeros((0, 9), np.float32), 0.01)[1].tolist() == []
