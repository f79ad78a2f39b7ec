"""GPU parity: sessd_voxelize_enqueue against the oracle (coords / counts bit-exact, features <= 1e-5)."""
import numpy as np
import pytest

from conftest import canonical_voxels

pytestmark = pytest.mark.gpu


def _run(gpu, frames, max_voxels, point_range=None, voxel_size=None, max_points=None, out_dtype=0, max_pts=5):
    import torch

    point_range = point_range or gpu.synth.POINT_RANGE
    voxel_size = voxel_size or gpu.synth.VOXEL_SIZE
    P = max_points or max(max(len(f) for f in frames), 1)
    pts = np.zeros((len(frames), P, 4), np.float32)
    sizes = np.zeros(len(frames), np.int32)
    for b, f in enumerate(frames):
        pts[b, :len(f)] = f
        sizes[b] = len(f)
    params = gpu.voxel_params(max_voxels, point_range, voxel_size, max_pts)
    r = gpu.voxelize(torch.from_numpy(pts).cuda(), torch.from_numpy(sizes).cuda(), params, out_dtype)
    return {k: (v.cpu().numpy() if hasattr(v, "cpu") else v) for k, v in r.items()}, params


def _compare(gpu, oracle, frames, max_voxels, point_range=None, voxel_size=None, max_pts=5, expect_status=0):
    point_range = point_range or gpu.synth.POINT_RANGE
    voxel_size = voxel_size or gpu.synth.VOXEL_SIZE
    r, params = _run(gpu, frames, max_voxels, point_range, voxel_size, max_pts=max_pts)
    grid = (params.grid_z, params.grid_y, params.grid_x)
    assert r["status"] == expect_status
    for b, f in enumerate(frames):
        vox, coors, npv, n, st = oracle.voxelize(f, point_range, voxel_size, max_voxels, max_pts, batch_idx=b)
        assert int(r["voxel_num"][b]) == n
        # the library numbers voxels exactly like the oracle (first point order) ...
        np.testing.assert_array_equal(r["coors"][b], coors)
        np.testing.assert_array_equal(r["num_points"][b], npv)
        # ... and sums the kept points in the same order, so fp32 features agree to the bit; the stated
        # tolerance of this path is 1e-5 relative
        np.testing.assert_allclose(r["voxels"][b], vox, rtol=1e-5, atol=0)
        np.testing.assert_array_equal(r["voxels"][b], vox)
        # canonical comparison (what the parity contract asks for): sort both by linear key
        og, kg = canonical_voxels(r["coors"][b], n, grid)
        oo, ko = canonical_voxels(coors, n, grid)
        np.testing.assert_array_equal(kg, ko)
        np.testing.assert_array_equal(r["num_points"][b][og], npv[oo])
        assert not r["voxels"][b][n:].any() and not r["coors"][b][n:].any()


def test_single_frame_20k_points(gpu, oracle):
    _compare(gpu, oracle, [gpu.synth.single_frame()], 20000)


def test_batch_of_ragged_frames(gpu, oracle):
    f = [gpu.synth.lidar_frame(100 + i, n_points=n, n_boxes=5) for i, n in enumerate([5000, 1, 12000, 300])]
    f.insert(2, np.zeros((0, 4), np.float32))   # an empty frame in the middle of the batch
    _compare(gpu, oracle, f, 16384)


def test_dense_sweep_frame_120k_points(gpu, oracle):
    _compare(gpu, oracle, [gpu.synth.sweep_frame(0)], 100000)


def test_points_outside_range_and_on_the_boundaries(gpu, oracle):
    rng, vs = (0.0, -2.0, -1.0, 4.0, 2.0, 1.0), (0.5, 0.5, 0.25)
    pts = np.array([[0, -2, -1, 1], [4, 0, 0, 1], [3.9999998, 1.9999999, 0.99999994, 1], [-1e-7, 0, 0, 1],
                    [2, 2, 0, 1], [2, 0, 1, 1], [np.nan, 0, 0, 1], [0.5, -1.5, -0.75, 1], [0.49999997, 0, 0, 1]],
                   np.float32)
    _compare(gpu, oracle, [pts], 64, rng, vs)


def test_more_than_five_points_in_a_voxel_keeps_lowest_indices(gpu, oracle):
    rs = np.random.RandomState(3)
    pts = np.concatenate([rs.uniform(0, 0.05, (200, 4)), rs.uniform(0, 0.5, (500, 4))]).astype(np.float32)
    pts[:, 1] -= 40.0
    pts[:, 2] -= 3.0
    pts = pts[rs.permutation(len(pts))]
    _compare(gpu, oracle, [pts], 4096)
    _compare(gpu, oracle, [pts], 4096, max_pts=3)
    _compare(gpu, oracle, [pts], 4096, max_pts=8)


def test_overflow_keeps_first_max_voxels_and_sets_status(gpu, oracle):
    f = gpu.synth.lidar_frame(7, n_points=4000, n_boxes=3)
    _compare(gpu, oracle, [f], 1000, expect_status=gpu.STATUS_VOXEL_OVERFLOW)


def test_fp16_output_is_the_rounded_fp32_mean(gpu, oracle):
    f = gpu.synth.lidar_frame(11, n_points=3000, n_boxes=3)
    r32, _ = _run(gpu, [f], 4096, out_dtype=gpu.F32)
    r16, _ = _run(gpu, [f], 4096, out_dtype=gpu.F16)
    np.testing.assert_array_equal(r16["voxels"], r32["voxels"].astype(np.float16))
    np.testing.assert_array_equal(r16["coors"], r32["coors"])


def test_repeat_runs_are_bitwise_identical(gpu):
    f = [gpu.synth.sweep_frame(1, n_points=40000)]
    a, _ = _run(gpu, f, 65536)
    b, _ = _run(gpu, f, 65536)
    for k in ("voxels", "coors", "voxel_num", "num_points"):
        np.testing.assert_array_equal(a[k], b[k])
