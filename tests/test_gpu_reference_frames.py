"""GPU known-answer tests on the lidar frames the reference ships (data/kitti_training_velodyne_reduced).

The frames are not part of this repository. The tests look for them under SESSD_KITTI_DIR or, failing that, in a
reference checkout beside the repository (SESSD_REFERENCE_ROOT), and are skipped when neither is there.
"""
import os

import numpy as np
import pytest

from test_gpu_backbone import _check_fp16_layers, _gpu_run, _oracle_layers

pytestmark = pytest.mark.gpu

_HERE = os.path.dirname(os.path.abspath(__file__))
_REFERENCE = os.environ.get("SESSD_REFERENCE_ROOT", os.path.join(_HERE, "..", "..", "reference"))
KITTI_DIR = os.environ.get("SESSD_KITTI_DIR", os.path.join(_REFERENCE, "data", "kitti_training_velodyne_reduced"))


def _frame(name):
    path = os.path.join(KITTI_DIR, name)
    if not os.path.exists(path):
        pytest.skip(f"reference lidar frame {name} not reachable")
    return np.fromfile(path, dtype=np.float32).reshape(-1, 4)


def test_first_reference_frame_gives_16825_voxels_on_the_gpu(gpu, oracle):
    """16825 is the one known answer the reference tree holds (comments at submConv3dlayer.cu:254 and :618, for its
    first frame with MAX_VOXELS 60000): the CUDA voxeliser must reproduce it, and agree with the oracle row for row."""
    import torch

    pts = _frame("000000.bin")
    params = gpu.voxel_params(60000)
    r = gpu.voxelize(torch.from_numpy(pts[None]).cuda(), torch.tensor([len(pts)], dtype=torch.int32, device="cuda"), params)
    assert r["status"] == 0
    n = int(r["voxel_num"][0])
    assert n == 16825
    ov, oc, _, on, st = oracle.voxelize(pts, gpu.synth.POINT_RANGE, gpu.synth.VOXEL_SIZE, 60000)
    assert (on, st) == (16825, 0)
    np.testing.assert_array_equal(r["coors"][0, :n].cpu().numpy(), oc[:n])
    np.testing.assert_allclose(r["voxels"][0, :n].cpu().numpy(), ov[:n], rtol=1e-5, atol=0)


@pytest.mark.parametrize("name", ["000001.bin", "000002.bin"])
def test_reference_frames_through_the_whole_front_end(gpu, oracle, name):
    """Two more of the reference's frames through voxeliser, 14 layers and BEV scatter in fp16 at the reference's own
    capacities (MAX_VOXELS 60000), every layer against the oracle."""
    S = gpu.synth
    w, sc, sh = gpu.random_weights()
    case = dict(points=_frame(name), range=S.POINT_RANGE, voxel=S.VOXEL_SIZE, max_voxels=60000,
                layers=gpu.schedule.LAYERS, weights=w, scale=sc, shift=sh, bev=(64, 2, 200, 176))
    want = _oracle_layers(oracle, case, fp16=True)
    dense, views = _gpu_run(gpu, case, 1)
    _check_fp16_layers(oracle, case, want, views)
    c, n, f = want[-1]
    gf, gc, gn = views[-1]
    np.testing.assert_array_equal(dense, oracle.sparse2dense(gf[0, :n], gc[0, :n], n, 64, 2, 200, 176))
