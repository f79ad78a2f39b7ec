"""GPU test of sessd_voxelize_enqueue_static, the voxeliser entry point that allocates nothing.

Hosts whose device memory is fixed before the library runs (a pre-sized plugin arena, a real-time loop
that must stay away from the allocator) cannot provide a workspace; this entry point keeps its scratch
in a device array inside the library. The test calls it through the C ABI twice in a row, with different
inputs, and requires outputs identical to those of the regular entry point and to those of the CPU oracle
(the array keeps the first call's contents, so the second call proves that everything that must start
clean is reset). The file is named so that pytest collects it last.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _call_static(gpu, params, pts, sizes, out_dtype=0):
    import torch

    B, P, V = pts.shape[0], pts.shape[1], params.max_voxels
    tdt = torch.float32 if out_dtype == 0 else torch.float16
    voxels = torch.full((B, V, 4), 7, dtype=tdt, device="cuda")
    coors = torch.full((B, V, 4), 7, dtype=torch.int32, device="cuda")
    num = torch.full((B,), 7, dtype=torch.int32, device="cuda")
    ins = (C.c_void_p * 2)(pts.data_ptr(), sizes.data_ptr())
    outs = (C.c_void_p * 3)(voxels.data_ptr(), coors.data_ptr(), num.data_ptr())
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = gpu.lib().sessd_voxelize_enqueue_static(C.byref(params), B, P, out_dtype, ins, outs, stream)
    torch.cuda.synchronize()
    return rc, voxels.cpu().numpy(), coors.cpu().numpy(), num.cpu().numpy()


def test_static_scratch_voxeliser_matches_regular_entry_point_twice(gpu, oracle):
    import torch

    params = gpu.voxel_params(20000)
    frames = [gpu.synth.single_frame(), gpu.synth.lidar_frame(4242, n_points=20000, n_boxes=9)]
    for f in frames:                       # two calls in a row on the shared array
        pts = torch.from_numpy(f[None]).cuda()
        sizes = torch.tensor([len(f)], dtype=torch.int32, device="cuda")
        rc, voxels, coors, num = _call_static(gpu, params, pts, sizes)
        assert rc == 0
        ref = gpu.voxelize(pts, sizes, params)
        assert ref["status"] == 0
        # integer outputs bit-exact; features within the 1e-5 relative tolerance of the voxeliser tests
        # (same kernels, same order of additions, so they are in fact identical)
        np.testing.assert_array_equal(num, ref["voxel_num"].cpu().numpy())
        np.testing.assert_array_equal(coors, ref["coors"].cpu().numpy())
        np.testing.assert_allclose(voxels, ref["voxels"].cpu().numpy(), rtol=1e-5, atol=0)
        assert int(num[0]) > 10000
        # and directly against the CPU oracle (voxelGenerator.cu:348-451, :255-321 restated): same rows in the
        # same order, same means
        ovox, ocoors, _, on, ost = oracle.voxelize(f, gpu.synth.POINT_RANGE, gpu.synth.VOXEL_SIZE, params.max_voxels)
        assert ost == 0 and int(num[0]) == on
        np.testing.assert_array_equal(coors[0, :on], ocoors[:on])
        np.testing.assert_allclose(voxels[0, :on], ovox[:on], rtol=1e-5, atol=0)
        assert not coors[0, on:].any() and not voxels[0, on:].any()


def test_static_scratch_rejects_requests_beyond_its_size(gpu):
    import torch

    big = gpu.voxel_params(200000)
    pts = torch.zeros((1, 120000, 4), dtype=torch.float32, device="cuda")
    sizes = torch.zeros((1,), dtype=torch.int32, device="cuda")
    rc, *_ = _call_static(gpu, big, pts, sizes)
    assert rc == -3
    assert b"built-in scratch" in gpu.lib().sessd_last_cuda_error()


def test_static_scratch_reports_lost_voxels_through_its_status_reader(gpu):
    """A frame with more voxels than max_voxels ends with voxel_num == max_voxels, exactly like a frame that fits
    exactly; the status word inside the built-in array tells the two apart."""
    import torch

    f = gpu.synth.single_frame()
    pts = torch.from_numpy(f[None]).cuda()
    sizes = torch.tensor([len(f)], dtype=torch.int32, device="cuda")
    small = gpu.voxel_params(4000)
    rc, voxels, coors, num = _call_static(gpu, small, pts, sizes)
    assert rc == 0 and int(num[0]) == 4000
    st = gpu.lib().sessd_voxelize_static_status(None)
    assert st >= 0 and st & gpu.STATUS_VOXEL_OVERFLOW
    rc, voxels, coors, num = _call_static(gpu, gpu.voxel_params(20000), pts, sizes)
    assert rc == 0 and gpu.lib().sessd_voxelize_static_status(None) == 0
