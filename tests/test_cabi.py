"""CPU checks of the C ABI: the library loads, exports what include/sessd.h declares, and validates
its arguments on the host (no kernel is launched here)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "sessd.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sessd_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib(pkg):
    pkg.build()
    return pkg.lib()


def test_library_exports_every_declared_symbol(lib, pkg):
    names = _declared()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(pkg.EXPORTS) == names
    assert b"sm_100a" in lib.sessd_version()


def test_struct_sizes_match_the_serialized_blobs(pkg):
    # VoxelGeneratorPlugin serializes 16 four-byte fields (voxelGenerator.cu:576-600), Sparse2Dense 4
    assert C.sizeof(pkg.VoxelParams) == 64
    assert C.sizeof(pkg.S2DParams) == 16
    assert C.sizeof(pkg.ConvParams) == 22 * 4


def test_voxel_configure_rounds_like_the_reference(pkg, lib):
    p = pkg.voxel_params(20000)
    assert (p.grid_x, p.grid_y, p.grid_z) == (1408, 1600, 40)
    bad = pkg.VoxelParams(100, 5, 4, 0, 1, 0, 1, 0, 1, 0.0, 1, 1, 4, 0, 0, 0)
    assert lib.sessd_voxel_configure(C.byref(bad)) == -2
    assert lib.sessd_voxel_configure(None) == -1


def test_workspace_sizes_and_argument_validation(pkg, lib):
    p = pkg.voxel_params(20000)
    n1 = lib.sessd_voxelize_workspace_bytes(C.byref(p), 1, 20000)
    n4 = lib.sessd_voxelize_workspace_bytes(C.byref(p), 4, 20000)
    assert 0 < n1 < n4 < 64 << 20 and n1 % 256 == 0
    assert lib.sessd_voxelize_workspace_bytes(C.byref(p), 0, 20000) == 0
    assert lib.sessd_voxelize_workspace_bytes(C.byref(p), 1, 0) == 0
    p9 = pkg.voxel_params(20000, max_points_per_voxel=9)
    assert lib.sessd_voxelize_workspace_bytes(C.byref(p9), 1, 20000) == 0
    null2, null3 = (C.c_void_p * 2)(), (C.c_void_p * 3)()
    assert lib.sessd_voxelize_enqueue(C.byref(p), 1, 20000, 0, null2, null3, None, C.c_size_t(0), None) == -1
    assert lib.sessd_voxelize_enqueue(None, 1, 20000, 0, null2, null3, None, C.c_size_t(0), None) == -1

    layer = pkg.schedule.LAYERS[2]
    cp = pkg.conv_params(layer, 60000)
    assert lib.sessd_conv_workspace_bytes(C.byref(cp), 1) > 27 * 60000 * 4
    cp.stride[0] = 7
    assert lib.sessd_conv_workspace_bytes(C.byref(cp), 1) == 0
    cp = pkg.conv_params(layer, 60000)
    cp.dilation = 2
    assert lib.sessd_conv_workspace_bytes(C.byref(cp), 1) == 0
    assert lib.sessd_conv_weights_create(C.byref(cp), None, None, None, 0, 0, None) == -1
    assert lib.sessd_read_status(None, None) == -1
    assert lib.sessd_sparse2dense_enqueue(None, 1, 10, 0, null3, null3, None, C.c_size_t(0), None) == -1
    assert lib.sessd_backbone_workspace_bytes(None, 1, 10) == 0
    assert lib.sessd_backbone_enqueue(None, 1, 10, None, None, None, None, C.c_size_t(0), None) == -1
    assert lib.sessd_pipeline_create(None, 1, 10, 1, None) == -1


def test_compute_calls_fail_loudly_without_a_gpu(pkg):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(pkg.SessdError):
        pkg.Backbone(1000, [])
