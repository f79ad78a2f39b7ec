"""CPU tests of the C/C++ side of the boundary: the constants header and the TensorRT shim gate."""
import json
import os
import shutil
import subprocess
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INCLUDE = os.path.join(ROOT, "include")

_DUMP = r'''
#include <cstdio>
#include "sessd_params.h"
int main() {
    std::printf("{\"layers\": [");
    for (int l = 0; l < SESSD_NUM_LAYERS; ++l) {
        const sessd_conv_params& p = sessd_layer_schedule[l];
        std::printf("%s{\"module\": %d, \"subm\": %d, \"cin\": %d, \"cout\": %d, \"max_voxels\": %d, "
                    "\"k\": [%d, %d, %d], \"s\": [%d, %d, %d], \"p\": [%d, %d, %d], "
                    "\"out\": [%d, %d, %d], \"in\": [%d, %d, %d], \"dilation\": %d}",
                    l ? ", " : "", sessd_layer_module_index[l], p.subm, p.in_channel, p.out_channel, p.max_voxels,
                    p.ksize[0], p.ksize[1], p.ksize[2], p.stride[0], p.stride[1], p.stride[2],
                    p.padding[0], p.padding[1], p.padding[2], p.out_shape_z, p.out_shape_y, p.out_shape_x,
                    p.spatial_shape_z, p.spatial_shape_y, p.spatial_shape_x, p.dilation);
    }
    std::printf("], \"names\": {\"SUBM_0_IN_CHANNEL\": %d, \"SPARSE_27_PADDING_0\": %d, \"SPARSE_39_KSIZE_1\": %d, "
                "\"SUBM_36_OUT_SHAPE_Z\": %d, \"MAX_VOXELS\": %d, \"MAX_BOX_NUM\": %d}, "
                "\"floats\": [%.9g, %.9g, %.9g, %.9g, %.9g, %.9g], \"bev\": [%d, %d, %d, %d], \"pad\": [%d, %d, %d, %d]}\n",
                (int)SUBM_0_IN_CHANNEL, (int)SPARSE_27_PADDING_0, (int)SPARSE_39_KSIZE_1, (int)SUBM_36_OUT_SHAPE_Z,
                MAX_VOXELS, MAX_BOX_NUM, (double)VOXEL_SIZE_X, (double)VOXEL_SIZE_Z, (double)X_MAX, (double)Y_MIN,
                (double)SCORE_THRESHOLD, (double)NMS_THRESH, sessd_default_s2d_params.feature_map_size_x,
                sessd_default_s2d_params.feature_map_size_y, sessd_default_s2d_params.feature_map_size_z,
                sessd_default_s2d_params.feature_map_channel, sessd_default_pad2d_params.top,
                sessd_default_pad2d_params.bottom, sessd_default_pad2d_params.left, sessd_default_pad2d_params.right);
    return 0;
}
'''


@pytest.mark.skipif(shutil.which("g++") is None, reason="no host C++ compiler")
def test_constants_header_compiles_and_matches_the_python_schedule(pkg):
    """A C++ host builds its 14 sessd_conv_params from include/sessd_params.h; the table must be the schedule the
    Python side (and the tests) use, and the reference's macro names must resolve to the reference's values."""
    S = pkg.schedule
    with tempfile.TemporaryDirectory() as tmp:
        src, exe = os.path.join(tmp, "dump.cpp"), os.path.join(tmp, "dump")
        with open(src, "w") as f:
            f.write(_DUMP)
        subprocess.check_call(["g++", "-std=c++17", "-Wall", "-Werror", "-Wno-unused-variable", "-I", INCLUDE, src, "-o", exe])
        got = json.loads(subprocess.check_output([exe]).decode())
        # and as plain C
        csrc = os.path.join(tmp, "c.c")
        with open(csrc, "w") as f:
            f.write('#include "sessd_params.h"\nint main(void) { return sessd_layer_schedule[13].ksize[0] == 3 ? 0 : 1; }\n')
        subprocess.check_call(["gcc", "-std=c11", "-Wall", "-Wno-unused-variable", "-I", INCLUDE, csrc, "-o", os.path.join(tmp, "c")])
        subprocess.check_call([os.path.join(tmp, "c")])
    assert len(got["layers"]) == len(S.LAYERS) == 14
    for l, g in zip(S.LAYERS, got["layers"]):
        assert g["module"] == int(l.name.lstrip("submparse"))
        assert (bool(g["subm"]), g["cin"], g["cout"]) == (l.subm, l.cin, l.cout)
        assert tuple(g["k"]) == l.ksize and tuple(g["s"]) == l.stride and tuple(g["p"]) == l.padding
        assert tuple(g["out"]) == l.out_shape and tuple(g["in"]) == l.in_shape
        assert g["max_voxels"] == S.MAX_VOXELS and g["dilation"] == 1
    assert got["names"] == {"SUBM_0_IN_CHANNEL": 4, "SPARSE_27_PADDING_0": 0, "SPARSE_39_KSIZE_1": 1,
                            "SUBM_36_OUT_SHAPE_Z": 5, "MAX_VOXELS": 60000, "MAX_BOX_NUM": 500}
    assert got["floats"] == [0.05, 0.1, 70.4, -40.0, 0.45, 0.01]
    assert got["bev"] == [176, 200, 2, 64] and got["pad"] == [1, 1, 1, 1]


def test_tensorrt_shim_is_gated_on_the_tensorrt_headers(pkg):
    """csrc/trt_shim.cpp holds the IPluginV2DynamicExt classes and the REGISTER_TENSORRT_PLUGIN lines; it compiles
    to nothing unless NvInferPlugin.h is found. The library says which way it was built, and exports everything
    either way."""
    import ctypes as C

    build = __import__("sys").modules["se_ssd_ai_trt_b200.build"]
    lib = C.CDLL(pkg.LIB_PATH) if hasattr(pkg, "LIB_PATH") else None
    if lib is None or not os.path.exists(pkg.LIB_PATH):
        pytest.skip("library not built")
    present = lib.sessd_tensorrt_shim_present()
    assert present == (1 if build.tensorrt_include_dir() else 0)
    shim = os.path.join(ROOT, "se-ssd-ai-trt_b200", "csrc", "trt_shim.cpp")
    text = open(shim).read()
    assert text.count("REGISTER_TENSORRT_PLUGIN(") == 7 and "IPluginV2DynamicExt" in text
    if not build.tensorrt_include_dir() and shutil.which("g++"):
        # without TensorRT the file must still be a valid (empty) translation unit
        subprocess.check_call(["g++", "-std=c++17", "-fsyntax-only", "-I", INCLUDE,
                               "-I", os.path.join(ROOT, "se-ssd-ai-trt_b200", "csrc"), shim])
    for name in pkg.EXPORTS:
        assert hasattr(lib, name), name
