"""Plugin layer: the reference's creator fields, tensor shapes, format rules and serialised byte layouts
(CPU), and a frame pushed through the four plugins the way the reference's network wires them (GPU)."""
import struct

import numpy as np
import pytest

from conftest import match_rows, canonical_rulebook  # noqa: F401  (shared helpers live in conftest)


def _voxel_fields(max_voxels=20000):
    return {"max_num_points_per_voxel": np.array([5], np.int32), "max_voxels": np.array([max_voxels], np.int32),
            "point_cloud_range": np.array([0.0, -40.0, -3.0, 70.4, 40.0, 1.0], np.float32),
            "voxel_feature_num": np.array([4], np.int32), "voxel_size": np.array([0.05, 0.05, 0.1], np.float32)}


def _subm_fields(layer, max_voxels, w):
    z, y, x = layer.out_shape
    return {"in_channel": np.array([layer.cin], np.int32), "out_channel": np.array([layer.cout], np.int32),
            "max_voxels": np.array([max_voxels], np.int32), "feature_num": np.array([layer.cin], np.int32),
            "out_shape": np.array([x, y, z], np.int32), "spatial_shape": np.array([x, y, z], np.int32),
            "ksize": np.array([3], np.int32), "stride": np.array([1], np.int32), "padding": np.array([1], np.int32),
            "dilation": np.array([1], np.int32), "out_padding": np.array([0], np.int32),
            "weights": np.ascontiguousarray(w, np.float32)}


def _sparse_fields(layer, max_voxels, w):
    z, y, x = layer.out_shape
    sz, sy, sx = layer.in_shape
    return {"in_channel": np.array([layer.cin], np.int32), "out_channel": np.array([layer.cout], np.int32),
            "max_voxels": np.array([max_voxels], np.int32), "feature_num": np.array([layer.cin], np.int32),
            "out_shape": np.array([x, y, z], np.int32), "spatial_shape": np.array([sx, sy, sz], np.int32),
            "ksize": np.array(layer.ksize, np.int32), "stride": np.array(layer.stride, np.int32),
            "padding": np.array(layer.padding, np.int32), "dilation": np.array([1], np.int32),
            "out_padding": np.array([0], np.int32), "weights": np.ascontiguousarray(w, np.float32)}


def test_creators_advertise_the_reference_field_names(pkg):
    P = pkg.plugins
    pkg.build()
    assert P.field_names("VoxelGeneratorPlugin") == ["max_num_points_per_voxel", "max_voxels", "point_cloud_range",
                                                     "voxel_feature_num", "voxel_size"]
    conv = ["in_channel", "out_channel", "max_voxels", "feature_num", "out_shape", "spatial_shape", "ksize", "stride",
            "padding", "dilation", "out_padding", "weights"]
    assert P.field_names("SubmConv3dLayerPlugin") == conv and P.field_names("SparseConv3dLayerPlugin") == conv
    assert P.field_names("Sparse2DensePlugin") == ["feature_map_size", "feature_map_channel"]
    assert P.field_names("ZeroPad2dPlugin") == ["zero_padding_2d_size"]
    assert P.field_names("GenerateAnchorDecodePlugin") == ["point_cloud_range", "feature_map_size", "car_size",
                                                           "direction_angle", "direction_angle_num"]
    assert P.field_names("FilterBoxByScorePlugin") == ["feature_map_size", "direction_angle_num", "max_box_num",
                                                       "score_threshold", "direction_offset"]
    assert P.field_names("NoSuchPlugin") is None
    lib = pkg.lib()
    for n in P.PLUGIN_EXPORTS:
        assert hasattr(lib, n)


def test_voxel_generator_blob_is_the_reference_layout(pkg):
    P = pkg.plugins
    v = P.Plugin.create("VoxelGeneratorPlugin", _voxel_fields())
    assert v.type() == "VoxelGeneratorPlugin" and v.version() == "1" and v.nb_outputs() == 3
    pts, size = P.TensorDesc.of((1, 80000, 4), P.DT_FLOAT), P.TensorDesc.of((1,), P.DT_INT32)
    assert [v.output_dims(i, [pts, size]).dims() for i in range(3)] == [(1, 20000, 4), (1, 20000, 4), (1,)]
    v.configure([pts, size], [])
    blob = v.serialize()
    # int maxV, int ptsPerVoxel, int feat, 6 x float range (xmin,xmax,ymin,ymax,zmin,zmax), 3 x float voxel,
    # int pointFeat, int gx, gy, gz  (voxelGenerator.cu:576-600)
    want = struct.pack("<3i9f4i", 20000, 5, 4, 0.0, 70.4, -40.0, 40.0, -3.0, 1.0, 0.05, 0.05, 0.1, 4, 1408, 1600, 40)
    assert blob == want and len(blob) == 64
    again = P.Plugin.deserialize("VoxelGeneratorPlugin", blob)
    assert again.serialize() == blob and again.clone().serialize() == blob
    outs = [P.TensorDesc.of((1, 20000, 4), P.DT_FLOAT), P.TensorDesc.of((1, 20000, 4), P.DT_INT32),
            P.TensorDesc.of((1,), P.DT_INT32)]
    assert all(v.supports_format(i, [pts, size] + outs, 2) for i in range(5))
    assert not v.supports_format(0, [P.TensorDesc.of((1, 80000, 4), P.DT_HALF), size] + outs, 2)
    assert v.workspace_size([pts, size], outs) == pkg.lib().sessd_voxelize_workspace_bytes(
        __import__("ctypes").byref(pkg.voxel_params(20000)), 1, 80000)


def test_conv_plugin_blobs_are_the_reference_layout(pkg):
    P = pkg.plugins
    rs = np.random.RandomState(0)
    l3, l6 = pkg.schedule.LAYERS[1], pkg.schedule.LAYERS[2]
    w3 = rs.randn(27, 16, 16).astype(np.float32)
    s = P.Plugin.create("SubmConv3dLayerPlugin", _subm_fields(l3, 60000, w3))
    blob = s.serialize()
    head = struct.pack("<16i", 16, 16, 60000, 16, 1408, 1600, 41, 1408, 1600, 41, 3, 1, 1, 1, 0, 27 * 16 * 16)
    assert blob == head + w3.tobytes()          # submConv3dlayer.cu:684-714
    assert P.Plugin.deserialize("SubmConv3dLayerPlugin", blob).serialize() == blob and s.clone().serialize() == blob
    feat = P.TensorDesc.of((1, 60000, 16), P.DT_FLOAT)
    assert s.nb_outputs() == 1 and s.output_dims(0, [feat]).dims() == (1, 60000, 16) and s.output_dims(1, [feat]) is None
    w6 = rs.randn(27, 16, 32).astype(np.float32)
    c = P.Plugin.create("SparseConv3dLayerPlugin", _sparse_fields(l6, 60000, w6))
    blob = c.serialize()
    head = struct.pack("<22i", 16, 32, 60000, 16, 704, 800, 21, 1408, 1600, 41, 3, 3, 3, 2, 2, 2, 1, 1, 1, 1, 0,
                       27 * 16 * 32)
    assert blob == head + w6.tobytes()          # sparseConv3dlayer.cu:863-899
    assert P.Plugin.deserialize("SparseConv3dLayerPlugin", blob).serialize() == blob
    assert c.nb_outputs() == 3
    assert [c.output_dims(i, [feat]).dims() for i in range(3)] == [(1, 60000, 32), (1, 60000, 4), (1,)]
    with pytest.raises(ValueError):
        P.Plugin.deserialize("SparseConv3dLayerPlugin", blob[:40])
    with pytest.raises(ValueError):
        P.Plugin.create("SubmConv3dLayerPlugin", {"in_channel": np.array([16], np.int32)})
    half = P.TensorDesc.of((1, 60000, 16), P.DT_HALF)
    coors, num = P.TensorDesc.of((1, 60000, 4), P.DT_INT32), P.TensorDesc.of((1,), P.DT_INT32)
    assert s.supports_format(3, [half, coors, num, P.TensorDesc.of((1, 60000, 16), P.DT_HALF)], 3)
    assert not s.supports_format(3, [half, coors, num, P.TensorDesc.of((1, 60000, 16), P.DT_FLOAT)], 3)
    assert s.workspace_size([feat, coors, num], []) > 27 * 60000 * 4


def test_sparse2dense_blob_and_dims(pkg):
    P = pkg.plugins
    d = P.Plugin.create("Sparse2DensePlugin", {"feature_map_size": np.array([176, 200, 2], np.int32),
                                              "feature_map_channel": np.array([64], np.int32)})
    assert d.serialize() == struct.pack("<4i", 176, 200, 2, 64)     # sparse2Dense.cu:283-295
    feat = P.TensorDesc.of((1, 60000, 64), P.DT_FLOAT)
    assert d.output_dims(0, [feat]).dims() == (1, 128, 200, 176)
    assert d.workspace_size([feat], []) == 0
    assert P.Plugin.deserialize("Sparse2DensePlugin", d.serialize()).type() == "Sparse2DensePlugin"


def test_zero_pad2d_blob_and_dims(pkg):
    P = pkg.plugins
    z = P.Plugin.create("ZeroPad2dPlugin", {"zero_padding_2d_size": np.array([1, 1, 1, 1], np.int32)})
    assert z.serialize() == struct.pack("<4i", 1, 1, 1, 1)          # zeroPad2d.cu:286-289
    m = P.TensorDesc.of((1, 128, 200, 176), P.DT_FLOAT)
    assert z.output_dims(0, [m]).dims() == (1, 128, 202, 178) and z.nb_outputs() == 1
    assert z.workspace_size([m], []) == 0
    assert P.Plugin.deserialize("ZeroPad2dPlugin", struct.pack("<4i", 2, 0, 1, 3)).output_dims(0, [m]).dims() == (1, 128, 202, 180)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [0, 1])
def test_zero_pad2d_plugin_and_fused_padded_scatter(gpu, oracle, dt):
    """ZeroPad2dPlugin on its own, and Sparse2Dense + ZeroPad2d fused into one pass, against the oracle."""
    import torch

    P = gpu.plugins
    rs = np.random.RandomState(8)
    tdt = torch.float32 if dt == 0 else torch.float16
    B, Cc, H, W = 2, 6, 9, 11
    x = rs.randn(B, Cc, H, W).astype(np.float32)
    if dt:
        x = x.astype(np.float16).astype(np.float32)
    for pad in [(1, 1, 1, 1), (0, 2, 3, 0)]:
        z = P.Plugin.create("ZeroPad2dPlugin", {"zero_padding_2d_size": np.array(pad, np.int32)})
        d_in = P.TensorDesc.of((B, Cc, H, W), P.DT_FLOAT if dt == 0 else P.DT_HALF)
        d_out = z.output_dims(0, [d_in])
        tin = torch.from_numpy(x).cuda().to(tdt)
        tout = torch.full(d_out.dims(), 5, dtype=tdt, device="cuda")
        assert z.enqueue([d_in], [d_out], [tin], [tout], None, torch.cuda.current_stream().cuda_stream) == 0
        torch.cuda.synchronize()
        np.testing.assert_array_equal(tout.float().cpu().numpy(), oracle.zero_pad2d(x, *pad))
    # fused: rows -> padded BEV map directly
    V, C2, D, H2, W2 = 256, 8, 2, 10, 12
    feat = np.zeros((B, V, C2), np.float32)
    coors = np.zeros((B, V, 4), np.int32)
    num = np.array([100, 37], np.int32)
    for b in range(B):
        cells = rs.permutation(D * H2 * W2)[:num[b]]
        coors[b, :num[b], 0] = b
        coors[b, :num[b], 1], coors[b, :num[b], 2], coors[b, :num[b], 3] = cells // (H2 * W2), (cells // W2) % H2, cells % W2
        feat[b, :num[b]] = rs.randn(num[b], C2)
    if dt:
        feat = feat.astype(np.float16).astype(np.float32)
    pad = gpu.Pad2DParams(1, 1, 1, 1)
    dense = gpu.sparse2dense(torch.from_numpy(feat).cuda().to(tdt), torch.from_numpy(coors).cuda(),
                             torch.from_numpy(num).cuda(), gpu.S2DParams(W2, H2, D, C2), dt, pad=pad)
    want = np.stack([oracle.sparse2dense(feat[b, :num[b]], np.concatenate([np.zeros((num[b], 1), np.int32), coors[b, :num[b], 1:]], 1),
                                         num[b], C2, D, H2, W2)[0] for b in range(B)])
    np.testing.assert_array_equal(dense.float().cpu().numpy(), oracle.zero_pad2d(want, 1, 1, 1, 1))


@pytest.mark.gpu
def test_backbone_with_folded_zero_padding(gpu, oracle):
    """sessd_backbone_set_padding: the fused front end writes the padded map the reference's ZeroPad2d layer produces."""
    import torch

    import make_golden_inputs as mk

    case = mk.small_case(gpu)
    pts = torch.from_numpy(case["points"][None]).cuda()
    sizes = torch.tensor([pts.shape[1]], dtype=torch.int32, device="cuda")
    outs = []
    for padded in (False, True):
        bb = gpu.Backbone(case["max_voxels"], case["weights"], case["scale"], case["shift"], dtype=gpu.F16,
                          layers=case["layers"], point_range=case["range"], voxel_size=case["voxel"])
        if padded:
            bb.set_padding(1, 1, 1, 1)
        dense, ws = bb.run(pts, sizes)
        torch.cuda.synchronize()
        assert gpu.read_status(ws) == 0
        outs.append(dense.float().cpu().numpy())
        bb.close()
    assert outs[1].shape == (1, 128, 12, 10)
    np.testing.assert_array_equal(outs[1], oracle.zero_pad2d(outs[0], 1, 1, 1, 1))


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [0, 1])
def test_frame_through_the_four_plugins_like_the_reference_network(gpu, oracle, dt):
    """voxel generator -> subm0 -> (host BN + ReLU, TensorRT's job in the reference) -> sparse6 -> sparse2dense on
    a small grid; every plugin is created from creator fields, cloned, serialised and deserialised first."""
    import torch

    import make_golden_inputs as mk

    P = gpu.plugins
    case = mk.small_case(gpu)
    maxV = case["max_voxels"]
    layers = case["layers"]
    pts_np = case["points"]
    tdt = torch.float32 if dt == 0 else torch.float16
    trt = P.DT_FLOAT if dt == 0 else P.DT_HALF
    stream = torch.cuda.current_stream().cuda_stream

    def roundtrip(p):
        q = P.Plugin.deserialize(p.type(), p.serialize()).clone()
        assert q.serialize() == p.serialize()
        return q

    fields = _voxel_fields(maxV)
    fields["point_cloud_range"] = np.array(case["range"], np.float32)
    vox = P.Plugin.create("VoxelGeneratorPlugin", fields)
    d_pts = P.TensorDesc.of((1, len(pts_np), 4), P.DT_FLOAT)
    d_size = P.TensorDesc.of((1,), P.DT_INT32)
    vox.configure([d_pts, d_size], [])
    vox = roundtrip(vox)
    pts = torch.from_numpy(pts_np[None]).cuda()
    size = torch.tensor([len(pts_np)], dtype=torch.int32, device="cuda")
    d_vox = P.TensorDesc.of((1, maxV, 4), trt)
    d_coors = P.TensorDesc.of((1, maxV, 4), P.DT_INT32)
    voxels = torch.empty((1, maxV, 4), dtype=tdt, device="cuda")
    coors = torch.empty((1, maxV, 4), dtype=torch.int32, device="cuda")
    num = torch.empty((1,), dtype=torch.int32, device="cuda")
    ws = torch.empty(vox.workspace_size([d_pts, d_size], []), dtype=torch.uint8, device="cuda")
    assert vox.enqueue([d_pts, d_size], [d_vox, d_coors, d_size], [pts, size], [voxels, coors, num], ws, stream) == 0

    l0, l6 = layers[0], layers[2]
    w0, w6 = case["weights"][0], gpu.synth.normal_f32(99, (27, 16, 32), 0.1)
    subm = roundtrip(P.Plugin.create("SubmConv3dLayerPlugin", _subm_fields(l0, maxV, w0)))
    d_f16 = P.TensorDesc.of((1, maxV, 16), trt)
    f0 = torch.empty((1, maxV, 16), dtype=tdt, device="cuda")
    ws = torch.empty(subm.workspace_size([d_vox, d_coors, d_size], []), dtype=torch.uint8, device="cuda")
    assert subm.enqueue([d_vox, d_coors, d_size], [d_f16], [voxels, coors, num], [f0], ws, stream) == 0
    f0 = torch.relu(f0.float() * 0.5 + 0.1).to(tdt)      # the scale + ReLU layers TensorRT runs between plugins

    l6s = gpu.schedule.ConvLayer("sparse6", False, 16, 32, l6.ksize, l6.stride, l6.padding, l6.in_shape, l6.out_shape)
    sp = roundtrip(P.Plugin.create("SparseConv3dLayerPlugin", _sparse_fields(l6s, maxV, w6)))
    d_f32 = P.TensorDesc.of((1, maxV, 32), trt)
    f6 = torch.empty((1, maxV, 32), dtype=tdt, device="cuda")
    coors6 = torch.empty((1, maxV, 4), dtype=torch.int32, device="cuda")
    num6 = torch.empty((1,), dtype=torch.int32, device="cuda")
    ws = torch.empty(sp.workspace_size([d_f16, d_coors, d_size], []), dtype=torch.uint8, device="cuda")
    assert sp.enqueue([d_f16, d_coors, d_size], [d_f32, d_coors, d_size], [f0, coors, num], [f6, coors6, num6], ws,
                      stream) == 0

    Z, Y, X = l6.out_shape
    s2d = roundtrip(P.Plugin.create("Sparse2DensePlugin", {"feature_map_size": np.array([X, Y, Z], np.int32),
                                                          "feature_map_channel": np.array([32], np.int32)}))
    d_dense = s2d.output_dims(0, [d_f32])
    dense = torch.empty(d_dense.dims(), dtype=tdt, device="cuda")
    assert s2d.enqueue([d_f32, d_coors, d_size], [d_dense], [f6, coors6, num6], [dense], None, stream) == 0
    torch.cuda.synchronize()

    # oracle, same wiring
    half = dt == 1
    ov, oc, onpv, on, st = oracle.voxelize(pts_np, case["range"], case["voxel"], maxV)
    assert int(num[0]) == on
    np.testing.assert_array_equal(coors[0].cpu().numpy(), oc)
    fin = ov[:on].astype(np.float16).astype(np.float32) if half else ov[:on]
    pairs, pnum, st = oracle.subm_rulebook(oc, on, l0.out_shape, maxV)
    y0 = oracle.conv_apply(fin, pairs, pnum, w0, on, half_inputs=half)
    if half:
        y0 = y0.astype(np.float16).astype(np.float32)
    y0 = torch.relu(torch.from_numpy(y0) * 0.5 + 0.1).to(tdt).float().numpy()
    c6, n6, pairs, pnum, st = oracle.spconv_rulebook(oc, on, l6.ksize, l6.stride, l6.padding, l6.out_shape, maxV)
    y6 = oracle.conv_apply(y0, pairs, pnum, w6, n6, half_inputs=half)
    if half:
        y6 = y6.astype(np.float16).astype(np.float32)
    assert int(num6[0]) == n6
    c6g = coors6[0].cpu().numpy()
    assert not c6g[n6:].any()
    perm = match_rows(c6g[:n6], c6[:n6])      # the plugin numbers its outputs in (z, y, x) order
    got6 = f6[0, :n6].float().cpu().numpy()[perm]
    tol = 1e-2 if half else 1e-5
    denom = np.maximum(np.abs(y6), np.abs(y6).max() * 1e-3)
    assert (np.abs(got6 - y6) / denom).max() <= tol
    want_dense = oracle.sparse2dense(got6, c6, n6, 32, Z, Y, X)
    np.testing.assert_array_equal(dense.float().cpu().numpy(), want_dense)


def _anchor_fields():
    return {"point_cloud_range": np.array([0.0, -40.0, -3.0, 70.4, 40.0, 1.0], np.float32),
            "feature_map_size": np.array([200, 176], np.int32), "car_size": np.array([3.9, 1.6, 1.56], np.float32),
            "direction_angle": np.array([0.0, 1.57], np.float32), "direction_angle_num": np.array([2], np.int32)}


def _filter_fields(max_box=500):
    return {"feature_map_size": np.array([200, 176], np.int32), "direction_angle_num": np.array([2], np.int32),
            "max_box_num": np.array([max_box], np.int32), "score_threshold": np.array([0.45], np.float32),
            "direction_offset": np.array([0.0], np.float32)}


def test_post_processing_blobs_and_dims(pkg):
    P = pkg.plugins
    a = P.Plugin.create("GenerateAnchorDecodePlugin", _anchor_fields())
    # 6 range floats, 2 ints, 5 floats, 1 int; the sixth float repeats max_y (generateAnchorDecode.cu:409)
    assert a.serialize() == struct.pack("<6f2i5fi", 0.0, 70.4, -40.0, 40.0, -3.0, 40.0, 200, 176, 3.9, 1.6, 1.56, 0.0, 1.57, 2)
    box = P.TensorDesc.of((1, 70400, 7), P.DT_FLOAT)
    assert a.nb_outputs() == 1 and a.output_dims(0, [box]).dims() == (1, 70400, 7) and a.workspace_size([box], []) == 0
    assert a.supports_format(0, [box, box], 1) and not a.supports_format(1, [box, P.TensorDesc.of((1, 70400, 7), P.DT_HALF)], 1)
    assert P.Plugin.deserialize("GenerateAnchorDecodePlugin", a.serialize()).serialize() == a.serialize()

    f = P.Plugin.create("FilterBoxByScorePlugin", _filter_fields())
    assert f.serialize() == struct.pack("<4i2f", 200, 176, 2, 500, 0.45, 0.0)     # filterBoxByScore.cu:430-441
    ins = [box, P.TensorDesc.of((1, 70400, 1), P.DT_FLOAT), P.TensorDesc.of((1, 70400, 1), P.DT_FLOAT),
           P.TensorDesc.of((1, 70400, 2), P.DT_FLOAT)]
    assert f.nb_outputs() == 5
    assert [f.output_dims(i, ins).dims() for i in range(5)] == [(1, 500, 9), (1, 500), (1, 500, 1), (1, 500, 1), (1, 1)]
    assert f.output_dtype(4, [P.DT_FLOAT] * 4) == P.DT_INT32 and f.output_dtype(0, [P.DT_FLOAT] * 4) == P.DT_FLOAT
    assert f.workspace_size(ins, []) >= 1024 + 4 * 275


@pytest.mark.gpu
def test_post_processing_plugins_chained(gpu, oracle):
    """GenerateAnchorDecodePlugin -> FilterBoxByScorePlugin, wired as at se-ssd-ai-trt.cpp:1421-1461."""
    import torch

    P, S = gpu.plugins, gpu.schedule
    rs = np.random.RandomState(12)
    n = 70400
    box = (rs.randn(1, n, 7) * 0.3).astype(np.float32)
    cls = (-4.0 + 1.5 * rs.randn(1, n, 1)).astype(np.float32)
    score = 1.0 / (1.0 + np.exp(-cls.astype(np.float64)))
    cls[np.abs(score - 0.45) < 1e-4] = -10.0
    iou = rs.uniform(-1, 1, (1, n, 1)).astype(np.float32)
    dr = rs.randn(1, n, 2).astype(np.float32)
    a = P.Plugin.create("GenerateAnchorDecodePlugin", _anchor_fields())
    f = P.Plugin.deserialize("FilterBoxByScorePlugin", struct.pack("<4i2f", 200, 176, 2, 500, 0.45, 0.0))
    stream = torch.cuda.current_stream().cuda_stream
    d_box = P.TensorDesc.of((1, n, 7), P.DT_FLOAT)
    t_box, t_cls, t_iou, t_dir = [torch.from_numpy(x).cuda() for x in (box, cls, iou, dr)]
    decoded = torch.empty_like(t_box)
    assert a.enqueue([d_box], [d_box], [t_box], [decoded], None, stream) == 0
    ins = [d_box, P.TensorDesc.of((1, n, 1), P.DT_FLOAT), P.TensorDesc.of((1, n, 1), P.DT_FLOAT),
           P.TensorDesc.of((1, n, 2), P.DT_FLOAT)]
    outs_d = [f.output_dims(i, ins) for i in range(5)]
    outs = [torch.full(d.dims(), 7, dtype=torch.int32 if i == 4 else torch.float32, device="cuda")
            for i, d in enumerate(outs_d)]
    ws = torch.empty(f.workspace_size(ins, outs_d), dtype=torch.uint8, device="cuda")
    assert f.enqueue(ins, outs_d, [decoded, t_cls, t_iou, t_dir], outs, ws, stream) == 0
    torch.cuda.synchronize()
    op = oracle.anchor_params(gpu.synth.POINT_RANGE, S.CAR_SIZE, S.DIRECTION_ANGLES)
    want_dec = oracle.anchor_decode(box[0], op, 200, 176, 2)
    ob, oc, oi, od, valid, passed = oracle.filter_boxes(want_dec, cls[0], iou[0], dr[0], 2, 500, 0.45, 0.0)
    assert int(outs[4][0, 0]) == valid and 0 < valid <= 500
    np.testing.assert_allclose(outs[0][0].cpu().numpy(), ob, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(outs[1][0].cpu().numpy(), oc, rtol=1e-5, atol=1e-6)
    np.testing.assert_array_equal(outs[3][0, :, 0].cpu().numpy(), od)
