"""B200 (sm_100a) sparse 3D front end for SE-SSD: Python view of the C ABI in include/sessd.h.

The product is libsessd.so (hand-written CUDA behind a C ABI that mirrors the reference's TensorRT
plugins). This module only binds it with ctypes and uses torch tensors as device buffers; there is no
CPU fallback: importing works without a GPU (so that the build can be checked), every compute call
needs the library and a CUDA device and raises otherwise.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import detector, formats, plugins, schedule, sharding, synth  # noqa: F401
from .build import LIB_PATH, build

F32, F16 = 0, 1
STATUS_VOXEL_OVERFLOW, STATUS_HASH_FULL, STATUS_PAIR_OVERFLOW, STATUS_BAD_COORD, STATUS_TIMEOUT = 1, 2, 4, 8, 16
STATUS_BOX_OVERFLOW = 32

EXPORTS = (
    "sessd_voxel_configure", "sessd_voxelize_workspace_bytes", "sessd_voxelize_enqueue", "sessd_voxelize_num_points",
    "sessd_voxelize_enqueue_static", "sessd_voxelize_static_status",
    "sessd_conv_weights_create", "sessd_conv_weights_destroy", "sessd_conv_workspace_bytes",
    "sessd_subm_conv_enqueue", "sessd_sparse_conv_enqueue", "sessd_conv_rulebook_export",
    "sessd_sparse2dense_enqueue", "sessd_sparse2dense_padded_enqueue", "sessd_zero_pad2d_enqueue",
    "sessd_backbone_set_padding", "sessd_backbone_create", "sessd_backbone_destroy",
    "sessd_backbone_workspace_bytes", "sessd_backbone_enqueue", "sessd_backbone_pair_counts",
    "sessd_backbone_layer_view",
    "sessd_backbone_final_level", "sessd_pipeline_create", "sessd_pipeline_destroy", "sessd_pipeline_run_host",
    "sessd_pipeline_run_device", "sessd_pipeline_run_host_bev", "sessd_pipeline_dense", "sessd_pipeline_workspace", "sessd_pipeline_use_graphs",
    "sessd_launch_count",
    "sessd_profile_begin", "sessd_profile_end", "sessd_read_status", "sessd_last_cuda_error", "sessd_version",
    "sessd_anchor_decode_enqueue", "sessd_filter_boxes_workspace_bytes", "sessd_filter_boxes_enqueue",
    "sessd_decode_filter_enqueue", "sessd_rotated_nms_workspace_bytes", "sessd_rotated_nms_enqueue",
    "sessd_wts_load", "sessd_wts_destroy", "sessd_wts_count", "sessd_wts_entry", "sessd_wts_find", "sessd_wts_save",
    "sessd_fold_batchnorm", "sessd_backbone_create_from_wts", "sessd_points_load", "sessd_conv_weights_debug_withhold",
)


class SessdError(RuntimeError):
    pass


class VoxelParams(C.Structure):
    _fields_ = [("max_voxels", C.c_int32), ("max_points_per_voxel", C.c_int32), ("voxel_feature_num", C.c_int32),
                ("x_min", C.c_float), ("x_max", C.c_float), ("y_min", C.c_float), ("y_max", C.c_float),
                ("z_min", C.c_float), ("z_max", C.c_float),
                ("voxel_x", C.c_float), ("voxel_y", C.c_float), ("voxel_z", C.c_float),
                ("point_feature_num", C.c_int32), ("grid_x", C.c_int32), ("grid_y", C.c_int32), ("grid_z", C.c_int32)]


class ConvParams(C.Structure):
    _fields_ = [("in_channel", C.c_int32), ("out_channel", C.c_int32), ("max_voxels", C.c_int32),
                ("feature_num", C.c_int32),
                ("out_shape_x", C.c_int32), ("out_shape_y", C.c_int32), ("out_shape_z", C.c_int32),
                ("spatial_shape_x", C.c_int32), ("spatial_shape_y", C.c_int32), ("spatial_shape_z", C.c_int32),
                ("ksize", C.c_int32 * 3), ("stride", C.c_int32 * 3), ("padding", C.c_int32 * 3),
                ("dilation", C.c_int32), ("out_padding", C.c_int32), ("subm", C.c_int32)]


class Pad2DParams(C.Structure):
    _fields_ = [("top", C.c_int32), ("bottom", C.c_int32), ("left", C.c_int32), ("right", C.c_int32)]


class AnchorParams(C.Structure):
    """GenerateAnchorDecodePlugin's parameters in its serialisation order (generateAnchorDecode.cu:400-421)."""
    _fields_ = [("min_x", C.c_float), ("max_x", C.c_float), ("min_y", C.c_float), ("max_y", C.c_float),
                ("min_z", C.c_float), ("max_z", C.c_float),
                ("feature_map_height", C.c_int32), ("feature_map_width", C.c_int32),
                ("car_length", C.c_float), ("car_width", C.c_float), ("car_height", C.c_float),
                ("direction_angle_0", C.c_float), ("direction_angle_1", C.c_float), ("direction_angle_num", C.c_int32)]


class FilterParams(C.Structure):
    """FilterBoxByScorePlugin's parameters in its serialisation order (filterBoxByScore.cu:430-441)."""
    _fields_ = [("feature_map_height", C.c_int32), ("feature_map_width", C.c_int32),
                ("direction_angle_num", C.c_int32), ("max_box_num", C.c_int32),
                ("score_threshold", C.c_float), ("direction_offset", C.c_float)]


class NmsParams(C.Structure):
    _fields_ = [("max_box_num", C.c_int32), ("nms_thresh", C.c_float)]


class S2DParams(C.Structure):
    _fields_ = [("feature_map_size_x", C.c_int32), ("feature_map_size_y", C.c_int32),
                ("feature_map_size_z", C.c_int32), ("feature_map_channel", C.c_int32)]


_lib = None


def lib():
    """The loaded CUDA library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise SessdError(f"{LIB_PATH} is missing: run build() (needs nvcc); there is no CPU fallback")
        L = C.CDLL(LIB_PATH)
        for name in ("sessd_voxelize_workspace_bytes", "sessd_conv_workspace_bytes", "sessd_backbone_workspace_bytes",
                     "sessd_filter_boxes_workspace_bytes", "sessd_rotated_nms_workspace_bytes"):
            getattr(L, name).restype = C.c_size_t
        for name in ("sessd_voxelize_num_points", "sessd_pipeline_dense", "sessd_pipeline_workspace"):
            getattr(L, name).restype = C.c_void_p
        L.sessd_launch_count.restype = C.c_uint64
        L.sessd_last_cuda_error.restype = C.c_char_p
        L.sessd_version.restype = C.c_char_p
        _lib = L
    return _lib


def _check(rc: int, what: str):
    if rc != 0:
        names = {-1: "null pointer", -2: "bad parameter", -3: "workspace too small", -4: "CUDA error",
                 -5: "unsupported configuration", -6: "file missing, unreadable or malformed"}
        extra = lib().sessd_last_cuda_error().decode() if rc == -4 else ""
        raise SessdError(f"{what} failed: {names.get(rc, rc)} {extra}")


def _torch():
    import torch

    if not torch.cuda.is_available():
        raise SessdError("a CUDA device is required (there is no CPU path in this package)")
    return torch


def _stream():
    return C.c_void_p(_torch().cuda.current_stream().cuda_stream)


def _vp(*tensors):
    return (C.c_void_p * len(tensors))(*[C.c_void_p(t.data_ptr()) if t is not None else None for t in tensors])


def _tdtype(dtype):
    torch = _torch()
    return torch.float32 if dtype == F32 else torch.float16


def voxel_params(max_voxels, point_range=synth.POINT_RANGE, voxel_size=synth.VOXEL_SIZE, max_points_per_voxel=5):
    """VoxelParams from (xmin, ymin, zmin, xmax, ymax, zmax) and (vx, vy, vz), grid filled like configurePlugin."""
    xmin, ymin, zmin, xmax, ymax, zmax = point_range
    p = VoxelParams(max_voxels, max_points_per_voxel, 4, xmin, xmax, ymin, ymax, zmin, zmax, *voxel_size, 4, 0, 0, 0)
    _check(lib().sessd_voxel_configure(C.byref(p)), "sessd_voxel_configure")
    return p


def conv_params(layer: schedule.ConvLayer, max_voxels: int) -> ConvParams:
    p = ConvParams()
    p.in_channel, p.out_channel, p.max_voxels, p.feature_num = layer.cin, layer.cout, max_voxels, layer.cin
    p.out_shape_z, p.out_shape_y, p.out_shape_x = layer.out_shape
    p.spatial_shape_z, p.spatial_shape_y, p.spatial_shape_x = layer.in_shape
    for j in range(3):
        p.ksize[j], p.stride[j], p.padding[j] = layer.ksize[j], layer.stride[j], layer.padding[j]
    p.dilation, p.out_padding, p.subm = 1, 0, int(layer.subm)
    return p


def read_status(workspace) -> int:
    rc = lib().sessd_read_status(C.c_void_p(workspace.data_ptr()), _stream())
    if rc < 0:
        _check(rc, "sessd_read_status")
    return rc


def voxelize(points, points_size, params: VoxelParams, out_dtype=F32):
    """points: cuda f32 [B, P, 4]; points_size: cuda i32 [B]. Returns dict of cuda tensors + status."""
    torch = _torch()
    B, P = points.shape[0], points.shape[1]
    nbytes = lib().sessd_voxelize_workspace_bytes(C.byref(params), B, P)
    if nbytes == 0:
        raise SessdError("sessd_voxelize_workspace_bytes rejected the parameters")
    ws = torch.empty(nbytes, dtype=torch.uint8, device=points.device)
    V = params.max_voxels
    voxels = torch.empty((B, V, 4), dtype=_tdtype(out_dtype), device=points.device)
    coors = torch.empty((B, V, 4), dtype=torch.int32, device=points.device)
    num = torch.empty((B,), dtype=torch.int32, device=points.device)
    _check(lib().sessd_voxelize_enqueue(C.byref(params), B, P, out_dtype, _vp(points, points_size),
                                        _vp(voxels, coors, num), C.c_void_p(ws.data_ptr()), C.c_size_t(nbytes),
                                        _stream()), "sessd_voxelize_enqueue")
    status = read_status(ws)
    npv_ptr = lib().sessd_voxelize_num_points(C.byref(params), B, P, C.c_void_p(ws.data_ptr()))
    off = (npv_ptr - ws.data_ptr())
    npv = ws[off:off + B * V * 4].view(torch.int32).reshape(B, V).clone()
    return dict(voxels=voxels, coors=coors, voxel_num=num, num_points=npv, status=status)


def voxelize_into(points, points_size, params: VoxelParams, voxels, coors, voxel_num, workspace, out_dtype=F32):
    """sessd_voxelize_enqueue into caller-owned outputs and workspace (nothing is allocated, nothing is read back)."""
    B, P = points.shape[0], points.shape[1]
    _check(lib().sessd_voxelize_enqueue(C.byref(params), B, P, out_dtype, _vp(points, points_size),
                                        _vp(voxels, coors, voxel_num), C.c_void_p(workspace.data_ptr()),
                                        C.c_size_t(workspace.numel()), _stream()), "sessd_voxelize_enqueue")


class ConvWeights:
    """Device weights of one sparse conv layer (+ optional folded scale/shift/ReLU epilogue)."""

    def __init__(self, params: ConvParams, weights, scale=None, shift=None, relu=False, dtype=F32):
        _torch()
        w = np.ascontiguousarray(weights, dtype=np.float32)
        self._keep = [w]
        fp = C.POINTER(C.c_float)
        sc = sh = None
        if scale is not None:
            s = np.ascontiguousarray(scale, dtype=np.float32)
            self._keep.append(s)
            sc = s.ctypes.data_as(fp)
        if shift is not None:
            s = np.ascontiguousarray(shift, dtype=np.float32)
            self._keep.append(s)
            sh = s.ctypes.data_as(fp)
        self.handle = C.c_void_p()
        self.dtype = dtype
        _check(lib().sessd_conv_weights_create(C.byref(params), w.ctypes.data_as(fp), sc, sh, int(relu), dtype,
                                               C.byref(self.handle)), "sessd_conv_weights_create")

    def close(self):
        if self.handle:
            lib().sessd_conv_weights_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _conv_workspace(params, B, device):
    torch = _torch()
    nbytes = lib().sessd_conv_workspace_bytes(C.byref(params), B)
    if nbytes == 0:
        raise SessdError("sessd_conv_workspace_bytes rejected the parameters")
    return torch.empty(nbytes, dtype=torch.uint8, device=device), nbytes


def subm_conv(feat, coors, voxel_num, params: ConvParams, weights: ConvWeights, keep_workspace=False):
    torch = _torch()
    B, V = feat.shape[0], params.max_voxels
    ws, nbytes = _conv_workspace(params, B, feat.device)
    out = torch.empty((B, V, params.out_channel), dtype=_tdtype(weights.dtype), device=feat.device)
    _check(lib().sessd_subm_conv_enqueue(C.byref(params), weights.handle, B, _vp(feat, coors, voxel_num), _vp(out),
                                         C.c_void_p(ws.data_ptr()), C.c_size_t(nbytes), _stream()),
           "sessd_subm_conv_enqueue")
    status = read_status(ws)
    r = dict(features=out, status=status)
    if keep_workspace:
        r["workspace"] = ws
    return r


def subm_conv_into(feat, coors, voxel_num, params: ConvParams, weights: ConvWeights, out, workspace):
    """sessd_subm_conv_enqueue into a caller-owned output and workspace (nothing is allocated or read back)."""
    _check(lib().sessd_subm_conv_enqueue(C.byref(params), weights.handle, feat.shape[0], _vp(feat, coors, voxel_num),
                                         _vp(out), C.c_void_p(workspace.data_ptr()), C.c_size_t(workspace.numel()),
                                         _stream()), "sessd_subm_conv_enqueue")


def sparse_conv(feat, coors, voxel_num, params: ConvParams, weights: ConvWeights, keep_workspace=False):
    torch = _torch()
    B, V = feat.shape[0], params.max_voxels
    ws, nbytes = _conv_workspace(params, B, feat.device)
    out = torch.empty((B, V, params.out_channel), dtype=_tdtype(weights.dtype), device=feat.device)
    ocoors = torch.empty((B, V, 4), dtype=torch.int32, device=feat.device)
    onum = torch.empty((B,), dtype=torch.int32, device=feat.device)
    _check(lib().sessd_sparse_conv_enqueue(C.byref(params), weights.handle, B, _vp(feat, coors, voxel_num),
                                           _vp(out, ocoors, onum), C.c_void_p(ws.data_ptr()), C.c_size_t(nbytes),
                                           _stream()), "sessd_sparse_conv_enqueue")
    status = read_status(ws)
    r = dict(features=out, coors=ocoors, voxel_num=onum, status=status)
    if keep_workspace:
        r["workspace"] = ws
    return r


def rulebook_export(params: ConvParams, B, frame, workspace, out_voxel_num):
    """Reference-layout rulebook of the last conv call that used `workspace` (cuda tensors)."""
    torch = _torch()
    kvol = params.ksize[0] * params.ksize[1] * params.ksize[2]
    pairs = torch.empty((kvol, 2, params.max_voxels), dtype=torch.int32, device=workspace.device)
    num = torch.zeros((kvol,), dtype=torch.int32, device=workspace.device)
    _check(lib().sessd_conv_rulebook_export(C.byref(params), B, frame, C.c_void_p(workspace.data_ptr()),
                                            C.c_void_p(pairs.data_ptr()), C.c_void_p(num.data_ptr()), _stream(),
                                            C.c_void_p(out_voxel_num.data_ptr())), "sessd_conv_rulebook_export")
    torch.cuda.current_stream().synchronize()
    return pairs, num


def sparse2dense(feat, coors, voxel_num, params: S2DParams, dtype=F32, pad: Pad2DParams = None):
    """Sparse rows -> dense BEV map; with `pad` the zero border of ZeroPad2dPlugin is written in the same pass."""
    torch = _torch()
    B, V = feat.shape[0], feat.shape[1]
    ph = (pad.top + pad.bottom) if pad else 0
    pw = (pad.left + pad.right) if pad else 0
    dense = torch.empty((B, params.feature_map_channel * params.feature_map_size_z, params.feature_map_size_y + ph,
                         params.feature_map_size_x + pw), dtype=_tdtype(dtype), device=feat.device)
    if pad is None:
        _check(lib().sessd_sparse2dense_enqueue(C.byref(params), B, V, dtype, _vp(feat, coors, voxel_num), _vp(dense),
                                                None, C.c_size_t(0), _stream()), "sessd_sparse2dense_enqueue")
    else:
        _check(lib().sessd_sparse2dense_padded_enqueue(C.byref(params), C.byref(pad), B, V, dtype,
                                                       _vp(feat, coors, voxel_num), _vp(dense), _stream()),
               "sessd_sparse2dense_padded_enqueue")
    return dense


def zero_pad2d(x, pad: Pad2DParams, dtype=F32):
    """[B, C, H, W] -> [B, C, top+H+bottom, left+W+right] with a zero border (ZeroPad2dPlugin)."""
    torch = _torch()
    B, Cc, H, W = x.shape
    out = torch.empty((B, Cc, H + pad.top + pad.bottom, W + pad.left + pad.right), dtype=_tdtype(dtype), device=x.device)
    _check(lib().sessd_zero_pad2d_enqueue(C.byref(pad), B, Cc, H, W, dtype, _vp(x), _vp(out), _stream()),
           "sessd_zero_pad2d_enqueue")
    return out


def anchor_params(point_range=synth.POINT_RANGE, height=schedule.FEATURE_MAP_HEIGHT, width=schedule.FEATURE_MAP_WIDTH,
                  car_size=schedule.CAR_SIZE, direction_angles=schedule.DIRECTION_ANGLES) -> AnchorParams:
    """AnchorParams from (xmin, ymin, zmin, xmax, ymax, zmax), (length, width, height) and the anchor yaws."""
    xmin, ymin, zmin, xmax, ymax, zmax = point_range
    return AnchorParams(xmin, xmax, ymin, ymax, zmin, zmax, height, width, *car_size, direction_angles[0],
                        direction_angles[1], len(direction_angles))


def filter_params(height=schedule.FEATURE_MAP_HEIGHT, width=schedule.FEATURE_MAP_WIDTH, direction_angle_num=2,
                  max_box_num=schedule.MAX_BOX_NUM, score_threshold=schedule.SCORE_THRESHOLD,
                  direction_offset=schedule.DIRECTION_OFFSET) -> FilterParams:
    return FilterParams(height, width, direction_angle_num, max_box_num, score_threshold, direction_offset)


def anchor_decode(box_preds, params: AnchorParams):
    """[B, N, 7] regression outputs -> [B, N, 7] boxes (GenerateAnchorDecodePlugin)."""
    torch = _torch()
    out = torch.empty_like(box_preds)
    _check(lib().sessd_anchor_decode_enqueue(C.byref(params), box_preds.shape[0], _vp(box_preds), _vp(out), _stream()),
           "sessd_anchor_decode_enqueue")
    return out


def filter_boxes(boxes, cls, iou, dirs, params: FilterParams, anchors: AnchorParams = None, read_back_status=True):
    """Score filter + ordered compaction (FilterBoxByScorePlugin). With `anchors`, `boxes` holds the regression
    outputs and decoding is fused in. Returns dict(box, score, iou, direction, valid, status); with
    read_back_status=False nothing synchronises (stream capture) and `workspace` is returned for read_status."""
    torch = _torch()
    B, M = boxes.shape[0], params.max_box_num
    f32 = dict(dtype=torch.float32, device=boxes.device)
    out = dict(box=torch.empty((B, M, 9), **f32), score=torch.empty((B, M), **f32), iou=torch.empty((B, M), **f32),
               direction=torch.empty((B, M), **f32), valid=torch.empty((B,), dtype=torch.int32, device=boxes.device))
    nbytes = lib().sessd_filter_boxes_workspace_bytes(C.byref(params), B)
    ws = torch.empty((nbytes,), dtype=torch.uint8, device=boxes.device)
    ins = _vp(boxes, cls, iou, dirs)
    outs = _vp(out["box"], out["score"], out["iou"], out["direction"], out["valid"])
    if anchors is None:
        _check(lib().sessd_filter_boxes_enqueue(C.byref(params), B, ins, outs, C.c_void_p(ws.data_ptr()),
                                                C.c_size_t(nbytes), _stream()), "sessd_filter_boxes_enqueue")
    else:
        _check(lib().sessd_decode_filter_enqueue(C.byref(anchors), C.byref(params), B, ins, outs,
                                                 C.c_void_p(ws.data_ptr()), C.c_size_t(nbytes), _stream()),
               "sessd_decode_filter_enqueue")
    if read_back_status:
        out["status"] = read_status(ws)
    else:
        out["workspace"] = ws
    return out


def rotated_nms(boxes, valid, nms_thresh=schedule.NMS_THRESH):
    """Greedy rotated NMS (the reference's host nms_cpu) of [B, M, 9] boxes with valid[b] rows each.
    Returns (kept [B, M, 9], kept_num [B])."""
    torch = _torch()
    B, M = boxes.shape[0], boxes.shape[1]
    p = NmsParams(M, nms_thresh)
    kept = torch.empty_like(boxes)
    kept_num = torch.empty((B,), dtype=torch.int32, device=boxes.device)
    nbytes = lib().sessd_rotated_nms_workspace_bytes(C.byref(p), B)
    ws = torch.empty((max(nbytes, 1),), dtype=torch.uint8, device=boxes.device)
    _check(lib().sessd_rotated_nms_enqueue(C.byref(p), B, _vp(boxes, valid), _vp(kept, kept_num),
                                           C.c_void_p(ws.data_ptr()), C.c_size_t(nbytes), _stream()),
           "sessd_rotated_nms_enqueue")
    return kept, kept_num


class Backbone:
    """voxelise -> conv stack (BN + ReLU folded) -> dense BEV, one C call per batch of frames."""

    def __init__(self, max_voxels, weights, scale=None, shift=None, dtype=F16, layers=schedule.LAYERS,
                 point_range=synth.POINT_RANGE, voxel_size=synth.VOXEL_SIZE, with_dense=True):
        _torch()
        self.layers, self.dtype, self.max_voxels = tuple(layers), dtype, max_voxels
        self.vp = voxel_params(max_voxels, point_range, voxel_size)
        n = len(self.layers)
        cps = (ConvParams * n)(*[conv_params(l, max_voxels) for l in self.layers])
        fp = C.POINTER(C.c_float)
        self._keep = [np.ascontiguousarray(w, dtype=np.float32) for w in weights]
        wptr = (fp * n)(*[w.ctypes.data_as(fp) for w in self._keep])
        scptr = shptr = None
        if scale is not None:
            sc = [np.ascontiguousarray(s, dtype=np.float32) for s in scale]
            sh = [np.ascontiguousarray(s, dtype=np.float32) for s in shift]
            self._keep += sc + sh
            scptr = (fp * n)(*[s.ctypes.data_as(fp) for s in sc])
            shptr = (fp * n)(*[s.ctypes.data_as(fp) for s in sh])
        last = self.layers[-1]
        self.s2d = S2DParams(last.out_shape[2], last.out_shape[1], last.out_shape[0], last.cout) if with_dense else None
        self.handle = C.c_void_p()
        _check(lib().sessd_backbone_create(C.byref(self.vp), cps, n, wptr, scptr, shptr,
                                           C.byref(self.s2d) if with_dense else None, dtype, C.byref(self.handle)),
               "sessd_backbone_create")

    @classmethod
    def from_wts(cls, wts, max_voxels, dtype=F16, layers=schedule.LAYERS, module_index=None,
                 prefix="backbone.middle_conv", eps=1e-5, point_range=synth.POINT_RANGE,
                 voxel_size=synth.VOXEL_SIZE, with_dense=True):
        """Backbone from a parsed weight file (formats.Wts): conv weights `<prefix>.<i>.weight`, batch norm
        `<prefix>.<i+1>.*` folded with eps, i = module_index[l] (default: the digits of the layer's name)."""
        _torch()
        self = cls.__new__(cls)
        self.layers, self.dtype, self.max_voxels = tuple(layers), dtype, max_voxels
        self.vp = voxel_params(max_voxels, point_range, voxel_size)
        n = len(self.layers)
        if module_index is None:
            module_index = [int("".join(ch for ch in l.name if ch.isdigit())) for l in self.layers]
        cps = (ConvParams * n)(*[conv_params(l, max_voxels) for l in self.layers])
        idx = (C.c_int32 * n)(*module_index)
        last = self.layers[-1]
        self.s2d = S2DParams(last.out_shape[2], last.out_shape[1], last.out_shape[0], last.cout) if with_dense else None
        self._keep = []
        self.handle = C.c_void_p()
        _check(lib().sessd_backbone_create_from_wts(C.byref(self.vp), cps, n, idx, wts.handle, prefix.encode(),
                                                    C.c_float(eps), C.byref(self.s2d) if with_dense else None,
                                                    dtype, C.byref(self.handle)), "sessd_backbone_create_from_wts")
        return self

    def workspace_bytes(self, batch, max_points) -> int:
        n = lib().sessd_backbone_workspace_bytes(self.handle, batch, max_points)
        if n == 0:
            raise SessdError("sessd_backbone_workspace_bytes rejected the parameters")
        return n

    def set_padding(self, top, bottom, left, right):
        """Folds ZeroPad2dPlugin into the dense output (call before run / before creating a Pipeline)."""
        self.pad = Pad2DParams(top, bottom, left, right)
        _check(lib().sessd_backbone_set_padding(self.handle, C.byref(self.pad)), "sessd_backbone_set_padding")

    def dense_shape(self, batch):
        pad = getattr(self, "pad", None)
        ph = (pad.top + pad.bottom) if pad else 0
        pw = (pad.left + pad.right) if pad else 0
        return (batch, self.s2d.feature_map_channel * self.s2d.feature_map_size_z, self.s2d.feature_map_size_y + ph,
                self.s2d.feature_map_size_x + pw)

    def run(self, points, points_size, workspace=None, dense=None):
        """points cuda f32 [B, P, 4], points_size cuda i32 [B] -> (dense, workspace)."""
        torch = _torch()
        B, P = points.shape[0], points.shape[1]
        nbytes = self.workspace_bytes(B, P)
        if workspace is None:
            workspace = torch.empty(nbytes, dtype=torch.uint8, device=points.device)
        if dense is None and self.s2d is not None:
            dense = torch.empty(self.dense_shape(B), dtype=_tdtype(self.dtype), device=points.device)
        _check(lib().sessd_backbone_enqueue(self.handle, B, P, C.c_void_p(points.data_ptr()),
                                            C.c_void_p(points_size.data_ptr()),
                                            C.c_void_p(dense.data_ptr()) if dense is not None else None,
                                            C.c_void_p(workspace.data_ptr()), C.c_size_t(workspace.numel()), _stream()),
               "sessd_backbone_enqueue")
        return dense, workspace

    def layer_view(self, workspace, batch, max_points, layer):
        """(features, coors, voxel_num) cuda tensors of conv layer `layer` (-1: voxeliser output)."""
        torch = _torch()
        f, c, n = C.c_void_p(), C.c_void_p(), C.c_void_p()
        _check(lib().sessd_backbone_layer_view(self.handle, batch, max_points, C.c_void_p(workspace.data_ptr()), layer,
                                               C.byref(f), C.byref(c), C.byref(n)), "sessd_backbone_layer_view")
        ch = 4 if layer < 0 else self.layers[layer].cout
        es = 4 if self.dtype == F32 else 2
        V = self.max_voxels
        base = workspace.data_ptr()

        def view(ptr, nbytes, dt, shape):
            off = ptr.value - base
            return workspace[off:off + nbytes].view(dt).reshape(shape)

        return (view(f, batch * V * ch * es, _tdtype(self.dtype), (batch, V, ch)),
                view(c, batch * V * 16, torch.int32, (batch, V, 4)),
                view(n, batch * 4, torch.int32, (batch,)))

    def close(self):
        if self.handle:
            lib().sessd_backbone_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Pipeline:
    """Streams + device buffers that push frames through a Backbone `batch` at a time."""

    def __init__(self, backbone: Backbone, batch, max_points, nstreams=2):
        self.backbone, self.batch, self.max_points, self.nstreams = backbone, batch, max_points, nstreams
        self.handle = C.c_void_p()
        _check(lib().sessd_pipeline_create(backbone.handle, batch, max_points, nstreams, C.byref(self.handle)),
               "sessd_pipeline_create")

    def use_graphs(self, enable=True):
        """Replay the launch sequence of full groups from CUDA graphs (captured per stream slot on second use)."""
        _check(lib().sessd_pipeline_use_graphs(self.handle, int(bool(enable))), "sessd_pipeline_use_graphs")

    def run_device(self, points, sizes) -> float:
        """points cuda f32 [F, P, 4], sizes cuda i32 [F]; returns device milliseconds."""
        ms = C.c_float(0)
        _check(lib().sessd_pipeline_run_device(self.handle, C.c_void_p(points.data_ptr()), C.c_void_p(sizes.data_ptr()),
                                               points.shape[0], C.byref(ms)), "sessd_pipeline_run_device")
        return float(ms.value)

    def run_host(self, points, sizes, voxel_num, status) -> float:
        """points pinned f32 [F, P, 4], sizes/voxel_num/status pinned i32 [F] (CPU tensors)."""
        ms = C.c_float(0)
        _check(lib().sessd_pipeline_run_host(self.handle, C.c_void_p(points.data_ptr()), C.c_void_p(sizes.data_ptr()),
                                             points.shape[0], C.c_void_p(voxel_num.data_ptr()),
                                             C.c_void_p(status.data_ptr()), C.byref(ms)), "sessd_pipeline_run_host")
        return float(ms.value)

    def run_host_bev(self, points, sizes, voxel_num, status, host_dense) -> float:
        """run_host, and every group's BEV maps are copied into host_dense, pinned [nstreams, batch, C*D, H, W]
        (the region of the stream slot the group ran on)."""
        ms = C.c_float(0)
        _check(lib().sessd_pipeline_run_host_bev(self.handle, C.c_void_p(points.data_ptr()), C.c_void_p(sizes.data_ptr()),
                                                 points.shape[0], C.c_void_p(voxel_num.data_ptr()),
                                                 C.c_void_p(status.data_ptr()), C.c_void_p(host_dense.data_ptr()),
                                                 C.byref(ms)), "sessd_pipeline_run_host_bev")
        return float(ms.value)

    def dense(self, s):
        """The dense BEV buffer of stream slot `s` as a cuda tensor [batch, C*D, H, W] (a view, not a copy)."""
        torch = _torch()
        ptr = lib().sessd_pipeline_dense(self.handle, s)
        if not ptr:
            raise ValueError("no such stream slot")
        shape = tuple(self.backbone.dense_shape(self.batch))
        typestr = "<f4" if self.backbone.dtype == F32 else "<f2"

        class _View:
            __cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (int(ptr), False), "version": 2}

        return torch.as_tensor(_View(), device="cuda")

    def status_bits(self) -> int:
        """OR of the status words of all stream workspaces (synchronises the device)."""
        torch = _torch()
        torch.cuda.synchronize()
        bits = 0
        for s in range(self.nstreams):
            ws = lib().sessd_pipeline_workspace(self.handle, s)
            rc = lib().sessd_read_status(C.c_void_p(ws), None)
            if rc < 0:
                _check(rc, "sessd_read_status")
            bits |= rc
        return bits

    def close(self):
        if self.handle:
            lib().sessd_pipeline_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def profile(fn):
    """Runs fn() with per-launch timing; returns [(kernel name, ms), ...] in launch order."""
    _check(lib().sessd_profile_begin(), "sessd_profile_begin")
    try:
        fn()
    finally:
        cap = 4096
        names = C.create_string_buffer(1 << 18)
        ms = (C.c_float * cap)()
        n = lib().sessd_profile_end(_stream(), names, C.c_size_t(len(names)), ms, cap)
    if n < 0:
        _check(n, "sessd_profile_end")
    nm = names.value.decode().split("\n")[:n]
    return [(nm[i], float(ms[i])) for i in range(min(n, cap))]


def pair_counts(backbone: Backbone, points, points_size, workspace, dense):
    """Runs the backbone once more and returns the number of rulebook pairs of every layer (list of int)."""
    B, P = points.shape[0], points.shape[1]
    out = (C.c_int64 * len(backbone.layers))()
    _check(lib().sessd_backbone_pair_counts(backbone.handle, B, P, C.c_void_p(points.data_ptr()),
                                            C.c_void_p(points_size.data_ptr()),
                                            C.c_void_p(dense.data_ptr()) if dense is not None else None,
                                            C.c_void_p(workspace.data_ptr()), C.c_size_t(workspace.numel()), _stream(),
                                            out), "sessd_backbone_pair_counts")
    return [int(v) for v in out]


def launch_count() -> int:
    return int(lib().sessd_launch_count())


def random_weights(seed=0x5E55D000 + 3, layers=schedule.LAYERS, std=0.02, with_bn=True):
    """Seeded N(0, std) weights per layer and a seeded BatchNorm folded to (scale, shift)."""
    ws, scs, shs = [], [], []
    for i, l in enumerate(layers):
        ws.append(synth.normal_f32(seed + 17 * i, (l.kvol, l.cin, l.cout), std))
        if with_bn:
            s = synth.Stream(seed + 17 * i + 7)
            gamma = 1.0 + 0.1 * s.normal(l.cout)
            beta = 0.05 * s.normal(l.cout)
            mean = 0.02 * s.normal(l.cout)
            var = 0.5 + s.uniform(l.cout) * 0.02
            # weights this small give conv outputs ~1e-2; scale them back to O(1) like a trained BN would
            var = var * (std * std * l.kvol * l.cin / 4.0)
            g32, b32, m32, v32 = [t.astype(np.float32) for t in (gamma, beta, mean, var)]
            sc = (g32 / np.sqrt(v32 + np.float32(schedule.BN_EPS))).astype(np.float32)
            sh = (b32 - m32 * g32 / np.sqrt(v32 + np.float32(schedule.BN_EPS))).astype(np.float32)
            scs.append(sc)
            shs.append(sh)
    return ws, (scs if with_bn else None), (shs if with_bn else None)
