"""ctypes view of liboracle.so.

Test infrastructure: imported only by the test-suite, the smoke check and the CPU-baseline
leg of the benchmark, never by the product package.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))  # repository root
_LIB = os.path.join(_ROOT, "oracle", "liboracle.so")

VOXEL_OVERFLOW = 1
PAIR_OVERFLOW = 2


def _ptr(a, t):
    return a.ctypes.data_as(C.POINTER(t)) if a is not None else None


def load():
    if not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(os.path.join(_ROOT, "oracle", "oracle.cpp")):
        subprocess.check_call(["make", "-C", os.path.join(_ROOT, "oracle")], stdout=subprocess.DEVNULL)
    lib = C.CDLL(_LIB)
    lib.oracle_front_end_frames.restype = C.c_double
    return lib


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = load()
    return _lib


def np_round(x: float) -> int:
    return lib().oracle_np_round(C.c_float(x))


def grid_size(point_range, voxel_size):
    r = np.asarray(point_range, dtype=np.float32)
    v = np.asarray(voxel_size, dtype=np.float32)
    g = np.zeros(3, dtype=np.int32)
    lib().oracle_grid_size(_ptr(r, C.c_float), _ptr(v, C.c_float), _ptr(g, C.c_int))
    return tuple(int(t) for t in g)  # gx, gy, gz


def voxelize(points, point_range, voxel_size, max_voxels, max_pts=5, batch_idx=0, num_points=None):
    points = np.ascontiguousarray(points, dtype=np.float32)
    n = points.shape[0] if num_points is None else num_points
    xmin, ymin, zmin, xmax, ymax, zmax = [np.float32(t) for t in point_range]
    vx, vy, vz = [np.float32(t) for t in voxel_size]
    gx, gy, gz = grid_size(point_range, voxel_size)
    voxels = np.zeros((max_voxels, 4), np.float32)
    coors = np.zeros((max_voxels, 4), np.int32)
    npv = np.zeros(max_voxels, np.int32)
    num = np.zeros(1, np.int32)
    st = lib().oracle_voxelize(_ptr(points, C.c_float), C.c_int(n), C.c_int(batch_idx),
                               C.c_float(xmin), C.c_float(xmax), C.c_float(ymin), C.c_float(ymax),
                               C.c_float(zmin), C.c_float(zmax), C.c_float(vx), C.c_float(vy), C.c_float(vz),
                               C.c_int(gx), C.c_int(gy), C.c_int(gz), C.c_int(max_voxels), C.c_int(max_pts),
                               _ptr(voxels, C.c_float), _ptr(coors, C.c_int32), _ptr(npv, C.c_int32),
                               _ptr(num, C.c_int32))
    return voxels, coors, npv, int(num[0]), st


def subm_rulebook(coors, n, shape_zyx, max_voxels, ksize=3, padding=1):
    coors = np.ascontiguousarray(coors, dtype=np.int32)
    kvol = ksize ** 3
    pairs = np.empty((kvol, 2, max_voxels), np.int32)
    num = np.zeros(kvol, np.uint32)
    st = lib().oracle_subm_rulebook(_ptr(coors, C.c_int32), C.c_int(n), C.c_int(shape_zyx[0]), C.c_int(shape_zyx[1]),
                                    C.c_int(shape_zyx[2]), C.c_int(ksize), C.c_int(1), C.c_int(padding), C.c_int(1),
                                    C.c_int(max_voxels), _ptr(pairs, C.c_int32), _ptr(num, C.c_uint32))
    return pairs, num, st


def spconv_rulebook(coors, n, ksize, stride, padding, out_shape_zyx, max_voxels):
    coors = np.ascontiguousarray(coors, dtype=np.int32)
    K = np.asarray(ksize, np.int32)
    S = np.asarray(stride, np.int32)
    P = np.asarray(padding, np.int32)
    kvol = int(K.prod())
    pairs = np.empty((kvol, 2, max_voxels), np.int32)
    num = np.zeros(kvol, np.uint32)
    out_coors = np.zeros((max_voxels, 4), np.int32)
    out_num = np.zeros(1, np.int32)
    st = lib().oracle_spconv_rulebook(_ptr(coors, C.c_int32), C.c_int(n), _ptr(K, C.c_int), _ptr(S, C.c_int),
                                      _ptr(P, C.c_int), C.c_int(1), C.c_int(out_shape_zyx[0]), C.c_int(out_shape_zyx[1]),
                                      C.c_int(out_shape_zyx[2]), C.c_int(max_voxels), _ptr(out_coors, C.c_int32),
                                      _ptr(out_num, C.c_int32), _ptr(pairs, C.c_int32), _ptr(num, C.c_uint32))
    return out_coors, int(out_num[0]), pairs, num, st


def conv_apply(feat, pairs, pair_num, weights, out_rows, half_inputs=False):
    feat = np.ascontiguousarray(feat, dtype=np.float32)
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    kvol, cin, cout = weights.shape
    out = np.zeros((max(out_rows, 1), cout), np.float32)
    lib().oracle_conv_apply(_ptr(feat, C.c_float), C.c_int(cin), C.c_int(cout), _ptr(pairs, C.c_int32),
                            _ptr(pair_num, C.c_uint32), C.c_int(kvol), C.c_int(pairs.shape[2]),
                            _ptr(weights, C.c_float), _ptr(out, C.c_float), C.c_int(out_rows), C.c_int(int(half_inputs)))
    return out[:out_rows]


def conv_apply_f64(feat, pairs, pair_num, weights, out_rows):
    feat = np.ascontiguousarray(feat, dtype=np.float32)
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    kvol, cin, cout = weights.shape
    out = np.zeros((max(out_rows, 1), cout), np.float64)
    lib().oracle_conv_apply_f64(_ptr(feat, C.c_float), C.c_int(cin), C.c_int(cout), _ptr(pairs, C.c_int32),
                                _ptr(pair_num, C.c_uint32), C.c_int(kvol), C.c_int(pairs.shape[2]),
                                _ptr(weights, C.c_float), _ptr(out, C.c_double), C.c_int(out_rows))
    return out[:out_rows]


def scale_shift_relu(x, scale, shift, relu=True, half_out=False):
    x = np.ascontiguousarray(x, dtype=np.float32).copy()
    n, c = x.shape
    sc = None if scale is None else np.ascontiguousarray(scale, np.float32)
    sh = None if shift is None else np.ascontiguousarray(shift, np.float32)
    lib().oracle_scale_shift_relu(_ptr(x, C.c_float), C.c_int(n), C.c_int(c), _ptr(sc, C.c_float), _ptr(sh, C.c_float),
                                  C.c_int(int(relu)), C.c_int(int(half_out)))
    return x


def fold_bn(gamma, beta, mean, var, eps=1e-5):
    g, b, m, v = [np.ascontiguousarray(t, np.float32) for t in (gamma, beta, mean, var)]
    sc = np.zeros_like(g)
    sh = np.zeros_like(g)
    lib().oracle_fold_bn(_ptr(g, C.c_float), _ptr(b, C.c_float), _ptr(m, C.c_float), _ptr(v, C.c_float),
                         C.c_float(eps), C.c_int(g.size), _ptr(sc, C.c_float), _ptr(sh, C.c_float))
    return sc, sh


def sparse2dense(feat, coors, n, C_, D, H, W, batch=1):
    feat = np.ascontiguousarray(feat, np.float32)
    coors = np.ascontiguousarray(coors, np.int32)
    dense = np.zeros((batch, C_ * D, H, W), np.float32)
    lib().oracle_sparse2dense(_ptr(feat, C.c_float), _ptr(coors, C.c_int32), C.c_int(n), C.c_int(C_), C.c_int(D),
                              C.c_int(H), C.c_int(W), C.c_int(batch), _ptr(dense, C.c_float))
    return dense


def zero_pad2d(x, top, bottom, left, right):
    x = np.ascontiguousarray(x, np.float32)
    planes = int(np.prod(x.shape[:-2]))
    H, W = x.shape[-2:]
    out = np.zeros(x.shape[:-2] + (H + top + bottom, W + left + right), np.float32)
    lib().oracle_zero_pad2d(_ptr(x, C.c_float), C.c_size_t(planes), C.c_int(H), C.c_int(W), C.c_int(top), C.c_int(bottom),
                            C.c_int(left), C.c_int(right), _ptr(out, C.c_float))
    return out


def anchor_params(point_range, car_size, direction_angles):
    """{min_x, max_x, min_y, max_y, min_z, max_z, car_length, car_width, car_height, angle0, angle1} as fp32."""
    xmin, ymin, zmin, xmax, ymax, zmax = point_range
    return np.asarray([xmin, xmax, ymin, ymax, zmin, zmax, *car_size, *direction_angles], np.float32)


def anchor_decode(box_preds, aparams, height, width, dir_num):
    """[N, 7] regression outputs -> [N, 7] boxes (N = height * width * dir_num), one frame."""
    box_preds = np.ascontiguousarray(box_preds, np.float32)
    assert box_preds.shape == (height * width * dir_num, 7)
    out = np.empty_like(box_preds)
    lib().oracle_anchor_decode(_ptr(box_preds, C.c_float), _ptr(np.ascontiguousarray(aparams, np.float32), C.c_float),
                               C.c_int(height), C.c_int(width), C.c_int(dir_num), _ptr(out, C.c_float))
    return out


def filter_boxes(boxes, cls, iou, dirs, dir_num, max_box, threshold, dir_offset):
    """Score filter + ordered compaction of one frame; returns (box9, cls, iou, dir, valid, passed)."""
    boxes = np.ascontiguousarray(boxes, np.float32)
    n = boxes.shape[0]
    cls = np.ascontiguousarray(cls, np.float32).reshape(n)
    iou = np.ascontiguousarray(iou, np.float32).reshape(n)
    dirs = np.ascontiguousarray(dirs, np.float32).reshape(n, 2)
    ob, oc = np.empty((max_box, 9), np.float32), np.empty(max_box, np.float32)
    oi, od = np.empty(max_box, np.float32), np.empty(max_box, np.float32)
    valid = np.zeros(1, np.uint32)
    lib().oracle_filter_boxes.restype = C.c_int
    passed = lib().oracle_filter_boxes(_ptr(boxes, C.c_float), _ptr(cls, C.c_float), _ptr(iou, C.c_float),
                                       _ptr(dirs, C.c_float), C.c_int(n), C.c_int(dir_num), C.c_int(max_box),
                                       C.c_float(threshold), C.c_float(dir_offset), _ptr(ob, C.c_float),
                                       _ptr(oc, C.c_float), _ptr(oi, C.c_float), _ptr(od, C.c_float),
                                       _ptr(valid, C.c_uint32))
    return ob, oc, oi, od, int(valid[0]), int(passed)


def rotated_nms(boxes, thresh):
    """Greedy rotated NMS of [n, 9] boxes; returns (kept [count, 9], order [count] input rows)."""
    boxes = np.ascontiguousarray(boxes, np.float32)
    n = boxes.shape[0]
    kept = np.zeros((max(n, 1), 9), np.float32)
    order = np.zeros(max(n, 1), np.int32)
    lib().oracle_rotated_nms.restype = C.c_int
    cnt = lib().oracle_rotated_nms(_ptr(boxes, C.c_float), C.c_int(n), C.c_float(thresh), _ptr(kept, C.c_float),
                                   _ptr(order, C.c_int32))
    return kept[:cnt], order[:cnt]


def bev_iou(a9, b9):
    lib().oracle_bev_iou.restype = C.c_float
    a9, b9 = np.ascontiguousarray(a9, np.float32), np.ascontiguousarray(b9, np.float32)
    return float(lib().oracle_bev_iou(_ptr(a9, C.c_float), _ptr(b9, C.c_float)))


def _vparams(point_range, voxel_size):
    xmin, ymin, zmin, xmax, ymax, zmax = point_range
    return np.asarray([xmin, xmax, ymin, ymax, zmin, zmax, *voxel_size, 0, 0, 0], np.float32)


def front_end(points, point_range, voxel_size, max_voxels, layers, weights, scale, shift, fp16=False,
              max_pts=5, with_dense=True, bev=(64, 2, 200, 176)):
    """Runs voxelise -> conv stack -> dense BEV for one frame; returns a dict of results."""
    points = np.ascontiguousarray(points, np.float32)
    vp = _vparams(point_range, voxel_size)
    grid = np.asarray(grid_size(point_range, voxel_size), np.int32)
    lay = np.asarray([l.as_ints() for l in layers], np.int32).ravel()
    weights = np.ascontiguousarray(weights, np.float32)
    sc = None if scale is None else np.ascontiguousarray(scale, np.float32)
    sh = None if shift is None else np.ascontiguousarray(shift, np.float32)
    Cc, D, H, W = bev
    dense = np.zeros((1, Cc * D, H, W), np.float32) if with_dense else None
    rows = np.zeros(len(layers), np.int32)
    prs = np.zeros(len(layers), np.int64)
    last_c = layers[-1].cout
    ffeat = np.zeros((max_voxels, last_c), np.float32)
    fcoors = np.zeros((max_voxels, 4), np.int32)
    fnum = np.zeros(1, np.int32)
    st = lib().oracle_front_end(_ptr(points, C.c_float), C.c_int(points.shape[0]), _ptr(vp, C.c_float),
                                _ptr(grid, C.c_int), C.c_int(max_voxels), C.c_int(max_pts), _ptr(lay, C.c_int),
                                C.c_int(len(layers)), _ptr(weights, C.c_float), _ptr(sc, C.c_float),
                                _ptr(sh, C.c_float), C.c_int(int(fp16)), C.c_int(Cc), C.c_int(D), C.c_int(H),
                                C.c_int(W), _ptr(dense, C.c_float), _ptr(rows, C.c_int32), _ptr(prs, C.c_int64),
                                _ptr(ffeat, C.c_float), _ptr(fcoors, C.c_int32), _ptr(fnum, C.c_int32))
    n = int(fnum[0])
    return dict(status=st, dense=dense, layer_rows=rows, layer_pairs=prs, feat=ffeat[:n], coors=fcoors[:n], num=n)


def front_end_frames(points, sizes, point_range, voxel_size, max_voxels, layers, weights, scale, shift,
                     fp16=True, nthreads=1, with_dense=True, max_pts=5, bev=(64, 2, 200, 176)):
    """Timed multi-threaded run over frames; returns (seconds, status)."""
    points = np.ascontiguousarray(points, np.float32)
    sizes = np.ascontiguousarray(sizes, np.int32)
    nframes, stride = points.shape[0], points.shape[1]
    vp = _vparams(point_range, voxel_size)
    grid = np.asarray(grid_size(point_range, voxel_size), np.int32)
    lay = np.asarray([l.as_ints() for l in layers], np.int32).ravel()
    weights = np.ascontiguousarray(weights, np.float32)
    sc = None if scale is None else np.ascontiguousarray(scale, np.float32)
    sh = None if shift is None else np.ascontiguousarray(shift, np.float32)
    Cc, D, H, W = bev
    status = C.c_int(0)
    sec = lib().oracle_front_end_frames(_ptr(points, C.c_float), _ptr(sizes, C.c_int32), C.c_int(nframes),
                                        C.c_int(stride), _ptr(vp, C.c_float), _ptr(grid, C.c_int),
                                        C.c_int(max_voxels), C.c_int(max_pts), _ptr(lay, C.c_int), C.c_int(len(layers)),
                                        _ptr(weights, C.c_float), _ptr(sc, C.c_float), _ptr(sh, C.c_float),
                                        C.c_int(int(fp16)), C.c_int(Cc), C.c_int(D), C.c_int(H), C.c_int(W),
                                        C.c_int(nthreads), C.c_int(int(with_dense)), C.byref(status))
    return float(sec), int(status.value)


def hardware_threads() -> int:
    return int(lib().oracle_hardware_threads())
