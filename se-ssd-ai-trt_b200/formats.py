"""ctypes view of the on-disk formats either side of the front end (include/sessd.h, last section): the
reference's weight files, its batch-norm folding and its point cloud files. Host code; needs no GPU."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np


def _lib():
    from . import lib

    return lib()


def _check(rc, what):
    from . import _check as check

    check(rc, what)


class Wts:
    """A parsed weight file (the reference's loadWeights, se-ssd-ai-trt.cpp:278-314)."""

    def __init__(self, path):
        self.handle = C.c_void_p()
        _check(_lib().sessd_wts_load(os.fsencode(path), C.byref(self.handle)), f"sessd_wts_load({path})")

    def __len__(self):
        return _lib().sessd_wts_count(self.handle)

    @staticmethod
    def _array(values, count):
        n = int(count.value)
        if n == 0:
            return np.zeros((0,), np.float32)
        return np.ctypeslib.as_array(values, shape=(n,)).copy()

    def entry(self, i):
        """(name, fp32 array) of blob i in file order."""
        name, values, count = C.c_char_p(), C.POINTER(C.c_float)(), C.c_int64()
        _check(_lib().sessd_wts_entry(self.handle, i, C.byref(name), C.byref(values), C.byref(count)), "sessd_wts_entry")
        return name.value.decode(), self._array(values, count)

    def find(self, name):
        """fp32 array of the blob called `name`, or None when the file has none."""
        values, count = C.POINTER(C.c_float)(), C.c_int64()
        rc = _lib().sessd_wts_find(self.handle, name.encode(), C.byref(values), C.byref(count))
        if rc == -2:
            return None
        _check(rc, "sessd_wts_find")
        return self._array(values, count)

    def close(self):
        if self.handle:
            _lib().sessd_wts_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def save_wts(path, blobs):
    """Writes {name: array} (or a list of pairs, to keep duplicates and order) in the exporter's format
    (tools/gen_wts.py:85-99)."""
    items = list(blobs.items()) if isinstance(blobs, dict) else list(blobs)
    n = len(items)
    arrays = [np.ascontiguousarray(v, dtype=np.float32).reshape(-1) for _, v in items]
    fp = C.POINTER(C.c_float)
    names = (C.c_char_p * max(n, 1))(*[k.encode() for k, _ in items])
    values = (fp * max(n, 1))(*[a.ctypes.data_as(fp) for a in arrays])
    counts = (C.c_int64 * max(n, 1))(*[a.size for a in arrays])
    _check(_lib().sessd_wts_save(os.fsencode(path), n, names, values, counts), f"sessd_wts_save({path})")


def fold_batchnorm(gamma, beta, mean, var, eps=1e-5):
    """(scale, shift) the reference's add_batchNorm1d_relu computes (se-ssd-ai-trt.cpp:808-826)."""
    arrs = [np.ascontiguousarray(a, dtype=np.float32) for a in (gamma, beta, mean, var)]
    n = arrs[0].size
    if any(a.size != n for a in arrs):
        raise ValueError("gamma, beta, mean and var must have one length")
    scale, shift = np.empty(n, np.float32), np.empty(n, np.float32)
    fp = C.POINTER(C.c_float)
    _check(_lib().sessd_fold_batchnorm(*[a.ctypes.data_as(fp) for a in arrs], n, C.c_float(eps),
                                       scale.ctypes.data_as(fp), shift.ctypes.data_as(fp)), "sessd_fold_batchnorm")
    return scale, shift


def load_points(path, max_points):
    """(points f32 [max_points, 4] zero-filled past the file's records, number of points): the reference's
    loadData (se-ssd-ai-trt.cpp:1515-1556)."""
    pts = np.empty((max_points, 4), np.float32)
    n = C.c_int32()
    _check(_lib().sessd_points_load(os.fsencode(path), pts.ctypes.data_as(C.POINTER(C.c_float)), max_points, C.byref(n)),
           f"sessd_points_load({path})")
    return pts, int(n.value)
