"""Shared fixtures. The package directory name contains dashes, so it is loaded by path."""
import importlib.util
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for _p in (ROOT, os.path.join(ROOT, "tests", "golden")):
    if _p not in sys.path:
        sys.path.insert(0, _p)


def load_package():
    name = "se_ssd_ai_trt_b200"
    if name in sys.modules:
        return sys.modules[name]
    path = os.path.join(ROOT, "se-ssd-ai-trt_b200", "__init__.py")
    spec = importlib.util.spec_from_file_location(name, path, submodule_search_locations=[os.path.dirname(path)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def oracle():
    from oracle import binding

    binding.lib()
    return binding


@pytest.fixture(scope="session")
def gpu(pkg):
    """The package with its CUDA library loaded; fails (does not skip) when the library is missing."""
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    pkg.lib()
    return pkg


def canonical_voxels(coors, n, grid_zyx):
    """Sort permutation of the first n rows by linear (b, z, y, x) key, and the keys."""
    c = np.asarray(coors[:n]).astype(np.int64)
    Z, Y, X = grid_zyx
    key = ((c[:, 0] * Z + c[:, 1]) * Y + c[:, 2]) * X + c[:, 3]
    order = np.argsort(key, kind="stable")
    return order, key[order]


def match_rows(got_coors, want_coors):
    """Index array `perm` with got_coors[perm] == want_coors, row for row: the library numbers the outputs of a
    strided layer in (z, y, x) order, the oracle in first-seen order (the reference: arrival order of an atomic),
    and the contract is equality after canonical sorting. Fails when the two coordinate sets differ."""
    def keys(c):
        c = np.asarray(c).astype(np.int64)
        return ((c[:, 0] * 4096 + c[:, 1]) * 4096 + c[:, 2]) * 4096 + c[:, 3]

    kg, kw = keys(got_coors), keys(want_coors)
    assert len(kg) == len(kw)
    og, ow = np.argsort(kg, kind="stable"), np.argsort(kw, kind="stable")
    np.testing.assert_array_equal(kg[og], kw[ow])
    assert len(np.unique(kw)) == len(kw)
    perm = np.empty(len(kw), np.int64)
    perm[ow] = og
    return perm


def canonical_rulebook(pairs, pair_num, in_coors, out_coors, in_shape, out_shape):
    """Rulebook as a sorted array of (k, in_key, out_key) triples: independent of row numbering."""
    def keys(c, shape):
        c = np.asarray(c).astype(np.int64)
        Z, Y, X = shape
        return ((c[:, 0] * Z + c[:, 1]) * Y + c[:, 2]) * X + c[:, 3]

    kin, kout = keys(in_coors, in_shape), keys(out_coors, out_shape)
    trip = []
    for k in range(pairs.shape[0]):
        m = int(pair_num[k])
        if m:
            i, o = pairs[k, 0, :m].astype(np.int64), pairs[k, 1, :m].astype(np.int64)
            trip.append(np.stack([np.full(m, k, np.int64), kin[i], kout[o]], axis=1))
    if not trip:
        return np.zeros((0, 3), np.int64)
    t = np.concatenate(trip)
    return t[np.lexsort((t[:, 2], t[:, 1], t[:, 0]))]


def rel_err(a, b):
    """max |a - b| / max(|b|, floor) with the floor at 1e-3 of the reference's largest magnitude."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    if a.size == 0:
        return 0.0
    floor = max(float(np.abs(b).max()) * 1e-3, 1e-30)
    return float((np.abs(a - b) / np.maximum(np.abs(b), floor)).max())
