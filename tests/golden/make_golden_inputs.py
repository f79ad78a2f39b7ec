"""Inputs of the committed golden cases (shared by the generator script and the tests)."""
import numpy as np


def small_layers(pkg, y=80, x=64):
    """The reference's 14-layer schedule on a grid shrunk in y and x (z keeps its 41 cells)."""
    S = pkg.schedule
    shapes = [(41, y, x), (21, y // 2, x // 2), (11, y // 4, x // 4), (5, y // 8, x // 8), (2, y // 8, x // 8)]
    by_shape = {l.in_shape: i for i, l in enumerate(S.LAYERS)}
    levels = sorted(set(l.in_shape for l in S.LAYERS), reverse=True)
    out = []
    for l in S.LAYERS:
        li = levels.index(l.in_shape)
        lo = levels.index(l.out_shape) if l.out_shape in levels else len(levels)
        out.append(S.ConvLayer(l.name, l.subm, l.cin, l.cout, l.ksize, l.stride, l.padding, shapes[li], shapes[lo]))
    return tuple(out)


def small_case(pkg, n_points=1500, seed=0x5E55D000 + 77):
    """1500 points on a 64 x 80 x 40 voxel grid, whole 14-layer stack, seeded weights and BatchNorm."""
    s = pkg.synth.Stream(seed)
    rng = (0.0, 0.0, -3.0, 3.2, 4.0, 1.0)
    u = s.uniform(3 * n_points)
    pts = np.empty((n_points, 4), np.float64)
    # a thin slanted sheet plus a blob, so that neighbourhoods are populated
    pts[:, 0] = u[0::3] * 3.2
    pts[:, 1] = u[1::3] * 4.0
    pts[:, 2] = -1.7 + 0.3 * (u[2::3] - 0.5) + 0.1 * pts[:, 0]
    blob = slice(0, n_points // 3)
    pts[blob, 0] = 1.0 + 0.6 * u[0::3][blob]
    pts[blob, 1] = 2.0 + 0.5 * u[1::3][blob]
    pts[blob, 2] = -1.2 + 1.0 * u[2::3][blob]
    pts[:, 3] = s.uniform(n_points)
    pts = pts[s.permutation(n_points)].astype(np.float32)
    layers = small_layers(pkg)
    w, sc, sh = pkg.random_weights(seed=seed + 1, layers=layers)
    return dict(points=np.ascontiguousarray(pts), range=rng, voxel=pkg.synth.VOXEL_SIZE, max_voxels=4096,
                layers=layers, weights=w, scale=sc, shift=sh, bev=(64, 2, 10, 8))
