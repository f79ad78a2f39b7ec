"""Seeded synthetic inputs for the sparse 3D front end.

The reference loops over KITTI "velodyne_reduced" lidar frames
(se-ssd-ai-trt.cpp:1824, loader at :1515-1559: float32 x, y, z, intensity). Those frames
are not redistributable inside this package, so the benchmark and the tests use point
clouds drawn here with the same ranges, sizes and a similar spatial distribution
(a ground sheet whose density falls as 1/r^2 plus box-shaped object clusters).

All randomness comes from one counter-based generator (splitmix64), so a frame is a pure
function of its seed and can be regenerated bit-identically by any language:
    z_i   = seed + (i + 1) * 0x9E3779B97F4A7C15                  (mod 2^64)
    z_i   = (z_i ^ (z_i >> 30)) * 0xBF58476D1CE4E5B9
    z_i   = (z_i ^ (z_i >> 27)) * 0x94D049BB133111EB
    out_i = z_i ^ (z_i >> 31);  U_i = (out_i >> 11) * 2^-53
Normals use Box-Muller on consecutive pairs: sqrt(-2 ln(1 - U_a)) * cos(2 pi U_b).
"""
from __future__ import annotations

import numpy as np

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)

SEED_BASE = 0x5E55D000

# Geometry of the reference (params.h:27-35).
POINT_RANGE = (0.0, -40.0, -3.0, 70.4, 40.0, 1.0)  # xmin, ymin, zmin, xmax, ymax, zmax
VOXEL_SIZE = (0.05, 0.05, 0.1)
GRID_ZYX = (41, 1600, 1408)


class Stream:
    """Sequential view of the splitmix64 counter stream for one seed."""

    def __init__(self, seed: int):
        self.seed = np.uint64(seed & 0xFFFFFFFFFFFFFFFF)
        self.pos = 0

    def bits(self, n: int) -> np.ndarray:
        with np.errstate(over="ignore"):
            idx = np.arange(self.pos + 1, self.pos + n + 1, dtype=np.uint64)
            z = self.seed + idx * _GAMMA
            z = (z ^ (z >> np.uint64(30))) * _M1
            z = (z ^ (z >> np.uint64(27))) * _M2
            z = z ^ (z >> np.uint64(31))
        self.pos += n
        return z

    def uniform(self, n: int) -> np.ndarray:
        return (self.bits(n) >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)

    def normal(self, n: int) -> np.ndarray:
        u = self.uniform(2 * n)
        return np.sqrt(-2.0 * np.log1p(-u[0::2])) * np.cos(2.0 * np.pi * u[1::2])

    def integers(self, n: int, hi: int) -> np.ndarray:
        return np.minimum((self.uniform(n) * hi).astype(np.int64), hi - 1)

    def permutation(self, n: int) -> np.ndarray:
        return np.argsort(self.bits(n), kind="stable")


def lidar_frame(seed: int, n_points: int = 20000, n_boxes: int = 15, ground_frac: float = 0.65) -> np.ndarray:
    """One synthetic frame, float32 [n_points, 4] = (x, y, z, intensity).

    ground_frac of the points lie on a ground sheet z = -1.7 + N(0, 0.05) whose radial density
    falls as 1/r^2 on r in [2, 80] m inside a +-49 degree sector (points outside the x/y range
    are redrawn); the rest are uniform inside n_boxes axis-aligned 4 x 1.8 x 1.6 m boxes with
    random centres (z centre -0.9). Row order is shuffled. 20,000 points / 15 boxes is the
    single-frame case, 120,000 / 40 the dense 64-beam-like case.
    """
    s = Stream(seed)
    xmin, ymin, zmin, xmax, ymax, zmax = POINT_RANGE
    n_ground = int(round(ground_frac * n_points))
    n_obj = n_points - n_ground
    gx = np.empty(0)
    gy = np.empty(0)
    rmin, rmax, half_sector = 2.0, 80.0, np.deg2rad(49.0)
    while gx.size < n_ground:
        m = 2 * (n_ground - gx.size) + 64
        u = s.uniform(2 * m)
        r = 1.0 / (1.0 / rmin - u[0::2] * (1.0 / rmin - 1.0 / rmax))
        az = (2.0 * u[1::2] - 1.0) * half_sector
        x, y = r * np.cos(az), r * np.sin(az)
        ok = (x >= xmin) & (x < xmax - 1e-3) & (y >= ymin) & (y < ymax - 1e-3)
        gx = np.concatenate([gx, x[ok]])
        gy = np.concatenate([gy, y[ok]])
    gx, gy = gx[:n_ground], gy[:n_ground]
    gz = -1.7 + 0.05 * s.normal(n_ground)
    cu = s.uniform(2 * n_boxes)
    cx = xmin + 2.5 + cu[0::2] * (xmax - xmin - 5.0)
    cy = ymin + 1.5 + cu[1::2] * (ymax - ymin - 3.0)
    which = s.integers(n_obj, n_boxes)
    u = s.uniform(3 * n_obj)
    ox = cx[which] + (u[0::3] - 0.5) * 4.0
    oy = cy[which] + (u[1::3] - 0.5) * 1.8
    oz = -0.9 + (u[2::3] - 0.5) * 1.6
    pts = np.empty((n_points, 4), dtype=np.float64)
    pts[:n_ground, 0], pts[:n_ground, 1], pts[:n_ground, 2] = gx, gy, gz
    pts[n_ground:, 0], pts[n_ground:, 1], pts[n_ground:, 2] = ox, oy, oz
    pts[:, 2] = np.clip(pts[:, 2], zmin + 1e-3, zmax - 1e-3)
    pts[:, 3] = s.uniform(n_points)
    pts = pts[s.permutation(n_points)]
    return np.ascontiguousarray(pts.astype(np.float32))


def sweep_frame(frame_index: int, n_points: int = 120000) -> np.ndarray:
    """Frame `frame_index` of the throughput sweep: 120,000 points, 40 object clusters."""
    return lidar_frame(SEED_BASE + 5 + 1000 * (frame_index + 1), n_points=n_points, n_boxes=40)


def single_frame() -> np.ndarray:
    """The 20,000-point frame of the voxelisation / backbone single-frame cases."""
    return lidar_frame(SEED_BASE + 2, n_points=20000, n_boxes=15)


def active_voxels(seed: int = SEED_BASE + 1, n: int = 16000, grid_zyx=GRID_ZYX, n_boxes: int = 30) -> np.ndarray:
    """`n` unique active voxel coordinates, int32 [n, 4] = (0, z, y, x), for single-layer cases.

    60 % on a ground sheet (z index 15..17, x density proportional to 1/(1 + x/200), y uniform),
    40 % inside n_boxes axis-aligned clusters of about 40 x 20 x 15 (x, y, z) voxels. Duplicates are
    redrawn; row order is shuffled.
    """
    s = Stream(seed)
    Z, Y, X = grid_zyx
    n_ground = int(round(0.6 * n))
    keys: list[np.ndarray] = []
    have = np.empty(0, dtype=np.int64)

    def add(z, y, x, limit):
        nonlocal have
        k = (z.astype(np.int64) * Y + y) * X + x
        _, first = np.unique(k, return_index=True)
        k = k[np.sort(first)]
        k = k[~np.isin(k, have)][:limit]
        have = np.concatenate([have, k])
        return k.size

    got = 0
    while got < n_ground:
        m = 2 * (n_ground - got) + 64
        u = s.uniform(3 * m)
        x = np.minimum((200.0 * np.expm1(u[0::3] * np.log1p(X / 200.0))).astype(np.int64), X - 1)
        y = np.minimum((u[1::3] * Y).astype(np.int64), Y - 1)
        z = 15 + np.minimum((u[2::3] * 3).astype(np.int64), 2)
        z = np.minimum(z, Z - 1)
        got += add(z, y, x, n_ground - got)
    bx, by, bz = min(40, X), min(20, Y), min(15, Z)
    cu = s.uniform(3 * n_boxes)
    ox = (cu[0::3] * (X - bx + 1)).astype(np.int64)
    oy = (cu[1::3] * (Y - by + 1)).astype(np.int64)
    oz = (cu[2::3] * (Z - bz + 1)).astype(np.int64)
    while got < n:
        m = 2 * (n - got) + 64
        which = s.integers(m, n_boxes)
        u = s.uniform(3 * m)
        x = ox[which] + np.minimum((u[0::3] * bx).astype(np.int64), bx - 1)
        y = oy[which] + np.minimum((u[1::3] * by).astype(np.int64), by - 1)
        z = oz[which] + np.minimum((u[2::3] * bz).astype(np.int64), bz - 1)
        got += add(z, y, x, n - got)
    k = have[s.permutation(n)]
    out = np.zeros((n, 4), dtype=np.int32)
    out[:, 1] = k // (Y * X)
    out[:, 2] = (k // X) % Y
    out[:, 3] = k % X
    return out


def normal_f32(seed: int, shape, std: float = 1.0) -> np.ndarray:
    """N(0, std) float32 array of `shape` from the stream of `seed`."""
    n = int(np.prod(shape))
    return (Stream(seed).normal(n) * std).astype(np.float32).reshape(shape)
