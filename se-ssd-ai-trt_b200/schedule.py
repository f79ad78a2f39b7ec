"""Layer schedule and geometry constants of the SE-SSD sparse front end.

Values are those of the reference's params.h (voxel geometry :19-36, per-layer shapes and
kernel/stride/padding :39-197) in the order the network wires them
(se-ssd-ai-trt.cpp:1147-1252): 14 sparse conv layers, each followed by BatchNorm1d(eps 1e-5)
and ReLU, then the sparse-to-dense BEV scatter.
"""
from __future__ import annotations

from dataclasses import dataclass

MAX_VOXELS = 60000            # params.h:19
MAX_POINTS = 80000            # params.h:20
MAX_POINTS_PER_VOXEL = 5      # params.h:21
VOXEL_FEATURE_NUM = 4         # params.h:36
BN_EPS = 1e-5                 # se-ssd-ai-trt.cpp:1151

BACKBONE_FEATURE_MAP_SIZE_X = 176   # params.h:194
BACKBONE_FEATURE_MAP_SIZE_Y = 200   # params.h:195
BACKBONE_FEATURE_MAP_SIZE_Z = 2     # params.h:196
BACKBONE_FEATURE_MAP_CHANNEL = 64   # params.h:197

# Detection post-processing (anchor decode + score filter), params.h:357-368
FEATURE_MAP_HEIGHT = 200
FEATURE_MAP_WIDTH = 176
DIRECTION_ANGLES = (0.0, 1.57)
CAR_SIZE = (3.9, 1.6, 1.56)         # length, width, height
MAX_BOX_NUM = 500
SCORE_THRESHOLD = 0.45
DIRECTION_OFFSET = 0.0
NMS_THRESH = 0.01                    # params.h:373


@dataclass(frozen=True)
class ConvLayer:
    name: str          # reference layer index in backbone.middle_conv
    subm: bool
    cin: int
    cout: int
    ksize: tuple       # (z, y, x)
    stride: tuple
    padding: tuple
    in_shape: tuple    # (Z, Y, X) of the input grid
    out_shape: tuple   # (Z, Y, X) of the output grid

    @property
    def kvol(self) -> int:
        return self.ksize[0] * self.ksize[1] * self.ksize[2]

    def as_ints(self):
        """The 16-int layer record used by the C entry points."""
        return [int(self.subm), self.cin, self.cout, *self.ksize, *self.stride, *self.padding,
                *self.out_shape, 0]


def _subm(name, cin, cout, shape):
    return ConvLayer(name, True, cin, cout, (3, 3, 3), (1, 1, 1), (1, 1, 1), shape, shape)


_R0 = (41, 1600, 1408)
_R1 = (21, 800, 704)
_R2 = (11, 400, 352)
_R3 = (5, 200, 176)
_R4 = (2, 200, 176)

LAYERS = (
    _subm("subm0", 4, 16, _R0),
    _subm("subm3", 16, 16, _R0),
    ConvLayer("sparse6", False, 16, 32, (3, 3, 3), (2, 2, 2), (1, 1, 1), _R0, _R1),
    _subm("subm9", 32, 32, _R1),
    _subm("subm12", 32, 32, _R1),
    ConvLayer("sparse15", False, 32, 64, (3, 3, 3), (2, 2, 2), (1, 1, 1), _R1, _R2),
    _subm("subm18", 64, 64, _R2),
    _subm("subm21", 64, 64, _R2),
    _subm("subm24", 64, 64, _R2),
    ConvLayer("sparse27", False, 64, 64, (3, 3, 3), (2, 2, 2), (0, 1, 1), _R2, _R3),
    _subm("subm30", 64, 64, _R3),
    _subm("subm33", 64, 64, _R3),
    _subm("subm36", 64, 64, _R3),
    ConvLayer("sparse39", False, 64, 64, (3, 1, 1), (2, 1, 1), (0, 0, 0), _R3, _R4),
)


def weight_count(layers=LAYERS) -> int:
    return sum(l.kvol * l.cin * l.cout for l in layers)


def channel_count(layers=LAYERS) -> int:
    return sum(l.cout for l in layers)
