/*
 * sessd_params.h - the network constants of the SE-SSD sparse front end for C and C++ hosts.
 *
 * The reference keeps its configuration as preprocessor constants (params.h:19-36 voxel geometry,
 * :39-197 one block per sparse layer, :194-203 BEV map and zero border, :357-373 post-processing) and
 * wires them layer by layer in se-ssd-ai-trt.cpp:1147-1252. This header provides the same names with
 * the same values, so that host code written against the reference compiles unchanged, plus what the
 * reference spreads over its wiring code: the 14-layer schedule as one table of sessd_conv_params
 * (ready for sessd_backbone_create / sessd_backbone_create_from_wts) and the module indices of the
 * layers inside `backbone.middle_conv`.
 *
 * The per-layer names (SUBM_<i>_IN_CHANNEL, SPARSE_<i>_KSIZE_0, ...) are enumeration constants
 * generated from the two layer lists below; the floating-point constants are macros. Axis order:
 * KSIZE_0/1/2, STRIDE_0/1/2, PADDING_0/1/2 are (z, y, x), as the reference passes them to
 * SparseConv3dLayerPlugin (se-ssd-ai-trt.cpp:1161-1170).
 */
#ifndef SESSD_PARAMS_H_
#define SESSD_PARAMS_H_

#include "sessd.h"

/* ---- capacities and voxel geometry (params.h:19-36) ---------------------------------------- */
#define MAX_VOXELS 60000
#define MAX_POINTS 80000
#define MAX_POINTS_PER_VOXEL 5
#define MAX_NUM_POINTS_PER_VOXEL 5
#define VOXEL_FEATURE_NUM 4
#define VOXEL_SIZE_X 0.05
#define VOXEL_SIZE_Y 0.05
#define VOXEL_SIZE_Z 0.1
#define X_MIN 0.0
#define X_MAX 70.4
#define Y_MIN -40.0
#define Y_MAX 40.0
#define Z_MIN -3.0
#define Z_MAX 1.0

/* ---- the sparse layers (params.h:39-192) ---------------------------------------------------
 * Submanifold layers: X(module index, Cin, Cout, grid x, grid y, grid z); kernel 3x3x3, stride 1,
 * padding 1, dilation 1 are fixed by the wiring code (se-ssd-ai-trt.cpp:701-705).
 * Strided layers: X(module index, Cin, Cout, out x, y, z, in x, y, z, kz, ky, kx, sz, sy, sx, pz, py, px). */
#define SESSD_SUBM_LAYERS(X)          \
    X(0, 4, 16, 1408, 1600, 41)       \
    X(3, 16, 16, 1408, 1600, 41)      \
    X(9, 32, 32, 704, 800, 21)        \
    X(12, 32, 32, 704, 800, 21)       \
    X(18, 64, 64, 352, 400, 11)       \
    X(21, 64, 64, 352, 400, 11)       \
    X(24, 64, 64, 352, 400, 11)       \
    X(30, 64, 64, 176, 200, 5)        \
    X(33, 64, 64, 176, 200, 5)        \
    X(36, 64, 64, 176, 200, 5)

#define SESSD_SPARSE_LAYERS(X)                                              \
    X(6, 16, 32, 704, 800, 21, 1408, 1600, 41, 3, 3, 3, 2, 2, 2, 1, 1, 1)   \
    X(15, 32, 64, 352, 400, 11, 704, 800, 21, 3, 3, 3, 2, 2, 2, 1, 1, 1)    \
    X(27, 64, 64, 176, 200, 5, 352, 400, 11, 3, 3, 3, 2, 2, 2, 0, 1, 1)     \
    X(39, 64, 64, 176, 200, 2, 176, 200, 5, 3, 1, 1, 2, 1, 1, 0, 0, 0)

#define SESSD_SUBM_NAMES(i, ci, co, x, y, z)                                                     \
    SUBM_##i##_MAX_VOXELS = MAX_VOXELS, SUBM_##i##_IN_CHANNEL = ci, SUBM_##i##_OUT_CHANNEL = co, \
    SUBM_##i##_OUT_SHAPE_X = x, SUBM_##i##_OUT_SHAPE_Y = y, SUBM_##i##_OUT_SHAPE_Z = z,
#define SESSD_SPARSE_NAMES(i, ci, co, ox, oy, oz, ix, iy, iz, k0, k1, k2, s0, s1, s2, p0, p1, p2)               \
    SPARSE_##i##_MAX_VOXELS = MAX_VOXELS, SPARSE_##i##_IN_CHANNEL = ci, SPARSE_##i##_OUT_CHANNEL = co,          \
    SPARSE_##i##_OUT_SHAPE_X = ox, SPARSE_##i##_OUT_SHAPE_Y = oy, SPARSE_##i##_OUT_SHAPE_Z = oz,                \
    SPARSE_##i##_SPATIAL_SHAPE_X = ix, SPARSE_##i##_SPATIAL_SHAPE_Y = iy, SPARSE_##i##_SPATIAL_SHAPE_Z = iz,    \
    SPARSE_##i##_KSIZE_0 = k0, SPARSE_##i##_KSIZE_1 = k1, SPARSE_##i##_KSIZE_2 = k2,                            \
    SPARSE_##i##_STRIDE_0 = s0, SPARSE_##i##_STRIDE_1 = s1, SPARSE_##i##_STRIDE_2 = s2,                         \
    SPARSE_##i##_PADDING_0 = p0, SPARSE_##i##_PADDING_1 = p1, SPARSE_##i##_PADDING_2 = p2,

enum sessd_layer_constants {
    SESSD_SUBM_LAYERS(SESSD_SUBM_NAMES)
    SESSD_SPARSE_LAYERS(SESSD_SPARSE_NAMES)
    SESSD_NUM_LAYERS = 14
};

/* ---- BEV map, zero border (params.h:194-203) ------------------------------------------------ */
#define BACKBONE_FEATURE_MAP_SIZE_X 176
#define BACKBONE_FEATURE_MAP_SIZE_Y 200
#define BACKBONE_FEATURE_MAP_SIZE_Z 2
#define BACKBONE_FEATURE_MAP_CHANNEL 64
#define ZERO_PADDING_2D_TOP 1
#define ZERO_PADDING_2D_BOTTOM 1
#define ZERO_PADDING_2D_LEFT 1
#define ZERO_PADDING_2D_RIGHT 1

/* ---- anchors, score filter, NMS (params.h:357-373) ------------------------------------------ */
#define FEATURE_MAP_HEIGHT 200
#define FEATURE_MAP_WIDTH 176
#define DIRECTION_ANGLE_0 0.0
#define DIRECTION_ANGLE_1 1.57
#define DIRECTION_ANGLE_NUM 2
#define CAR_LENGTH 3.9
#define CAR_WIDTH 1.6
#define CAR_HEIGHT 1.56
#define MAX_BOX_NUM 500
#define SCORE_THRESHOLD 0.45
#define DIRECTION_OFFSET 0.0
#define NMS_THRESH 0.01
#define LAST_DIMS 9

/* Epsilon of every BatchNorm1d after a sparse layer (se-ssd-ai-trt.cpp:1151). */
#define SESSD_BATCHNORM_EPS 1e-5f

/* ---- the schedule as data --------------------------------------------------------------------
 * Layer l of the table is module sessd_layer_module_index[l] of `backbone.middle_conv`; its batch norm is
 * module index + 1 (se-ssd-ai-trt.cpp:1147-1249). feature_num is the plugin's fourth integer (unused by
 * the kernels, kept for the serialized blob); dilation 1 and out_padding 0 as the wiring code passes. */
#define SESSD_SUBM_ROW(i, ci, co, x, y, z) \
    {ci, co, MAX_VOXELS, 4, x, y, z, x, y, z, {3, 3, 3}, {1, 1, 1}, {1, 1, 1}, 1, 0, 1}
#define SESSD_SPARSE_ROW(i, ci, co, ox, oy, oz, ix, iy, iz, k0, k1, k2, s0, s1, s2, p0, p1, p2) \
    {ci, co, MAX_VOXELS, 4, ox, oy, oz, ix, iy, iz, {k0, k1, k2}, {s0, s1, s2}, {p0, p1, p2}, 1, 0, 0}

static const int32_t sessd_layer_module_index[SESSD_NUM_LAYERS] = {0, 3, 6, 9, 12, 15, 18, 21, 24, 27, 30, 33, 36, 39};

static const sessd_conv_params sessd_layer_schedule[SESSD_NUM_LAYERS] = {
    SESSD_SUBM_ROW(0, 4, 16, 1408, 1600, 41),
    SESSD_SUBM_ROW(3, 16, 16, 1408, 1600, 41),
    SESSD_SPARSE_ROW(6, 16, 32, 704, 800, 21, 1408, 1600, 41, 3, 3, 3, 2, 2, 2, 1, 1, 1),
    SESSD_SUBM_ROW(9, 32, 32, 704, 800, 21),
    SESSD_SUBM_ROW(12, 32, 32, 704, 800, 21),
    SESSD_SPARSE_ROW(15, 32, 64, 352, 400, 11, 704, 800, 21, 3, 3, 3, 2, 2, 2, 1, 1, 1),
    SESSD_SUBM_ROW(18, 64, 64, 352, 400, 11),
    SESSD_SUBM_ROW(21, 64, 64, 352, 400, 11),
    SESSD_SUBM_ROW(24, 64, 64, 352, 400, 11),
    SESSD_SPARSE_ROW(27, 64, 64, 176, 200, 5, 352, 400, 11, 3, 3, 3, 2, 2, 2, 0, 1, 1),
    SESSD_SUBM_ROW(30, 64, 64, 176, 200, 5),
    SESSD_SUBM_ROW(33, 64, 64, 176, 200, 5),
    SESSD_SUBM_ROW(36, 64, 64, 176, 200, 5),
    SESSD_SPARSE_ROW(39, 64, 64, 176, 200, 2, 176, 200, 5, 3, 1, 1, 2, 1, 1, 0, 0, 0),
};

/* The voxel generator's parameter block with the constants above (grid sizes are filled by
 * sessd_voxel_configure, as VoxelGeneratorPlugin::configurePlugin does, voxelGenerator.cu:228-235). */
static const sessd_voxel_params sessd_default_voxel_params = {
    MAX_VOXELS, MAX_NUM_POINTS_PER_VOXEL, VOXEL_FEATURE_NUM,
    (float)X_MIN, (float)X_MAX, (float)Y_MIN, (float)Y_MAX, (float)Z_MIN, (float)Z_MAX,
    (float)VOXEL_SIZE_X, (float)VOXEL_SIZE_Y, (float)VOXEL_SIZE_Z, 4, 0, 0, 0};

static const sessd_s2d_params sessd_default_s2d_params = {
    BACKBONE_FEATURE_MAP_SIZE_X, BACKBONE_FEATURE_MAP_SIZE_Y, BACKBONE_FEATURE_MAP_SIZE_Z, BACKBONE_FEATURE_MAP_CHANNEL};

static const sessd_pad2d_params sessd_default_pad2d_params = {
    ZERO_PADDING_2D_TOP, ZERO_PADDING_2D_BOTTOM, ZERO_PADDING_2D_LEFT, ZERO_PADDING_2D_RIGHT};

#endif /* SESSD_PARAMS_H_ */
