/*
 * sessd.h - C ABI of the B200 (sm_100a) sparse 3D front end for SE-SSD.
 *
 * Every entry point replaces one piece of the reference's TensorRT plugin code; the
 * reference location is cited at each declaration (paths are relative to the reference
 * project root). Conventions shared by all entry points:
 *
 *   - plain C types only; device buffers are raw pointers, `stream` is a cudaStream_t passed
 *     as void*; nothing is allocated or freed inside an *_enqueue call and nothing blocks
 *     (the reference's enqueue() has the same contract, e.g. submConv3dlayer.cu:539-641);
 *   - tensors use the reference's layouts (row-major, batch outermost):
 *       points      f32 [B][max_points][4]      (x, y, z, intensity)   voxelGenerator.cu:361
 *       points_size i32 [B]
 *       features    f32|f16 [B][max_voxels][C]
 *       coors       i32 [B][max_voxels][4]      (b, z, y, x)           voxelGenerator.cu:404
 *       voxel_num   i32 [B]
 *       dense       f32|f16 [B][C*D][H][W]                             sparse2Dense.cu:201-206
 *     rows at index >= voxel_num[b] of an output are zero, as the reference leaves them;
 *   - the reference runs batch 1 only (se-ssd-ai-trt.cpp:1125); B > 1 processes B independent
 *     frames in one call, frame b using rows [b][...] of every tensor;
 *   - return value: SESSD_OK (0) or a negative sessd_error. The reference aborts the process on
 *     any CUDA error (voxelGenerator.cu:8-19); this library never aborts;
 *   - conditions only the device can see (capacity overflows) are reported as bits OR-ed into
 *     the int32 status word that occupies the first 4 bytes of the caller's workspace (the first
 *     1024 bytes of every workspace are reserved for it and for counters); it is
 *     cleared at the start of every *_enqueue and may be read after the stream has been
 *     synchronised (sessd_read_status does the copy);
 *   - a workspace must start on a 256-byte boundary (cudaMalloc and TensorRT workspaces do); an *_enqueue
 *     given one that does not returns SESSD_ERR_PARAM.
 */
#ifndef SESSD_H_
#define SESSD_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SESSD_OK 0
typedef enum sessd_error {
    SESSD_ERR_NULL = -1,        /* a required pointer is null */
    SESSD_ERR_PARAM = -2,       /* a parameter is out of its supported range */
    SESSD_ERR_WORKSPACE = -3,   /* workspace_bytes is smaller than *_workspace_bytes() */
    SESSD_ERR_CUDA = -4,        /* a CUDA runtime call failed; see sessd_last_cuda_error() */
    SESSD_ERR_UNSUPPORTED = -5, /* channel count / dtype combination has no kernel */
    SESSD_ERR_IO = -6           /* a file could not be opened, read or written, or is malformed */
} sessd_error;

/* Bits of the device status word. */
#define SESSD_STATUS_VOXEL_OVERFLOW 1 /* more voxels / active outputs than max_voxels; extra ones dropped */
#define SESSD_STATUS_HASH_FULL 2      /* a coordinate table ran out of probes; entry dropped */
#define SESSD_STATUS_PAIR_OVERFLOW 4  /* a rulebook column exceeded max_voxels entries on export */
#define SESSD_STATUS_BAD_COORD 8      /* an input coordinate lies outside the declared grid; row ignored */
#define SESSD_STATUS_TIMEOUT 16       /* a bounded wait inside a kernel gave up; the call's outputs are invalid */
#define SESSD_STATUS_BOX_OVERFLOW 32  /* more boxes passed the score filter than max_box_num; extra ones dropped */

typedef enum sessd_dtype { SESSD_F32 = 0, SESSD_F16 = 1 } sessd_dtype;

/* ------------------------------------------------------------------------------------------
 * Voxel generator.  Replaces VoxelGeneratorPlugin (voxelGenerator.h:19-110).
 * The struct is the plugin's serialized blob, field for field (voxelGenerator.cu:576-600).
 * ---------------------------------------------------------------------------------------- */
typedef struct sessd_voxel_params {
    int32_t max_voxels;            /* voxelNum_   */
    int32_t max_points_per_voxel;  /* pointNum_   (<= 8) */
    int32_t voxel_feature_num;     /* featureNum_ (4)   */
    float x_min, x_max, y_min, y_max, z_min, z_max;
    float voxel_x, voxel_y, voxel_z;
    int32_t point_feature_num;     /* 4 */
    int32_t grid_x, grid_y, grid_z;
} sessd_voxel_params;

/* Fills grid_x/y/z = np_round((max - min) / voxel) in fp32.
 * Replaces VoxelGeneratorPlugin::configurePlugin (voxelGenerator.cu:228-235) and np_round (:61-68). */
int sessd_voxel_configure(sessd_voxel_params* p);

/* Replaces VoxelGeneratorPlugin::getWorkspaceSize (voxelGenerator.cu:237-252). */
size_t sessd_voxelize_workspace_bytes(const sessd_voxel_params* p, int batch, int max_points);

/* Replaces VoxelGeneratorPlugin::enqueue (voxelGenerator.cu:480-542) with its two kernels
 * generateVoxels_kernel (:348-451) and generateAverage_kernel (:255-321).
 * inputs  = { points f32 [B][max_points][4], points_size i32 [B] }
 * outputs = { voxels [B][max_voxels][4] (out_dtype), coors i32 [B][max_voxels][4], voxel_num i32 [B] }
 * Voxel rows are numbered by their lowest point index; a voxel averages its
 * max_points_per_voxel lowest-indexed points. */
int sessd_voxelize_enqueue(const sessd_voxel_params* p, int batch, int max_points, int out_dtype,
                           const void* const* inputs, void* const* outputs,
                           void* workspace, size_t workspace_bytes, void* stream);

/* Device pointer (inside `workspace`) to the clamped per-voxel point counts, i32 [B][max_voxels],
 * valid after sessd_voxelize_enqueue. The reference keeps the same array in its workspace
 * (num_points_per_voxel, voxelGenerator.cu:507-509). */
void* sessd_voxelize_num_points(const sessd_voxel_params* p, int batch, int max_points, void* workspace);

/* Voxel generator for callers that cannot allocate: same inputs, outputs and results as
 * sessd_voxelize_enqueue, but the scratch memory is a 4 MiB device array built into the library instead
 * of a caller workspace, and the call performs no cudaMalloc / cudaFree or any other allocation. It is
 * meant for hosts whose device memory is fixed before this library runs (a pre-sized plugin arena, a
 * real-time loop that may not touch the allocator). This entry point has no counterpart in the reference,
 * whose plugins always receive a TensorRT workspace.
 * Limits and rules:
 *   - batch, max_points and p->max_voxels must fit the built-in scratch (e.g. one frame of up to 32768
 *     points with max_voxels <= 32768); larger requests return SESSD_ERR_WORKSPACE and
 *     sessd_last_cuda_error() explains why;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress); make
 *     that first call outside any stream capture;
 *   - all calls on one device share the array: it keeps the previous call's contents (each call resets
 *     what it needs), and two calls that overlap on the GPU (different streams) race. Serialise them;
 *   - the device status word lives inside the array; sessd_voxelize_static_status() reads it (a full frame and a
 *     frame that lost voxels both end with voxel_num[b] == p->max_voxels, only the status bit tells them apart);
 *   - the looked-up address is kept per device ordinal for the life of the process: after cudaDeviceReset (or
 *     any other destruction of the device's primary context) the library must not be used again without being
 *     reloaded. */
int sessd_voxelize_enqueue_static(const sessd_voxel_params* p, int batch, int max_points, int out_dtype,
                                  const void* const* inputs, void* const* outputs, void* stream);
/* Status word left by the last sessd_voxelize_enqueue_static call on the current device: synchronises `stream`
 * and returns the word (>= 0, SESSD_STATUS_* bits) or a negative sessd_error (SESSD_ERR_PARAM before the first
 * call on this device). Allocates nothing. Like the entry point it serves, it has no counterpart in the reference. */
int sessd_voxelize_static_status(void* stream);

/* ------------------------------------------------------------------------------------------
 * Sparse convolutions.  Replace SubmConv3dLayerPlugin (submConv3dlayer.h:19-121) and
 * SparseConv3dLayerPlugin (sparseConv3dlayer.h:18-126). The struct holds the integer lists both
 * plugins serialize (submConv3dlayer.cu:684-714, sparseConv3dlayer.cu:863-899); ksize/stride/padding
 * are (z, y, x) triples = the reference's ksize0..2.
 * ---------------------------------------------------------------------------------------- */
typedef struct sessd_conv_params {
    int32_t in_channel, out_channel, max_voxels, feature_num;
    int32_t out_shape_x, out_shape_y, out_shape_z;
    int32_t spatial_shape_x, spatial_shape_y, spatial_shape_z;
    int32_t ksize[3], stride[3], padding[3];
    int32_t dilation, out_padding;
    int32_t subm; /* 1: submanifold (outputs = inputs); 0: strided, outputs = union of candidates */
} sessd_conv_params;

/* Device-resident weights of one layer, repacked for the kernels. */
typedef struct sessd_conv_weights sessd_conv_weights;

/* Uploads weights f32 [kvol][Cin][Cout] (host pointer, the layout of submConv3dlayer.cu:510).
 * Replaces the cudaMalloc + cudaMemcpy in the plugin constructors (submConv3dlayer.cu:146-150,
 * sparseConv3dlayer.cu:157-161). scale/shift (host f32 [Cout], may be null) and relu fold the
 * BatchNorm1d + ReLU the reference inserts after every layer (se-ssd-ai-trt.cpp:808-856) into the
 * kernel epilogue: y = max(0, x*scale + shift); with null/null/0 the layer is the bare plugin. */
int sessd_conv_weights_create(const sessd_conv_params* p, const float* weights, const float* scale,
                              const float* shift, int relu, int dtype, sessd_conv_weights** out);
/* Replaces SubmConv3dLayerPlugin::terminate (submConv3dlayer.cu:671-677). */
void sessd_conv_weights_destroy(sessd_conv_weights* w);

/* Replaces getWorkspaceSize (submConv3dlayer.cu:247-267, sparseConv3dlayer.cu:286-306). */
size_t sessd_conv_workspace_bytes(const sessd_conv_params* p, int batch);

/* Replaces SubmConv3dLayerPlugin::enqueue (submConv3dlayer.cu:539-641): rulebook kernels
 * prepareSubMGridKernel (:441-459), getValidOutPosKernel (:271-358), getSubMIndicePairsKernel
 * (:376-424) and the 27 sparseGatherConvScatter launches (:479-518, :632-638).
 * inputs = { features [B][max_voxels][Cin], coors, voxel_num }, outputs = { features [B][max_voxels][Cout] } */
int sessd_subm_conv_enqueue(const sessd_conv_params* p, const sessd_conv_weights* w, int batch,
                            const void* const* inputs, void* const* outputs,
                            void* workspace, size_t workspace_bytes, void* stream);

/* Replaces SparseConv3dLayerPlugin::enqueue (sparseConv3dlayer.cu:606-813): getValidOutPosKernel
 * (:310-386), fillGridKernel1/2 (:475-541), getSparseIndicePairsKernel (:405-454) and the per-offset
 * sparseGatherConvScatter launches (:557-589, :804-809).
 * outputs = { features [B][max_voxels][Cout], coors i32 [B][max_voxels][4], voxel_num i32 [B] }.
 * Output rows are numbered in the order a sequential pass over (input row, candidate) first meets
 * them (the rule of the host loop kept in comments at sparseConv3dlayer.cu:738-757). */
int sessd_sparse_conv_enqueue(const sessd_conv_params* p, const sessd_conv_weights* w, int batch,
                              const void* const* inputs, void* const* outputs,
                              void* workspace, size_t workspace_bytes, void* stream);

/* Writes the rulebook of the last *_conv_enqueue that used `workspace`, for frame `frame`, in the
 * reference's own layout: indice_pairs i32 [kvol][2][max_voxels] (input row, output row; -1 unused) and
 * indice_num u32 [kvol] (submConv3dlayer.cu:254-255, :413-419). Both are device pointers, as is
 * out_voxel_num (i32 [B]: the layer's output row counts, i.e. the input voxel_num for a submanifold
 * layer and outputs[2] for a strided one). Within one offset, pairs are ordered by output row. Used by the parity tests; the kernels themselves work from
 * an output-stationary neighbour map and never build this list. */
int sessd_conv_rulebook_export(const sessd_conv_params* p, int batch, int frame, void* workspace,
                               int32_t* indice_pairs, uint32_t* indice_num, void* stream,
                               const void* out_voxel_num);

/* ------------------------------------------------------------------------------------------
 * Sparse -> dense BEV.  Replaces Sparse2DensePlugin (sparse2Dense.h:18-86); the struct is its
 * serialized blob (sparse2Dense.cu:283-295).
 * ---------------------------------------------------------------------------------------- */
typedef struct sessd_s2d_params {
    int32_t feature_map_size_x, feature_map_size_y, feature_map_size_z, feature_map_channel;
} sessd_s2d_params;

/* Replaces Sparse2DensePlugin::enqueue (sparse2Dense.cu:224-249) and sparse2dense_kernel (:182-207).
 * inputs = { features [B][max_voxels][C], coors, voxel_num }, outputs = { dense [B][C*D][H][W] }.
 * Needs no workspace beyond the 256-byte status block (workspace may be null: then no status). */
int sessd_sparse2dense_enqueue(const sessd_s2d_params* p, int batch, int max_voxels, int dtype,
                               const void* const* inputs, void* const* outputs,
                               void* workspace, size_t workspace_bytes, void* stream);

/* ZeroPad2dPlugin (zeroPad2d.h:18-87); the struct is its serialized blob (zeroPad2d.cu:286-289). */
typedef struct sessd_pad2d_params {
    int32_t top, bottom, left, right;
} sessd_pad2d_params;

/* Replaces ZeroPad2dPlugin::enqueue (zeroPad2d.cu:219-246) and zero_padding2d_kernel (:183-200):
 * inputs = { map [B][C][H][W] }, outputs = { map [B][C][top+H+bottom][left+W+right] }, zero border.
 * (The reference kernel indexes one frame only; here every frame of the batch is padded.) */
int sessd_zero_pad2d_enqueue(const sessd_pad2d_params* pad, int batch, int channels, int height, int width, int dtype,
                             const void* const* inputs, void* const* outputs, void* stream);

/* Sparse2DensePlugin followed by ZeroPad2dPlugin in one pass (the pair wired at se-ssd-ai-trt.cpp:1251-1253):
 * outputs = { dense [B][C*D][top+H+bottom][left+W+right] }, row i of the features lands at channel c*D+z,
 * pixel (top + y, left + x); saves the intermediate map, its memset and the copy. */
int sessd_sparse2dense_padded_enqueue(const sessd_s2d_params* p, const sessd_pad2d_params* pad, int batch,
                                      int max_voxels, int dtype, const void* const* inputs, void* const* outputs,
                                      void* stream);

/* ------------------------------------------------------------------------------------------
 * Whole front end: voxelise -> conv stack (BN + ReLU folded) -> dense BEV, the layer sequence
 * wired at se-ssd-ai-trt.cpp:1138-1252, as one call. Coordinate tables and neighbour maps are built
 * once per resolution and shared by the layers that use them (the reference rebuilds the rulebook
 * inside every plugin call).
 * ---------------------------------------------------------------------------------------- */
typedef struct sessd_backbone sessd_backbone;

/* weights[l] / scale[l] / shift[l]: host pointers per layer, as for sessd_conv_weights_create. */
int sessd_backbone_create(const sessd_voxel_params* vp, const sessd_conv_params* layers, int nlayers,
                          const float* const* weights, const float* const* scale, const float* const* shift,
                          const sessd_s2d_params* s2d, int dtype, sessd_backbone** out);
void sessd_backbone_destroy(sessd_backbone* bb);
size_t sessd_backbone_workspace_bytes(const sessd_backbone* bb, int batch, int max_points);

/* points f32 [B][max_points][4], points_size i32 [B] -> dense [B][C*D][H][W] (all device pointers).
 * Replaces the sparse part of one IExecutionContext::enqueueV2 call (se-ssd-ai-trt.cpp:1868). */
int sessd_backbone_enqueue(const sessd_backbone* bb, int batch, int max_points,
                           const void* points, const void* points_size, void* dense,
                           void* workspace, size_t workspace_bytes, void* stream);

/* Folds the reference's ZeroPad2dPlugin into the backbone's dense output: after this call
 * sessd_backbone_enqueue writes dense [B][C*D][top+H+bottom][left+W+right]. Call before creating pipelines. */
int sessd_backbone_set_padding(sessd_backbone* bb, const sessd_pad2d_params* pad);

/* Same work as sessd_backbone_enqueue, plus a count of the rulebook pairs of every layer (the P of the
 * flop count 2*P*Cin*Cout), copied to host_counts[nlayers] after synchronising the stream. For benchmarks
 * and tests; the reference exposes the same numbers as indice_num (submConv3dlayer.cu:413). */
int sessd_backbone_pair_counts(const sessd_backbone* bb, int batch, int max_points,
                               const void* points, const void* points_size, void* dense,
                               void* workspace, size_t workspace_bytes, void* stream, int64_t* host_counts);

/* Device pointers (inside `workspace`) to what layer `layer` produced in the last enqueue:
 * features [B][max_voxels][Cout], coors, voxel_num. layer = -1 selects the voxeliser's outputs. */
int sessd_backbone_layer_view(const sessd_backbone* bb, int batch, int max_points, void* workspace, int layer,
                              void** features, void** coors, void** voxel_num);

/* Host-buffer variant used for end-to-end timing: copies `nframes` frames of points from (ideally
 * pinned) host memory, runs them in groups of `batch` on `nstreams` streams and copies each frame's
 * final voxel count and status word back to the host. Replaces the per-frame body of the reference's
 * inference loop (se-ssd-ai-trt.cpp:1858-1894: H2D copy, enqueueV2, D2H copy, stream sync). The dense
 * BEV map of the last group stays on the device (the reference also keeps it there for its 2D head).
 * A pipeline owns its device buffers and streams; create/destroy allocate and free them. Host-buffer runs
 * (without graph replay) copy a slot's next group in on a stream of their own while its current group
 * computes, and the BEV maps of sessd_pipeline_run_host_bev out on another: the first such run allocates a
 * second set of input (and BEV) buffers per slot for this. */
typedef struct sessd_pipeline sessd_pipeline;
int sessd_pipeline_create(const sessd_backbone* bb, int batch, int max_points, int nstreams, sessd_pipeline** out);
void sessd_pipeline_destroy(sessd_pipeline* pl);
/* host_points f32 [nframes][max_points][4], host_sizes i32 [nframes];
 * host_voxel_num i32 [nframes], host_status i32 [nframes]: the status word of the stream slot the frame's group ran
 * on, as it stood after that group. Within one run a slot's word is not cleared between groups, so it also holds
 * the conditions of the slot's earlier groups, and the words of the last group of every slot together cover the
 * whole run (a run clears them when it starts). */
int sessd_pipeline_run_host(sessd_pipeline* pl, const float* host_points, const int32_t* host_sizes, int nframes,
                            int32_t* host_voxel_num, int32_t* host_status, float* elapsed_ms);
/* The same, and every group's dense BEV maps are also copied to the host: host_dense (ideally pinned) holds
 * nstreams regions of batch maps each, [nstreams][batch][C*D][H][W] in the backbone's data type; the maps of a group
 * land in the region of the stream slot it ran on (group g uses slot g % nstreams) and are overwritten by that slot's
 * next group. The reference itself copies only the filtered boxes back (se-ssd-ai-trt.cpp:1876-1879); this variant
 * measures what it costs a host-side consumer of the map. */
int sessd_pipeline_run_host_bev(sessd_pipeline* pl, const float* host_points, const int32_t* host_sizes, int nframes,
                                int32_t* host_voxel_num, int32_t* host_status, void* host_dense, float* elapsed_ms);
/* Same work with the points already on the device: points f32 [nframes][max_points][4], sizes i32 [nframes].
 * Kernels are enqueued on the pipeline's streams; elapsed device time between the first and the last
 * stream event is returned in *elapsed_ms when it is non-null. */
int sessd_pipeline_run_device(sessd_pipeline* pl, const void* points, const void* sizes, int nframes,
                              float* elapsed_ms);
/* With enable != 0, every stream slot captures the launch sequence of one full group into a CUDA graph the second
 * time it runs one and replays it from then on (partial last groups and profiled runs use plain launches).
 * Device-resident inputs are then copied into the slot's staging buffers first. Off by default. No counterpart
 * in the reference, which launches every kernel of every frame from the host. */
int sessd_pipeline_use_graphs(sessd_pipeline* pl, int enable);
/* Dense BEV buffer / workspace of stream `s` (device pointers; dense is [batch][C*D][H][W]): the buffer the slot's
 * latest group wrote (a slot alternates between two during sessd_pipeline_run_host_bev). */
void* sessd_pipeline_dense(sessd_pipeline* pl, int s);
void* sessd_pipeline_workspace(sessd_pipeline* pl, int s);
/* Index of the last coordinate level of a backbone (number of strided layers). */
int sessd_backbone_final_level(const sessd_backbone* bb);

/* ------------------------------------------------------------------------------------------
 * Detection post-processing (the two plugins after the 2D head, se-ssd-ai-trt.cpp:1421-1461).
 * Tensors: box_preds f32 [B][N][7], cls_preds f32 [B][N][1], iou_preds f32 [B][N][1], dir_preds f32 [B][N][2],
 * N = feature_map_height * feature_map_width * direction_angle_num anchors per frame (70,400).
 * ---------------------------------------------------------------------------------------- */

/* GenerateAnchorDecodePlugin's serialized blob, field for field (generateAnchorDecode.cu:400-421; note
 * that the reference writes max_y a second time where max_z belongs, :409 - the plugin mirror repeats it). */
typedef struct sessd_anchor_params {
    float min_x, max_x, min_y, max_y, min_z, max_z;
    int32_t feature_map_height, feature_map_width;
    float car_length, car_width, car_height;
    float direction_angle_0, direction_angle_1;
    int32_t direction_angle_num;   /* 1 or 2 */
} sessd_anchor_params;

/* FilterBoxByScorePlugin's serialized blob, field for field (filterBoxByScore.cu:430-441). */
typedef struct sessd_filter_params {
    int32_t feature_map_height, feature_map_width, direction_angle_num, max_box_num;
    float score_threshold, direction_offset;
} sessd_filter_params;

/* Replaces GenerateAnchorDecodePlugin::enqueue (generateAnchorDecode.cu:331-360: memset, generate_anchor_kernel
 * :201-247, decode_kernel :268-316). inputs = { box_preds }, outputs = { boxes f32 [B][N][7] =
 * (x, y, z, w, l, h, yaw) }. No workspace (as the reference, :193-198). Anchors are computed in registers,
 * not stored. */
int sessd_anchor_decode_enqueue(const sessd_anchor_params* p, int batch, const void* const* inputs,
                                void* const* outputs, void* stream);

/* Replaces FilterBoxByScorePlugin::getWorkspaceSize (filterBoxByScore.cu:252-256, which returns 0): the ordered
 * compaction needs one counter per 256 anchors and the status block. */
size_t sessd_filter_boxes_workspace_bytes(const sessd_filter_params* p, int batch);

/* Replaces FilterBoxByScorePlugin::enqueue (filterBoxByScore.cu:339-381) and filter_box_by_score_kernel (:260-324).
 * inputs = { boxes (decoded), cls_preds, iou_preds, dir_preds },
 * outputs = { box f32 [B][max_box][9] = (x, y, z, w, l, h, yaw', 0, score), score f32 [B][max_box],
 *             iou f32 [B][max_box], direction f32 [B][max_box], valid_line_num u32 [B] }.
 * Rows are appended in ascending anchor index (the reference: arrival order of an atomic) and only the first
 * max_box_num are kept: valid_line_num = min(passed, max_box_num), SESSD_STATUS_BOX_OVERFLOW when more passed
 * (the reference writes past its outputs). Outputs are cleared first, as the reference does. */
int sessd_filter_boxes_enqueue(const sessd_filter_params* p, int batch, const void* const* inputs,
                               void* const* outputs, void* workspace, size_t workspace_bytes, void* stream);

/* Both plugins in one pass: inputs[0] holds the regression outputs (what GenerateAnchorDecodePlugin receives)
 * and only the anchors that pass the score threshold are decoded; outputs and workspace as
 * sessd_filter_boxes_enqueue. The two parameter blocks must agree on the feature map and direction count. */
int sessd_decode_filter_enqueue(const sessd_anchor_params* anchors, const sessd_filter_params* p, int batch,
                                const void* const* inputs, void* const* outputs, void* workspace,
                                size_t workspace_bytes, void* stream);

/* Rotated non-maximum suppression in the bird's-eye view: the host step after the score filter
 * (nms_cpu and box_overlap, se-ssd-ai-trt.cpp:97-273, called at :1892 with NMS_THRESH = 0.01, params.h:373). */
typedef struct sessd_nms_params {
    int32_t max_box_num;   /* rows of the box table (<= 2048) */
    float nms_thresh;      /* a box is dropped when an earlier kept box overlaps it with IoU >= nms_thresh */
} sessd_nms_params;

size_t sessd_rotated_nms_workspace_bytes(const sessd_nms_params* p, int batch);

/* inputs = { box f32 [B][max_box][9] = (x, y, z, w, l, h, yaw, label, score), valid_line_num u32 [B] } (the first
 * and last outputs of sessd_filter_boxes_enqueue), outputs = { kept f32 [B][max_box][9], kept_num u32 [B] }.
 * Boxes are visited in descending score (equal scores: lower row first; the reference's std::sort leaves that
 * open); kept boxes are written in that order, rows after kept_num[b] are zero. IoU by the reference's polygon
 * rule in fp32. Replaces save_result + nms_cpu (se-ssd-ai-trt.cpp:1709-1721, :247-273) without the device-to-host
 * copy of the box table. */
int sessd_rotated_nms_enqueue(const sessd_nms_params* p, int batch, const void* const* inputs, void* const* outputs,
                              void* workspace, size_t workspace_bytes, void* stream);

/* Per-launch timing for benchmarks (takes the place of the reference's unused Tn::Profiler,
 * Utils.h:24-49). Between begin and end every kernel this library launches from the calling thread is
 * bracketed by CUDA events on its own stream. end synchronises the device, writes the kernel names
 * (newline separated) and their durations in milliseconds, and returns the number of launches. */
int sessd_profile_begin(void);
int sessd_profile_end(void* stream, char* names, size_t names_cap, float* ms, int cap);
/* Number of kernel launches issued by this library since process start (for launch accounting). */
uint64_t sessd_launch_count(void);

/* Synchronises `stream`, copies the status word of `workspace` to the host and returns it (>= 0),
 * or a negative sessd_error. */
int sessd_read_status(const void* workspace, void* stream);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char* sessd_last_cuda_error(void);
/* Library version string. */
const char* sessd_version(void);
/* Test hook for the time-out path, per weight object, off by default: while on, the tensor-core convolution
 * kernel launched with these weights keeps its weight streamer silent, so the kernel's bounded waits run out (about
 * 0.1 s), every block leaves through its abort path, the call returns SESSD_OK and the status word carries
 * SESSD_STATUS_TIMEOUT with the code of the wait in the second status word. Nothing faults or hangs; other weight
 * objects and the next call with the hook off are not affected. */
int sessd_conv_weights_debug_withhold(sessd_conv_weights* w, int on);

/* ------------------------------------------------------------------------------------------
 * On-disk formats either side of the path (host code, no GPU needed).
 * ---------------------------------------------------------------------------------------- */

/* A parsed weight file. Replaces loadWeights (se-ssd-ai-trt.cpp:278-314) and its std::map<std::string, Weights>:
 * first token = number of blobs, then per blob `name count` and `count` hexadecimal words, each the bit pattern
 * of one fp32 value (written by tools/gen_wts.py:85-99). A malformed or truncated file gives SESSD_ERR_IO
 * (the reference asserts or reads garbage); a name that occurs twice keeps its last blob, as the map does. */
typedef struct sessd_wts sessd_wts;
int sessd_wts_load(const char* path, sessd_wts** out);
void sessd_wts_destroy(sessd_wts* w);
int sessd_wts_count(const sessd_wts* w);   /* blobs in file order (duplicates included), or a negative error */
/* Blob `index` in file order / the blob called `name` (SESSD_ERR_PARAM when absent; the reference's
 * weightMap[name] silently creates an empty entry). The pointers stay valid until sessd_wts_destroy. */
int sessd_wts_entry(const sessd_wts* w, int index, const char** name, const float** values, int64_t* count);
int sessd_wts_find(const sessd_wts* w, const char* name, const float** values, int64_t* count);
/* Writes a file the reference's loadWeights reads back bit for bit (the exporter's format, tools/gen_wts.py:85-99). */
int sessd_wts_save(const char* path, int n, const char* const* names, const float* const* values,
                   const int64_t* counts);

/* scale = gamma / sqrt(var + eps), shift = beta - mean * gamma / sqrt(var + eps), in fp32: the numbers
 * add_batchNorm1d_relu (se-ssd-ai-trt.cpp:808-826) hands to its IScaleLayer, ready for the `scale` / `shift`
 * arguments of sessd_conv_weights_create. */
int sessd_fold_batchnorm(const float* gamma, const float* beta, const float* mean, const float* var, int len,
                         float eps, float* scale, float* shift);

/* sessd_backbone_create from a weight file: layer l takes `<prefix>.<module_index[l]>.weight` (the flattened
 * [k0][k1][k2][Cin][Cout] tensor) and folds the batch norm `<prefix>.<module_index[l] + 1>.{weight, bias,
 * running_mean, running_var}` with `eps`, which is what se-ssd-ai-trt.cpp:1147-1249 wires with
 * prefix "backbone.middle_conv", module indices 0, 3, ..., 39 and eps 1e-5. A missing blob or one of the wrong
 * size gives SESSD_ERR_PARAM. */
int sessd_backbone_create_from_wts(const sessd_voxel_params* vp, const sessd_conv_params* layers, int nlayers,
                                   const int32_t* module_index, const sessd_wts* w, const char* prefix, float eps,
                                   const sessd_s2d_params* s2d, int dtype, sessd_backbone** out);

/* Reads one point cloud file (fp32 x, y, z, intensity records, the KITTI ".bin" layout) into
 * points [max_points][4], zero-fills the rest and sets *points_size = bytes / 16. Replaces loadData
 * (se-ssd-ai-trt.cpp:1515-1556) and the size computation at :1848; a file larger than the buffer gives
 * SESSD_ERR_PARAM (the reference exits the process). */
int sessd_points_load(const char* path, float* points, int max_points, int32_t* points_size);

#ifdef __cplusplus
}
#endif
#endif /* SESSD_H_ */
