// Detection post-processing plugins: anchor generation + box decoding, score filter with compaction.
//
// Replaces generate_anchor_kernel + decode_kernel (generateAnchorDecode.cu:201-316) and
// filter_box_by_score_kernel (filterBoxByScore.cu:260-324). Differences from the reference, all of them
// deliberate: the batch dimension is honoured (the reference kernels index frame 0 only); anchors are
// never materialised (they are a closed form of the anchor index); the filter appends rows in ascending
// anchor index instead of the arrival order of an atomic, and stops at max_box_num rows (the reference
// writes past its outputs, filterBoxByScore.cu:275); and one entry point fuses both plugins, decoding only
// the few anchors that pass the score threshold.
//
// Ordered compaction without inter-block waits: a count pass stores the number of passing anchors of
// every 256-anchor chunk, the emit pass sums the counts of the chunks before its own and numbers its
// rows with a block scan.
#include "common.cuh"

namespace sessd {

namespace {

constexpr float kPiReference = 3.1415926f;   // the constant of filterBoxByScore.cu:309
constexpr size_t kStatusBytes = 1024;        // status block at the start of every workspace

struct AnchorGeom {
    float x_start, y_start, stride_x, stride_y;
    float car_l, car_w, car_h, angle0, angle1;
    int width, dir_num, anchors;   // anchors per frame = height * width * dir_num
};

__host__ AnchorGeom anchor_geom(const sessd_anchor_params& p) {
    AnchorGeom g;
    g.stride_x = (p.max_x - p.min_x) / (float)p.feature_map_width;     // generateAnchorDecode.cu:209-213
    g.stride_y = (p.max_y - p.min_y) / (float)p.feature_map_height;
    g.x_start = p.min_x + g.stride_x / 2;
    g.y_start = p.min_y + g.stride_y / 2;
    g.car_l = p.car_length;
    g.car_w = p.car_width;
    g.car_h = p.car_height;
    g.angle0 = p.direction_angle_0;
    g.angle1 = p.direction_angle_1;
    g.width = p.feature_map_width;
    g.dir_num = p.direction_angle_num;
    g.anchors = p.feature_map_height * p.feature_map_width * p.direction_angle_num;
    return g;
}

// Decoded box of anchor i from its 7 regression outputs t; explicit round-to-nearest operations so that no
// multiply-add is contracted (the CPU restatement used by the tests is compiled the same way).
__device__ __forceinline__ void decode_box(const AnchorGeom& g, int i, const float* __restrict__ t, float* o) {
    const float ax = __fadd_rn(g.x_start, __fmul_rn((float)((i % (g.width * g.dir_num)) / g.dir_num), g.stride_x));
    const float ay = __fadd_rn(g.y_start, __fmul_rn((float)(i / (g.width * g.dir_num)), g.stride_y));
    const int d = i % g.dir_num;
    const float ar = d == 0 ? g.angle0 : (d == 1 ? g.angle1 : 0.0f);
    const float diagonal = sqrtf(__fadd_rn(__fmul_rn(g.car_l, g.car_l), __fmul_rn(g.car_w, g.car_w)));
    o[0] = __fadd_rn(__fmul_rn(t[0], diagonal), ax);
    o[1] = __fadd_rn(__fmul_rn(t[1], diagonal), ay);
    o[2] = __fadd_rn(__fmul_rn(t[2], g.car_h), -1.0f);
    o[3] = __fmul_rn(expf(t[3]), g.car_w);
    o[4] = __fmul_rn(expf(t[4]), g.car_l);
    o[5] = __fmul_rn(expf(t[5]), g.car_h);
    o[6] = __fadd_rn(t[6], ar);
}

__device__ __forceinline__ float sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }   // filterBoxByScore.cu:105

__global__ void __launch_bounds__(kThreads)
anchor_decode_kernel(const float* __restrict__ box_preds, float* __restrict__ out, AnchorGeom g, int batch) {
    const int64_t total = (int64_t)batch * g.anchors;
    for (int64_t e = (int64_t)blockIdx.x * kThreads + threadIdx.x; e < total; e += (int64_t)gridDim.x * kThreads) {
        const int i = (int)(e % g.anchors);
        float t[7], o[7];
#pragma unroll
        for (int j = 0; j < 7; ++j) t[j] = __ldg(box_preds + e * 7 + j);
        decode_box(g, i, t, o);
#pragma unroll
        for (int j = 0; j < 7; ++j) out[e * 7 + j] = o[j];
    }
}

struct FilterArgs {
    const float* boxes;   // [B][N][7]: decoded boxes, or regression outputs when DECODE
    const float* cls;     // [B][N]
    const float* iou;     // [B][N]
    const float* dir;     // [B][N][2]
    float* out_box;       // [B][max_box][9]
    float* out_cls;       // [B][max_box]
    float* out_iou;       // [B][max_box]
    float* out_dir;       // [B][max_box]
    uint32_t* valid;      // [B]
    int32_t* chunk_counts;   // [B][chunks]
    int32_t* status;
    int batch, anchors, chunks, dir_num, max_box;
    float threshold, dir_offset;
};

// Pass 1: passing anchors per chunk; also clears the outputs (FilterBoxByScorePlugin::enqueue clears
// them with five memsets, filterBoxByScore.cu:353-371).
__global__ void __launch_bounds__(kThreads)
box_count_kernel(FilterArgs a) {
    const int items = a.batch * a.chunks;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / a.chunks, chunk = it - b * a.chunks;
        const int i = chunk * kThreads + threadIdx.x;
        int keep = 0;
        if (i < a.anchors) keep = sigmoid(__ldg(a.cls + (size_t)b * a.anchors + i)) >= a.threshold ? 1 : 0;
        const int n = block_sum(keep);
        if (threadIdx.x == 0) a.chunk_counts[it] = n;
    }
    const int64_t rows = (int64_t)a.batch * a.max_box;
    for (int64_t r = (int64_t)blockIdx.x * kThreads + threadIdx.x; r < rows; r += (int64_t)gridDim.x * kThreads) {
#pragma unroll
        for (int j = 0; j < 9; ++j) a.out_box[r * 9 + j] = 0.0f;
        a.out_cls[r] = 0.0f;
        a.out_iou[r] = 0.0f;
        a.out_dir[r] = 0.0f;
    }
}

// Pass 2: every chunk numbers its passing anchors after those of the chunks before it and writes the rows
// below max_box. DECODE: `boxes` holds regression outputs and the box is decoded here.
template <bool DECODE>
__global__ void __launch_bounds__(kThreads)
box_emit_kernel(FilterArgs a, AnchorGeom g) {
    const int items = a.batch * a.chunks;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / a.chunks, chunk = it - b * a.chunks;
        int before = 0;
        for (int c = threadIdx.x; c < chunk; c += kThreads) before += a.chunk_counts[b * a.chunks + c];
        const int base = block_sum(before);
        const int i = chunk * kThreads + threadIdx.x;
        const size_t e = (size_t)b * a.anchors + i;
        float score = 0.0f;
        int keep = 0;
        if (i < a.anchors) {
            score = sigmoid(__ldg(a.cls + e));
            keep = score >= a.threshold ? 1 : 0;
        }
        int total;
        const int idx = base + block_exclusive_scan(keep, &total);
        if (chunk == a.chunks - 1 && threadIdx.x == 0) {
            const int passed = base + total;
            a.valid[b] = (uint32_t)(passed < a.max_box ? passed : a.max_box);
            if (passed > a.max_box) atomicOr(a.status, SESSD_STATUS_BOX_OVERFLOW);
        }
        if (!keep || idx >= a.max_box) continue;
        const size_t r = (size_t)b * a.max_box + idx;
        const float q = __fmul_rn(__fadd_rn(__ldg(a.iou + e), 1.0f), 0.5f);          // filterBoxByScore.cu:284
        a.out_iou[r] = q;
        const float s = __fmul_rn(__fmul_rn(__fmul_rn(__fmul_rn(score, q), q), q), q);   // :288-289
        a.out_cls[r] = s;
        int best = 0;
        float best_v = -1000000.0f;
        for (int j = 0; j < a.dir_num; ++j) {           // last maximum wins (>=), row stride 2 (:295-302)
            const float v = __ldg(a.dir + e * 2 + j);
            if (v >= best_v) {
                best_v = v;
                best = j;
            }
        }
        a.out_dir[r] = (float)best;
        float t[7], bx[7];
#pragma unroll
        for (int j = 0; j < 7; ++j) t[j] = __ldg(a.boxes + e * 7 + j);
        if (DECODE) {
            decode_box(g, i, t, bx);
        } else {
#pragma unroll
            for (int j = 0; j < 7; ++j) bx[j] = t[j];
        }
        float* o = a.out_box + r * 9;
#pragma unroll
        for (int j = 0; j < 6; ++j) o[j] = bx[j];
        const float rel = __fadd_rn(bx[6], -a.dir_offset);
        const bool flip = (best == 1 && rel < 0.0f) || (best == 0 && rel > 0.0f);   // :307-315
        o[6] = flip ? __fadd_rn(bx[6], kPiReference) : bx[6];
        o[7] = 0.0f;
        o[8] = s;
    }
}

bool anchor_params_ok(const sessd_anchor_params* p) {
    return p->feature_map_height > 0 && p->feature_map_width > 0 && p->direction_angle_num > 0 &&
           p->direction_angle_num <= 2 &&
           (int64_t)p->feature_map_height * p->feature_map_width * p->direction_angle_num < (1 << 28);
}

bool filter_params_ok(const sessd_filter_params* p) {
    return p->feature_map_height > 0 && p->feature_map_width > 0 && p->direction_angle_num > 0 &&
           p->direction_angle_num <= 2 && p->max_box_num > 0 && p->max_box_num <= (1 << 20) &&
           (int64_t)p->feature_map_height * p->feature_map_width * p->direction_angle_num < (1 << 28);
}

int filter_chunks(const sessd_filter_params* p) {
    const int n = p->feature_map_height * p->feature_map_width * p->direction_angle_num;
    return (n + kThreads - 1) / kThreads;
}

int run_filter(const sessd_anchor_params* ap, const sessd_filter_params* p, int batch, const void* const* inputs,
               void* const* outputs, void* workspace, size_t workspace_bytes, void* stream_v) {
    if (!p || !inputs || !outputs || !workspace) return SESSD_ERR_NULL;
    for (int i = 0; i < 4; ++i)
        if (!inputs[i]) return SESSD_ERR_NULL;
    for (int i = 0; i < 5; ++i)
        if (!outputs[i]) return SESSD_ERR_NULL;
    if (!filter_params_ok(p) || batch < 1 || batch > kMaxBatch) return SESSD_ERR_PARAM;
    if (ap) {
        if (!anchor_params_ok(ap) || ap->feature_map_height != p->feature_map_height ||
            ap->feature_map_width != p->feature_map_width || ap->direction_angle_num != p->direction_angle_num)
            return SESSD_ERR_PARAM;
    }
    if (workspace_bytes < sessd_filter_boxes_workspace_bytes(p, batch)) return SESSD_ERR_WORKSPACE;
    if (!workspace_aligned(workspace)) return SESSD_ERR_PARAM;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    FilterArgs a{};
    a.boxes = static_cast<const float*>(inputs[0]);
    a.cls = static_cast<const float*>(inputs[1]);
    a.iou = static_cast<const float*>(inputs[2]);
    a.dir = static_cast<const float*>(inputs[3]);
    a.out_box = static_cast<float*>(outputs[0]);
    a.out_cls = static_cast<float*>(outputs[1]);
    a.out_iou = static_cast<float*>(outputs[2]);
    a.out_dir = static_cast<float*>(outputs[3]);
    a.valid = static_cast<uint32_t*>(outputs[4]);
    a.status = static_cast<int32_t*>(workspace);
    a.chunk_counts = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + kStatusBytes);
    a.batch = batch;
    a.anchors = p->feature_map_height * p->feature_map_width * p->direction_angle_num;
    a.chunks = filter_chunks(p);
    a.dir_num = p->direction_angle_num;
    a.max_box = p->max_box_num;
    a.threshold = p->score_threshold;
    a.dir_offset = p->direction_offset;
    SESSD_CUDA(cudaMemsetAsync(workspace, 0, kStatusBytes, stream));
    const int64_t items = (int64_t)batch * a.chunks;
    const int grid = (int)(items < persistent_grid(8) ? items : persistent_grid(8));
    SESSD_LAUNCH(box_count_kernel, grid, kThreads, 0, stream, a);
    if (ap) {
        SESSD_LAUNCH(box_emit_kernel<true>, grid, kThreads, 0, stream, a, anchor_geom(*ap));
    } else {
        SESSD_LAUNCH(box_emit_kernel<false>, grid, kThreads, 0, stream, a, AnchorGeom{});
    }
    return SESSD_OK;
}

}  // namespace

}  // namespace sessd

using namespace sessd;

extern "C" {

int sessd_anchor_decode_enqueue(const sessd_anchor_params* p, int batch, const void* const* inputs,
                                void* const* outputs, void* stream) {
    if (!p || !inputs || !outputs || !inputs[0] || !outputs[0]) return SESSD_ERR_NULL;
    if (!anchor_params_ok(p) || batch < 1 || batch > kMaxBatch) return SESSD_ERR_PARAM;
    const AnchorGeom g = anchor_geom(*p);
    const int64_t total = (int64_t)batch * g.anchors;
    const int64_t blocks = (total + kThreads - 1) / kThreads;
    const int grid = (int)(blocks < persistent_grid(8) ? blocks : persistent_grid(8));
    SESSD_LAUNCH(anchor_decode_kernel, grid, kThreads, 0, static_cast<cudaStream_t>(stream),
                 static_cast<const float*>(inputs[0]), static_cast<float*>(outputs[0]), g, batch);
    return SESSD_OK;
}

size_t sessd_filter_boxes_workspace_bytes(const sessd_filter_params* p, int batch) {
    if (!p || !filter_params_ok(p) || batch < 1 || batch > kMaxBatch) return 0;
    const size_t bytes = kStatusBytes + sizeof(int32_t) * (size_t)batch * filter_chunks(p);
    return (bytes + kAlign - 1) / kAlign * kAlign;
}

int sessd_filter_boxes_enqueue(const sessd_filter_params* p, int batch, const void* const* inputs,
                               void* const* outputs, void* workspace, size_t workspace_bytes, void* stream) {
    return run_filter(nullptr, p, batch, inputs, outputs, workspace, workspace_bytes, stream);
}

int sessd_decode_filter_enqueue(const sessd_anchor_params* ap, const sessd_filter_params* p, int batch,
                                const void* const* inputs, void* const* outputs, void* workspace,
                                size_t workspace_bytes, void* stream) {
    if (!ap) return SESSD_ERR_NULL;
    return run_filter(ap, p, batch, inputs, outputs, workspace, workspace_bytes, stream);
}

}  // extern "C"
