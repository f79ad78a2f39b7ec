// Rotated non-maximum suppression in the bird's-eye view on the GPU.
//
// Replaces the host functions nms_cpu / box_overlap of the reference (se-ssd-ai-trt.cpp:97-273), which run
// after the score filter on at most max_box_num boxes per frame. Three small kernels per call:
//   1. per frame: rank the boxes by descending score (equal scores: lower row first; the reference's
//      std::sort leaves that open) and store every box's rotated corners and the cos/sin of -yaw once
//      (the reference recomputes them for every pair);
//   2. pairs: one thread per (box i, later box j) computes the IoU by the reference's polygon rule; a warp
//      covers 32 consecutive j and packs its "i suppresses j" bits with a ballot;
//   3. per frame: one warp walks the boxes in rank order, 64 at a time, keeps the ones not yet suppressed,
//      ORs their bit rows into the suppressed set, and writes the kept boxes in that order.
// Arithmetic is fp32 with explicit round-to-nearest operations (no contraction), in the reference's order.
#include "common.cuh"

namespace sessd {

namespace {

constexpr float kEps = 1e-8f;       // ThresHold, se-ssd-ai-trt.cpp:66
constexpr float kMargin = 1e-2f;    // MARGIN, :103
constexpr int kGeomFloats = 16;     // x, y, w, l, cos(-yaw), sin(-yaw), 2 unused, 4 corners (x, y)
constexpr size_t kStatusBytes = 1024;

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float dvd(float a, float b) { return __fdiv_rn(a, b); }

struct P2 {
    float x, y;
};

// (a - o) x (b - o), se-ssd-ai-trt.cpp:98-100
__device__ __forceinline__ float cross_at(P2 a, P2 b, P2 o) {
    return sub(mul(sub(a.x, o.x), sub(b.y, o.y)), mul(sub(b.x, o.x), sub(a.y, o.y)));
}

struct BevBox {
    float x, y, w, l, ncos, nsin;   // ncos/nsin: cos and sin of -yaw (check_box2d, :105-106)
    P2 corner[5];
};

__device__ __forceinline__ BevBox load_geom(const float* g) {
    BevBox b;
    b.x = g[0], b.y = g[1], b.w = g[2], b.l = g[3], b.ncos = g[4], b.nsin = g[5];
#pragma unroll
    for (int k = 0; k < 4; ++k) b.corner[k] = P2{g[8 + 2 * k], g[9 + 2 * k]};
    b.corner[4] = b.corner[0];
    return b;
}

__device__ __forceinline__ bool inside_with_margin(const BevBox& b, P2 p) {   // check_box2d, :102-112
    const float dx = sub(p.x, b.x), dy = sub(p.y, b.y);
    const float rx = add(mul(dx, b.ncos), mul(dy, -b.nsin));
    const float ry = add(mul(dx, b.nsin), mul(dy, b.ncos));
    return fabsf(rx) < add(b.w / 2, kMargin) && fabsf(ry) < add(b.l / 2, kMargin);
}

__device__ __forceinline__ bool segments_meet(P2 p1, P2 p0, P2 q1, P2 q0, P2* out) {   // intersection, :114-148
    const bool boxes_meet = fminf(p0.x, p1.x) <= fmaxf(q0.x, q1.x) && fminf(q0.x, q1.x) <= fmaxf(p0.x, p1.x) &&
                            fminf(p0.y, p1.y) <= fmaxf(q0.y, q1.y) && fminf(q0.y, q1.y) <= fmaxf(p0.y, p1.y);
    if (!boxes_meet) return false;
    const float s1 = cross_at(q0, p1, p0), s2 = cross_at(p1, q1, p0);
    const float s3 = cross_at(p0, q1, q0), s4 = cross_at(q1, p1, q0);
    if (!(mul(s1, s2) > 0.f && mul(s3, s4) > 0.f)) return false;
    const float s5 = cross_at(q1, p1, p0);
    if (fabsf(sub(s5, s1)) > kEps) {
        const float den = sub(s5, s1);
        out->x = dvd(sub(mul(s5, q0.x), mul(s1, q1.x)), den);
        out->y = dvd(sub(mul(s5, q0.y), mul(s1, q1.y)), den);
    } else {
        const float a0 = sub(p0.y, p1.y), b0 = sub(p1.x, p0.x), c0 = sub(mul(p0.x, p1.y), mul(p1.x, p0.y));
        const float a1 = sub(q0.y, q1.y), b1 = sub(q1.x, q0.x), c1 = sub(mul(q0.x, q1.y), mul(q1.x, q0.y));
        const float det = sub(mul(a0, b1), mul(a1, b0));
        out->x = dvd(sub(mul(b0, c1), mul(b1, c0)), det);
        out->y = dvd(sub(mul(a1, c0), mul(a0, c1)), det);
    }
    return true;
}

__device__ float bev_overlap(const BevBox& a, const BevBox& b) {   // box_overlap, :157-245
    P2 pts[16];
    float mx = 0.f, my = 0.f;
    int cnt = 0;
    for (int i = 0; i < 4; ++i)
        for (int j = 0; j < 4; ++j) {
            P2 p;
            if (segments_meet(a.corner[i + 1], a.corner[i], b.corner[j + 1], b.corner[j], &p)) {
                mx = add(mx, p.x), my = add(my, p.y);
                pts[cnt++] = p;
            }
        }
    for (int k = 0; k < 4; ++k) {
        if (inside_with_margin(a, b.corner[k])) {
            mx = add(mx, b.corner[k].x), my = add(my, b.corner[k].y);
            pts[cnt++] = b.corner[k];
        }
        if (inside_with_margin(b, a.corner[k])) {
            mx = add(mx, a.corner[k].x), my = add(my, a.corner[k].y);
            pts[cnt++] = a.corner[k];
        }
    }
    if (cnt < 3) return 0.f;   // the reference's loops yield 0 for fewer than three points
    mx = dvd(mx, (float)cnt), my = dvd(my, (float)cnt);
    float ang[16];
    for (int k = 0; k < cnt; ++k) ang[k] = atan2f(sub(pts[k].y, my), sub(pts[k].x, mx));
    for (int j = 0; j < cnt - 1; ++j)   // bubble sort by angle, as the reference (:222-233)
        for (int i = 0; i < cnt - j - 1; ++i)
            if (ang[i] > ang[i + 1]) {
                const P2 tp = pts[i];
                pts[i] = pts[i + 1];
                pts[i + 1] = tp;
                const float ta = ang[i];
                ang[i] = ang[i + 1];
                ang[i + 1] = ta;
            }
    float area = 0.f;
    for (int k = 0; k < cnt - 1; ++k) {
        const float ax = sub(pts[k].x, pts[0].x), ay = sub(pts[k].y, pts[0].y);
        const float bx = sub(pts[k + 1].x, pts[0].x), by = sub(pts[k + 1].y, pts[0].y);
        area = add(area, sub(mul(ax, by), mul(ay, bx)));
    }
    return fabsf(area) / 2.0f;
}

struct NmsArgs {
    const float* boxes;       // [B][M][9]
    const uint32_t* valid;    // [B]
    float* kept;              // [B][M][9]
    uint32_t* kept_num;       // [B]
    int32_t* order;           // [B][M]  rank -> input row
    float* geom;              // [B][M][16]
    unsigned long long* mask; // [B][M][words]
    int batch, max_box, words;
    float thresh;
};

__device__ __forceinline__ int frame_count(const NmsArgs& a, int b) {
    const uint32_t v = a.valid[b];
    return v > (uint32_t)a.max_box ? a.max_box : (int)v;
}

// Scores are ranked as a total order: a NaN score (a non-finite head output can produce one) counts as minus
// infinity, so that every box gets a rank of its own and every rank is written.
__device__ __forceinline__ float rank_score(float s) { return s != s ? -INFINITY : s; }

// Kernel 1: rank by (score descending, row ascending) by counting, then the geometry of every ranked box.
__global__ void __launch_bounds__(kThreads)
nms_rank_kernel(NmsArgs a) {
    for (int b = blockIdx.x; b < a.batch; b += gridDim.x) {
        const int n = frame_count(a, b);
        const float* bx = a.boxes + (size_t)b * a.max_box * 9;
        for (int i = threadIdx.x; i < n; i += kThreads) {
            const float si = rank_score(bx[i * 9 + 8]);
            int rank = 0;
            for (int j = 0; j < n; ++j) {
                const float sj = rank_score(bx[j * 9 + 8]);
                rank += (sj > si || (sj == si && j < i)) ? 1 : 0;
            }
            a.order[(size_t)b * a.max_box + rank] = i;
            const float* p = bx + i * 9;
            const float x = p[0], y = p[1], w = p[3], l = p[4], yaw = p[6];
            float* g = a.geom + ((size_t)b * a.max_box + rank) * kGeomFloats;
            g[0] = x, g[1] = y, g[2] = w, g[3] = l;
            g[4] = cosf(-yaw), g[5] = sinf(-yaw);
            g[6] = g[7] = 0.f;
            const float cs = cosf(yaw), sn = sinf(yaw);   // corners, :159-196
            const float hx = w / 2, hy = l / 2;
            const float lx[4] = {sub(x, hx), add(x, hx), add(x, hx), sub(x, hx)};
            const float ly[4] = {sub(y, hy), sub(y, hy), add(y, hy), add(y, hy)};
#pragma unroll
            for (int k = 0; k < 4; ++k) {   // rotate_around_center, :150-155
                const float dx = sub(lx[k], x), dy = sub(ly[k], y);
                g[8 + 2 * k] = add(add(mul(dx, cs), mul(dy, -sn)), x);
                g[9 + 2 * k] = add(add(mul(dx, sn), mul(dy, cs)), y);
            }
        }
    }
}

// Kernel 2: bit j of mask[b][i][w] = ranked box i suppresses ranked box w*64 + j (only j > i matter).
// One warp per (box i, 32-box column segment): lane = column, one IoU per thread, the 32 decisions packed
// by a ballot into half of a 64-bit mask word. Segments from the word that holds i itself up to the last
// word in use are always written (zeros where j <= i or j >= n), so the greedy pass never reads stale bits.
constexpr int kMaskWarps = 8;
__global__ void __launch_bounds__(kMaskWarps * 32)
nms_mask_kernel(NmsArgs a) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int segs = a.words * 2;
    const int64_t per_frame = (int64_t)a.max_box * segs;
    const int64_t items = (int64_t)a.batch * per_frame;
    for (int64_t it = (int64_t)blockIdx.x * kMaskWarps + warp; it < items; it += (int64_t)gridDim.x * kMaskWarps) {
        const int b = (int)(it / per_frame);
        const int r = (int)(it - (int64_t)b * per_frame);
        const int i = r / segs, seg = r - i * segs;
        const int n = frame_count(a, b);
        if (i >= n || seg < (i >> 6) * 2 || seg >= ((n + 63) >> 6) * 2) continue;   // uniform over the warp
        const int j = seg * 32 + lane;
        bool hit = false;
        if (j > i && j < n) {
            const float* gb = a.geom + (size_t)b * a.max_box * kGeomFloats;
            const float* gi = gb + (size_t)i * kGeomFloats;
            const float* gj = gb + (size_t)j * kGeomFloats;
            // boxes whose centres are farther apart than their half diagonals (plus the corner margin)
            // cannot touch: overlap 0, IoU 0, which is below any positive threshold
            const float dx = gj[0] - gi[0], dy = gj[1] - gi[1];
            const float rad_i = sqrtf(add(mul(gi[2], gi[2]), mul(gi[3], gi[3]))) * 0.5f;
            const float rad_j = sqrtf(gj[2] * gj[2] + gj[3] * gj[3]) * 0.5f;
            const float reach = rad_i + rad_j + 0.1f;
            float iou = 0.f;
            if (!(a.thresh > 0.f) || dx * dx + dy * dy <= reach * reach) {
                const BevBox bi = load_geom(gi);
                const BevBox bj = load_geom(gj);
                const float ov = bev_overlap(bi, bj);
                iou = dvd(ov, fmaxf(sub(add(mul(bi.w, bi.l), mul(bj.w, bj.l)), ov), kEps));   // nms_cpu, :262-265
            }
            hit = iou >= a.thresh;
        }
        const uint32_t bits = __ballot_sync(0xFFFFFFFFu, hit);
        if (lane == 0)   // little-endian halves of the 64-bit word: even segment = low half
            reinterpret_cast<uint32_t*>(a.mask + ((size_t)b * a.max_box + i) * a.words)[seg] = bits;
    }
}

// Kernel 3: greedy pass in rank order, one block per frame. When the frame's part of the mask fits the
// block's shared memory all threads stage it there first; warp 0 then walks the boxes 64 at a time (lane w
// holds word w of the suppressed set): the 64 x 64 diagonal block of the mask is fetched with one load per
// lane and resolved with shuffles (no memory access between dependent steps), then the full mask rows of the
// boxes kept in the block are ORed into the suppressed set with independent loads. All threads write the
// kept boxes in rank order.
constexpr int kReduceThreads = 256;
__global__ void __launch_bounds__(kReduceThreads)
nms_reduce_kernel(NmsArgs a, int smem_words) {
    extern __shared__ unsigned long long s_mask[];
    __shared__ unsigned long long s_keep[32];
    __shared__ int s_base[33];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int b = blockIdx.x; b < a.batch; b += gridDim.x) {
        const int n = frame_count(a, b);
        const int words_n = (n + 63) >> 6;
        const float* bx = a.boxes + (size_t)b * a.max_box * 9;
        float* out = a.kept + (size_t)b * a.max_box * 9;
        const unsigned long long* mask = a.mask + (size_t)b * a.max_box * a.words;
        int stride = a.words;
        __syncthreads();   // the previous frame is done with the shared arrays
        if (n * words_n <= smem_words) {
            // only words from the one that holds the row itself onward are ever written or read
            for (int e = threadIdx.x; e < n * words_n; e += kReduceThreads) {
                const int i = e / words_n, w = e - i * words_n;
                s_mask[e] = w >= (i >> 6) ? mask[(size_t)i * a.words + w] : 0ull;
            }
            mask = s_mask;
            stride = words_n;
        }
        __syncthreads();
        if (warp == 0) {
            unsigned long long removed = 0ull, keepw = 0ull;
            for (int c = 0; c < words_n; ++c) {
                const int i0 = c * 64 + lane, i1 = i0 + 32;
                const unsigned long long d0 = i0 < n ? mask[(size_t)i0 * stride + c] : 0ull;
                const unsigned long long d1 = i1 < n ? mask[(size_t)i1 * stride + c] : 0ull;
                unsigned long long rem = __shfl_sync(0xFFFFFFFFu, removed, c);
                unsigned long long keep = 0ull;
                const int rows = min(64, n - c * 64);
                for (int r = 0; r < rows; ++r) {           // every quantity here is uniform over the warp
                    const unsigned long long row = __shfl_sync(0xFFFFFFFFu, r < 32 ? d0 : d1, r & 31);
                    if (!((rem >> r) & 1ull)) {
                        keep |= 1ull << r;
                        rem |= row;
                    }
                }
                if (lane == c) keepw = keep;
                // eight rows per round, so that eight loads are in flight before the first OR waits for one
                unsigned long long acc = 0ull;
                const bool mine = lane > c && lane < words_n;
                for (unsigned long long kk = keep; kk;) {
                    unsigned long long v[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        v[u] = 0ull;
                        if (kk) {
                            const int r = __ffsll((long long)kk) - 1;
                            kk &= kk - 1ull;
                            if (mine) v[u] = mask[(size_t)(c * 64 + r) * stride + lane];
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) acc |= v[u];
                }
                removed |= acc;
            }
            const int cnt = __popcll(keepw);
            int incl = cnt;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
                if (lane >= d) incl += v;
            }
            s_keep[lane] = keepw;
            s_base[lane] = incl - cnt;
            if (lane == 31) s_base[32] = incl;
        }
        __syncthreads();
        // output rows: kept boxes in rank order
        const int total = s_base[32];
        for (int i = threadIdx.x; i < n; i += kReduceThreads) {
            const int c = i >> 6, r = i & 63;
            const unsigned long long kw = s_keep[c];
            if ((kw >> r) & 1ull) {
                const int pos = s_base[c] + __popcll(kw & ((1ull << r) - 1ull));
                const int src = a.order[(size_t)b * a.max_box + i];
                if ((unsigned)src >= (unsigned)n) continue;   // cannot happen with a total order; never read out of bounds
#pragma unroll
                for (int e = 0; e < 9; ++e) out[(size_t)pos * 9 + e] = bx[(size_t)src * 9 + e];
            }
        }
        for (int e = total * 9 + threadIdx.x; e < a.max_box * 9; e += kReduceThreads) out[e] = 0.f;   // rows after the count
        if (threadIdx.x == 0) a.kept_num[b] = (uint32_t)total;
    }
}

bool nms_params_ok(const sessd_nms_params* p, int batch) {
    return p && p->max_box_num > 0 && p->max_box_num <= 2048 && batch >= 1 && batch <= kMaxBatch;
}

}  // namespace

}  // namespace sessd

using namespace sessd;

extern "C" {

size_t sessd_rotated_nms_workspace_bytes(const sessd_nms_params* p, int batch) {
    if (!nms_params_ok(p, batch)) return 0;
    const size_t M = (size_t)p->max_box_num, words = (M + 63) / 64;
    Bump bump(nullptr);
    bump.take<char>(kStatusBytes);
    bump.take<int32_t>((size_t)batch * M);
    bump.take<float>((size_t)batch * M * kGeomFloats);
    bump.take<unsigned long long>((size_t)batch * M * words);
    return bump.total();
}

int sessd_rotated_nms_enqueue(const sessd_nms_params* p, int batch, const void* const* inputs, void* const* outputs,
                              void* workspace, size_t workspace_bytes, void* stream_v) {
    if (!p || !inputs || !outputs || !workspace || !inputs[0] || !inputs[1] || !outputs[0] || !outputs[1])
        return SESSD_ERR_NULL;
    if (!nms_params_ok(p, batch)) return SESSD_ERR_PARAM;
    if (workspace_bytes < sessd_rotated_nms_workspace_bytes(p, batch)) return SESSD_ERR_WORKSPACE;
    if (!workspace_aligned(workspace)) return SESSD_ERR_PARAM;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const size_t M = (size_t)p->max_box_num, words = (M + 63) / 64;
    Bump bump(workspace);
    bump.take<char>(kStatusBytes);
    NmsArgs a{};
    a.boxes = static_cast<const float*>(inputs[0]);
    a.valid = static_cast<const uint32_t*>(inputs[1]);
    a.kept = static_cast<float*>(outputs[0]);
    a.kept_num = static_cast<uint32_t*>(outputs[1]);
    a.order = bump.take<int32_t>((size_t)batch * M);
    a.geom = bump.take<float>((size_t)batch * M * kGeomFloats);
    a.mask = bump.take<unsigned long long>((size_t)batch * M * words);
    a.batch = batch;
    a.max_box = p->max_box_num;
    a.words = (int)words;
    a.thresh = p->nms_thresh;
    SESSD_CUDA(cudaMemsetAsync(workspace, 0, kStatusBytes, stream));
    const int frames_grid = batch < persistent_grid(8) ? batch : persistent_grid(8);
    SESSD_LAUNCH(nms_rank_kernel, frames_grid, kThreads, 0, stream, a);
    const int64_t pair_blocks = ((int64_t)batch * M * words * 2 + kMaskWarps - 1) / kMaskWarps;
    const int pair_grid = (int)(pair_blocks < persistent_grid(8) ? pair_blocks : persistent_grid(8));
    SESSD_LAUNCH(nms_mask_kernel, pair_grid, kMaskWarps * 32, 0, stream, a);
    // the staged copy of a frame's mask must fit the 48 KB a block gets without opting in; larger tables are read in place
    const size_t stage_bytes = M * words * sizeof(unsigned long long);
    const int smem_words = stage_bytes <= 40 * 1024 ? (int)(M * words) : 0;
    SESSD_LAUNCH(nms_reduce_kernel, frames_grid, kReduceThreads, (size_t)smem_words * sizeof(unsigned long long), stream, a,
                 smem_words);
    return SESSD_OK;
}

}  // extern "C"
