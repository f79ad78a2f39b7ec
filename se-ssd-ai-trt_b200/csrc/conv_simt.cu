// Output-stationary sparse convolution on CUDA cores (fp32 and fp16 storage, fp32 accumulate).
//
// Replaces the reference's per-offset gather / multiply / atomicAdd kernel, launched kvol times per
// layer with one thread per rulebook pair and Cout global atomics per pair
// (submConv3dlayer.cu:479-518, :632-638). Here one launch covers the layer: a thread owns CO_T
// output channels of one output row, walks the row's kvol neighbour slots, and for each present
// neighbour accumulates s = sum_ci in[ci]*W[k][ci][co] as one fused-multiply-add chain (ci ascending),
// then acc += s with k ascending. That is the arithmetic of the reference kernel with the order of
// the atomic additions fixed, so fp32 results are reproducible bit for bit. BatchNorm scale/shift and
// ReLU (a separate TensorRT scale + activation layer in the reference, se-ssd-ai-trt.cpp:808-856)
// run in the epilogue, and the last layer can scatter straight into the dense BEV map.
//
// This path serves the memory-bound small-channel layers (4->16, 16->16, 16->32) and every fp32 layer.
#include <string>

#include "common.cuh"

namespace sessd {

namespace {

template <typename T, int N>
struct RowLoader;

template <int N>
struct RowLoader<float, N> {
    static __device__ __forceinline__ void load(const float* __restrict__ p, float (&x)[N]) {
        static_assert(N % 4 == 0, "row length must be a multiple of 4");
        const float4* v = reinterpret_cast<const float4*>(p);
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
            const float4 t = __ldg(v + i);
            x[4 * i + 0] = t.x; x[4 * i + 1] = t.y; x[4 * i + 2] = t.z; x[4 * i + 3] = t.w;
        }
    }
};

template <int N>
struct RowLoader<__half, N> {
    static __device__ __forceinline__ void load(const __half* __restrict__ p, float (&x)[N]) {
        static_assert(N % 4 == 0, "row length must be a multiple of 4");
        if constexpr (N % 8 == 0) {
            const uint4* v = reinterpret_cast<const uint4*>(p);
#pragma unroll
            for (int i = 0; i < N / 8; ++i) {
                const uint4 t = __ldg(v + i);
                const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(h[j]);
                    x[8 * i + 2 * j] = f.x; x[8 * i + 2 * j + 1] = f.y;
                }
            }
        } else {
            const uint2* v = reinterpret_cast<const uint2*>(p);
#pragma unroll
            for (int i = 0; i < N / 4; ++i) {
                const uint2 t = __ldg(v + i);
                const __half2* h = reinterpret_cast<const __half2*>(&t);
                const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
                x[4 * i] = a.x; x[4 * i + 1] = a.y; x[4 * i + 2] = b.x; x[4 * i + 3] = b.y;
            }
        }
    }
};

template <typename T, int N>
__device__ __forceinline__ void store_row(T* __restrict__ p, const float (&y)[N]) {
    if constexpr (sizeof(T) == 4) {
        float4* v = reinterpret_cast<float4*>(p);
#pragma unroll
        for (int i = 0; i < N / 4; ++i) v[i] = make_float4(y[4 * i], y[4 * i + 1], y[4 * i + 2], y[4 * i + 3]);
    } else {
        uint4* v = reinterpret_cast<uint4*>(p);
#pragma unroll
        for (int i = 0; i < N / 8; ++i) {
            uint4 t;
            __half2* h = reinterpret_cast<__half2*>(&t);
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(y[8 * i + 2 * j], y[8 * i + 2 * j + 1]);
            v[i] = t;
        }
    }
}

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

constexpr int CO_T = 16;  // output channels per thread

template <typename T, int CIN, int COUT>
__global__ void __launch_bounds__(kThreads)
conv_simt_kernel(const T* __restrict__ in, T* __restrict__ out, const int32_t* __restrict__ nbr,
                 const int32_t* __restrict__ out_num, const T* __restrict__ weights, const float* __restrict__ scale,
                 const float* __restrict__ shift, int relu, int batch, int max_voxels, int kvol,
                 T* __restrict__ dense, const int4* __restrict__ out_coors, int D, int H, int W) {
    constexpr int TPR = COUT / CO_T;          // threads per output row
    constexpr int ROWS = kThreads / TPR;      // rows per block iteration
    constexpr int KVOL_MAX = 27;              // 3 x 3 x 3 is the largest kernel the geometry code accepts
    constexpr bool COMPACT = CIN <= 16;
    __shared__ int32_t s_idx[COMPACT ? KVOL_MAX : 1][kThreads];
    const int chunks = (max_voxels + ROWS - 1) / ROWS;
    const int items = batch * chunks;
    const int cg = threadIdx.x % TPR;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / chunks;
        const int o = (it - b * chunks) * ROWS + threadIdx.x / TPR;
        int n = out_num[b];
        n = n > max_voxels ? max_voxels : n;
        if (o >= n) continue;
        float acc[CO_T];
#pragma unroll
        for (int c = 0; c < CO_T; ++c) acc[c] = 0.f;
        const int32_t* nb = nbr + nbr_index(kvol, max_voxels, b, 0, o);
        const T* in_b = in + (size_t)b * max_voxels * CIN;
        // one neighbour: s = sum_ci x[ci] * W[k][ci][:] as a fused chain, then acc += s
        auto add_neighbour = [&](int k, const float (&x)[CIN]) {
            float s[CO_T];
#pragma unroll
            for (int c = 0; c < CO_T; ++c) s[c] = 0.f;
            const T* wk = weights + (size_t)k * CIN * COUT + cg * CO_T;
#pragma unroll
            for (int ci = 0; ci < CIN; ++ci) {
                float w[CO_T];
                RowLoader<T, CO_T>::load(wk + ci * COUT, w);
#pragma unroll
                for (int c = 0; c < CO_T; ++c) s[c] = fmaf(x[ci], w[c], s[c]);
            }
#pragma unroll
            for (int c = 0; c < CO_T; ++c) acc[c] = __fadd_rn(acc[c], s[c]);
        };
        if constexpr (COMPACT) {
            // Narrow rows (the full-resolution layers, where a row has 5 of its 27 neighbours on average): all
            // slots are read first, then every thread walks its own present neighbours in ascending k (two
            // row loads in flight for the 4-channel input). A warp then runs as many steps as its fullest row has
            // neighbour pairs, instead of one step for every offset any of its 32 rows has. Same order of additions as below.
            uint32_t present = 0;
#pragma unroll
            for (int k = 0; k < KVOL_MAX; ++k) {
                const int idx = k < kvol ? __ldg(nb + k * kNbrRun) : -1;
                s_idx[k][threadIdx.x] = idx;          // read back by this thread only
                present |= (idx >= 0 ? 1u : 0u) << k;
            }
            constexpr int NP = CIN <= 4 ? 2 : 1;      // row loads in flight per thread (four measured no faster than two)
            while (present) {
                int ks[NP];
                float x[NP][CIN];
#pragma unroll
                for (int u = 0; u < NP; ++u) {
                    ks[u] = present ? __ffs((int)present) - 1 : -1;
                    present &= present - 1u;          // no-op when nothing is left
                    if (ks[u] >= 0) RowLoader<T, CIN>::load(in_b + (size_t)s_idx[ks[u]][threadIdx.x] * CIN, x[u]);
                }
#pragma unroll
                for (int u = 0; u < NP; ++u)
                    if (ks[u] >= 0) add_neighbour(ks[u], x[u]);
            }
        } else {
            for (int k = 0; k < kvol; ++k) {
                const int idx = __ldg(nb + k * kNbrRun);
                if (idx < 0) continue;
                float x[CIN];
                RowLoader<T, CIN>::load(in_b + (size_t)idx * CIN, x);
                add_neighbour(k, x);
            }
        }
#pragma unroll
        for (int c = 0; c < CO_T; ++c) {
            float v = acc[c];
            if (scale) v = fmaf(v, __ldg(scale + cg * CO_T + c), shift ? __ldg(shift + cg * CO_T + c) : 0.f);
            if (relu) v = v > 0.f ? v : 0.f;
            acc[c] = v;
        }
        store_row<T, CO_T>(out + ((size_t)b * max_voxels + o) * COUT + cg * CO_T, acc);
        if (dense) {
            // Fused BEV scatter (sparse2Dense.cu:201-206): channel c*D + z, pixel (y, x).
            const int4 c4 = __ldg(&out_coors[(size_t)b * max_voxels + o]);
            T* d = dense + (size_t)b * COUT * D * H * W + ((size_t)c4.y * H + c4.z) * W + c4.w;
#pragma unroll
            for (int c = 0; c < CO_T; ++c) d[(size_t)(cg * CO_T + c) * D * H * W] = from_float<T>(acc[c]);
        }
    }
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }

// Any channel counts (the reference's kernel takes in_channel and out_channel as run-time values,
// submConv3dlayer.cu:479-518): one warp per output row, lane = output channel (in rounds of 32), the same order of
// additions as above - per neighbour a fused chain over ci, neighbours added in ascending k. The pairs of the
// network's schedule never come here; this keeps the plugin entry points usable for other layer shapes.
template <typename T>
__global__ void __launch_bounds__(kThreads)
conv_generic_kernel(const T* __restrict__ in, T* __restrict__ out, const int32_t* __restrict__ nbr,
                    const int32_t* __restrict__ out_num, const T* __restrict__ weights, const float* __restrict__ scale,
                    const float* __restrict__ shift, int relu, int batch, int max_voxels, int kvol, int cin, int cout,
                    T* __restrict__ dense, const int4* __restrict__ out_coors, int D, int H, int W) {
    constexpr int ROWS = kThreads / 32;
    const int lane = threadIdx.x & 31, wrow = threadIdx.x >> 5;
    const int chunks = (max_voxels + ROWS - 1) / ROWS;
    const int items = batch * chunks;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / chunks;
        const int o = (it - b * chunks) * ROWS + wrow;
        int n = out_num[b];
        n = n > max_voxels ? max_voxels : n;
        if (o >= n) continue;
        const int32_t* nb = nbr + nbr_index(kvol, max_voxels, b, 0, o);
        const T* in_b = in + (size_t)b * max_voxels * cin;
        T* d = nullptr;
        if (dense) {
            const int4 c4 = __ldg(&out_coors[(size_t)b * max_voxels + o]);
            d = dense + (size_t)b * cout * D * H * W + ((size_t)c4.y * H + c4.z) * W + c4.w;
        }
        for (int co = lane; co < cout; co += 32) {
            float acc = 0.f;
            for (int k = 0; k < kvol; ++k) {
                const int idx = __ldg(nb + k * kNbrRun);
                if (idx < 0) continue;
                const T* x = in_b + (size_t)idx * cin;
                const T* wk = weights + (size_t)k * cin * cout + co;
                float sum = 0.f;
                for (int ci = 0; ci < cin; ++ci) sum = fmaf(to_float(x[ci]), to_float(wk[(size_t)ci * cout]), sum);
                acc = __fadd_rn(acc, sum);
            }
            if (scale) acc = fmaf(acc, __ldg(scale + co), shift ? __ldg(shift + co) : 0.f);
            if (relu) acc = acc > 0.f ? acc : 0.f;
            const T v = from_float<T>(acc);
            out[((size_t)b * max_voxels + o) * cout + co] = v;
            if (d) d[(size_t)co * D * H * W] = v;
        }
    }
}

template <typename T>
int launch_generic(const ConvLaunch& c, cudaStream_t stream) {
    SESSD_LAUNCH_NAMED(sizeof(T) == 4 ? "conv_generic<f32>" : "conv_generic<f16>", conv_generic_kernel<T>,
                       persistent_grid(8), kThreads, 0, stream, static_cast<const T*>(c.in), static_cast<T*>(c.out), c.nbr,
                       c.out_num, static_cast<const T*>(c.weights), c.scale, c.shift, c.relu, c.batch, c.max_voxels,
                       c.kvol, c.cin, c.cout, static_cast<T*>(c.dense), reinterpret_cast<const int4*>(c.out_coors), c.D,
                       c.H, c.W);
    return SESSD_OK;
}

template <typename T, int CIN, int COUT>
int launch_one(const ConvLaunch& c, cudaStream_t stream) {
    static const std::string name = std::string("conv_simt<") + (sizeof(T) == 4 ? "f32," : "f16,") +
                                    std::to_string(CIN) + "," + std::to_string(COUT) + ">";
    SESSD_LAUNCH_NAMED(name.c_str(), (conv_simt_kernel<T, CIN, COUT>), persistent_grid(4), kThreads, 0, stream,
                 static_cast<const T*>(c.in), static_cast<T*>(c.out), c.nbr, c.out_num,
                 static_cast<const T*>(c.weights), c.scale, c.shift, c.relu, c.batch, c.max_voxels, c.kvol,
                 static_cast<T*>(c.dense), reinterpret_cast<const int4*>(c.out_coors), c.D, c.H, c.W);
    return SESSD_OK;
}

template <typename T>
int dispatch(const ConvLaunch& c, cudaStream_t stream) {
#define SESSD_CASE(CI, CO) \
    if (c.cin == CI && c.cout == CO) return launch_one<T, CI, CO>(c, stream);
    SESSD_CASE(4, 16)
    SESSD_CASE(16, 16)
    SESSD_CASE(16, 32)
    SESSD_CASE(32, 32)
    SESSD_CASE(32, 64)
    SESSD_CASE(64, 64)
#undef SESSD_CASE
    return launch_generic<T>(c, stream);   // any other pair of channel counts
}

}  // namespace

bool conv_simt_supported(int cin, int cout) { return cin >= 1 && cout >= 1 && cin <= 4096 && cout <= 4096; }

int launch_conv_simt(const ConvLaunch& c, cudaStream_t stream) {
    return c.dtype == SESSD_F32 ? dispatch<float>(c, stream) : dispatch<__half>(c, stream);
}

}  // namespace sessd
