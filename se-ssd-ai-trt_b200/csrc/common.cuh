// Shared host/device helpers of the sparse front end library (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <vector>

#include "sessd.h"

namespace sessd {

constexpr uint32_t kEmpty = 0xFFFFFFFFu;   // empty key / unset rank in a coordinate table
constexpr size_t kAlign = 256;             // sub-buffer alignment inside a workspace
constexpr int kChunk = 1024;               // entries per compaction chunk (256 threads x 4)
constexpr int kThreads = 256;
constexpr int kMaxBatch = 4096;

// ---- host side ---------------------------------------------------------------------------

extern std::atomic<uint64_t> g_launches;
void set_cuda_error(cudaError_t e, const char* what);

// Optional per-launch timing: while a recorder is installed on the calling thread, every launch
// made through SESSD_LAUNCH is bracketed by two events on its stream.
struct StageRecorder {
    std::vector<cudaEvent_t> events;   // 2 per launch
    std::vector<const char*> names;
    void before(cudaStream_t s);
    void after(const char* name, cudaStream_t s);
};
extern thread_local StageRecorder* g_recorder;

#define SESSD_CUDA(call)                                   \
    do {                                                   \
        cudaError_t e__ = (call);                          \
        if (e__ != cudaSuccess) {                          \
            ::sessd::set_cuda_error(e__, #call);           \
            return SESSD_ERR_CUDA;                         \
        }                                                  \
    } while (0)

// Launches `kernel` and accounts for it under `name`; returns from the caller on a launch error.
#define SESSD_LAUNCH_NAMED(name, kernel, grid, block, smem, stream, ...)      \
    do {                                                                     \
        if (::sessd::g_recorder) ::sessd::g_recorder->before(stream);        \
        kernel<<<(grid), (block), (smem), (stream)>>>(__VA_ARGS__);          \
        ::sessd::g_launches.fetch_add(1, std::memory_order_relaxed);         \
        if (::sessd::g_recorder) ::sessd::g_recorder->after(name, stream);   \
        SESSD_CUDA(cudaGetLastError());                                      \
    } while (0)
#define SESSD_LAUNCH(kernel, grid, block, smem, stream, ...) \
    SESSD_LAUNCH_NAMED(#kernel, kernel, grid, block, smem, stream, __VA_ARGS__)

// Number of SMs of the current device (cached per device).
int sm_count();
// Grid for a persistent grid-stride kernel: `per_sm` blocks on every SM.
inline int persistent_grid(int per_sm) { return sm_count() * per_sm; }

// Two-pass workspace layout: with base == nullptr it only measures.
// A caller's workspace must start on a kAlign boundary (cudaMalloc and TensorRT workspaces do): the kernels use
// 16- and 32-byte vector accesses relative to it.
inline bool workspace_aligned(const void* p) { return reinterpret_cast<uintptr_t>(p) % kAlign == 0; }

struct Bump {
    char* base;
    size_t off;
    explicit Bump(void* b) : base(static_cast<char*>(b)), off(0) {}
    template <typename T>
    T* take(size_t count) {
        off = (off + kAlign - 1) / kAlign * kAlign;
        T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
        off += count * sizeof(T);
        return p;
    }
    size_t total() const { return (off + kAlign - 1) / kAlign * kAlign; }
};

inline uint32_t pow2_at_least(uint64_t v) {
    uint32_t c = 64;
    while (c < v) c <<= 1;
    return c;
}
inline int ilog2(uint32_t v) {
    int l = 0;
    while ((1u << l) < v) ++l;
    return l;
}

// One open-addressing coordinate table per frame: frame b owns slots [b*cap, (b+1)*cap).
// keys: linear cell index inside the frame's grid, kEmpty when free.
// rank: smallest producer index seen for the key (drives deterministic numbering); stride
//       `rank_stride` between consecutive slots so that the voxeliser's per-slot point lists
//       (whose first element is that minimum) can serve as the rank array.
// vals: row index of the key, -1 when the key has no row.
// Output tables of strided layers pack key and rank into one 64-bit slot (key in the high word), so that
// claiming a cell and lowering its rank is a single atomic; keys/rank then point into that array with
// stride 2.
struct Table {
    uint32_t* keys;
    uint32_t* rank;
    int32_t* vals;
    uint32_t cap;       // power of two
    int shift;          // 32 - log2(cap)
    int rank_stride;
    int key_stride;     // 1 for separate key / rank arrays; 2 when a slot is one 64-bit word (key << 32 | rank)
};

// x-grouped coordinate table of one resolution level: frame b owns buckets [b*cap, (b+1)*cap), a
// bucket is 8 words = {row of cell x&3 == 0..3, group key (cell index >> 2), 3 unused}; all words are
// 0xFFFFFFFF when free.
struct Buckets {
    uint32_t* data;
    uint32_t cap;   // buckets per frame, power of two
    int shift;      // 32 - log2(cap)
};

// Occupancy grid of one resolution level: frame b owns records [b*words, (b+1)*words); record w covers the 64 cells
// x = 64*(w % xw) .. +63 of line (z, y) = w / xw and holds {bits lo, bits hi, rows before this word, unused}.
// Rows are numbered in record order, i.e. in (z, y, x) order.
struct BitGrid {
    uint4* rec;
    int Z, Y, X;
    int xw;      // records per x line
    int words;   // records per frame
    int chunks;  // 1024-record chunks per frame
};
inline BitGrid bitgrid_shape(const int shape[3]) {
    BitGrid g{};
    g.Z = shape[0], g.Y = shape[1], g.X = shape[2];
    g.xw = (g.X + 63) / 64;
    g.words = g.Z * g.Y * g.xw;
    g.chunks = (g.words + kChunk - 1) / kChunk;
    return g;
}

// Neighbour maps are tile-major: [frame][tile of 128 output rows][kernel offset][kNbrRun], entry (k, o) of a frame
// holding the input row under offset k of output row o, or -1. All offsets of a tile lie side by side, kNbrRun
// words apart (the 128 entries and 16 bytes of padding), which is also how the tensor-core kernel keeps them in
// shared memory: the offsets of one of its stages arrive with a single copy, already spaced for its index reads.
constexpr int kNbrRun = 132;
__host__ __device__ inline size_t nbr_frame_words(int kvol, int max_voxels) {
    return (size_t)((max_voxels + 127) / 128) * kvol * kNbrRun;
}
__host__ __device__ inline size_t nbr_index(int kvol, int max_voxels, int b, int k, int o) {
    return (size_t)b * nbr_frame_words(kvol, max_voxels) + ((size_t)(o >> 7) * kvol + k) * kNbrRun + (o & 127);
}

// Geometry of one sparse convolution (z, y, x order everywhere).
struct ConvGeom {
    int K[3], S[3], P[3];
    int dil;
    int in_shape[3];
    int out_shape[3];
    int kvol;
    int span_max[3];  // most candidate outputs one input can have per axis
    int ncand;        // product of span_max
    int cand_shift;   // log2(ncand) when ncand is a power of two, else -1
};

// ---- device side -------------------------------------------------------------------------

__device__ __forceinline__ uint32_t hash_slot(uint32_t key, int shift) {
    return (key * 0x9E3779B1u) >> shift;
}

// Finds or claims the slot of `key`. Returns the slot index inside the frame's table or -1
// when `cap` probes found neither the key nor a free slot.
__device__ __forceinline__ int table_insert(uint32_t* keys, uint32_t cap, int shift, uint32_t key) {
    uint32_t h = hash_slot(key, shift);
    for (uint32_t probe = 0; probe < cap; ++probe) {
        uint32_t cur = keys[h];
        if (cur == key) return (int)h;
        if (cur == kEmpty) {
            uint32_t old = atomicCAS(&keys[h], kEmpty, key);
            if (old == kEmpty || old == key) return (int)h;
        }
        h = (h + 1) & (cap - 1);
    }
    return -1;
}

__device__ __forceinline__ int table_find(const uint32_t* __restrict__ keys, uint32_t cap, int shift, uint32_t key) {
    uint32_t h = hash_slot(key, shift);
    for (uint32_t probe = 0; probe < cap; ++probe) {
        uint32_t cur = __ldg(&keys[h]);
        if (cur == key) return (int)h;
        if (cur == kEmpty) return -1;
        h = (h + 1) & (cap - 1);
    }
    return -1;
}

// Exclusive prefix sum of `v` over the block (blockDim.x == kThreads); *total gets the block sum.
__device__ __forceinline__ int block_exclusive_scan(int v, int* total) {
    __shared__ int warp_sums[kThreads / 32];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int t = __shfl_up_sync(0xFFFFFFFFu, incl, d);
        if (lane >= d) incl += t;
    }
    __syncthreads();  // protects warp_sums against a previous call
    if (lane == 31) warp_sums[wid] = incl;
    __syncthreads();
    int base = 0, sum = 0;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) {
        int s = warp_sums[w];
        if (w < wid) base += s;
        sum += s;
    }
    *total = sum;
    return base + incl - v;
}

__device__ __forceinline__ int block_sum(int v) {
    int total;
    block_exclusive_scan(v, &total);
    return total;
}

// ---- pieces shared between translation units --------------------------------------------

// Ordered-unique numbering. Entry e of frame b (e < entries(b)) points at table slot
// slot_of[b][e] (or -1). The entry whose index equals the slot's rank owns the slot; owners are
// numbered 0,1,2,... in entry order. count pass + emit pass, no block waits on another block.
struct NumberingArgs {
    const int32_t* slot_of;     // [B][entry_stride]
    uint32_t slot_mask;         // bits of a non-negative slot_of value that hold the slot (the rest is the caller's)
    int64_t entry_stride;
    const int32_t* entry_count; // [B] device counts (points_size or voxel_num)
    int entry_mul;              // entries(b) = min(entry_count[b], entry_limit) * entry_mul
    int entry_limit;
    int32_t* chunk_counts;      // [B][chunks_per_frame]
    int chunks_per_frame;
    int batch;
};

int launch_count_owners(const NumberingArgs& a, const Table& t, cudaStream_t stream);

// Zeroes rows [voxel_num[b], max_voxels) of a [B][max_voxels][row_bytes] tensor (row_bytes % 4 == 0).
int launch_zero_tail(void* tensor, int row_bytes, const int32_t* voxel_num, int batch, int max_voxels,
                     cudaStream_t stream);
int launch_fill_zero(void* ptr, size_t bytes, cudaStream_t stream);  // bytes % 16 == 0, ptr 16-byte aligned
int launch_fill_ones(void* ptr, size_t bytes, cudaStream_t stream);  // every byte 0xFF; same constraints
// Several fills as one launch: range r is n16[r] 16-byte words at ptr[r] (16-byte aligned), 0xFF bytes when ones[r]
// is set, else zeros; unused ranges have n16 = 0.
struct FillRanges {
    uint4* ptr[4];
    size_t n16[4];
    int ones[4];
};
int launch_fill_ranges(const FillRanges& f, cudaStream_t stream);

// rulebook.cu
int conv_geom_from_params(const sessd_conv_params* p, ConvGeom* g);
int launch_table_build(const int32_t* coors, const int32_t* voxel_num, int batch, int max_voxels, const int shape[3],
                       const Table& t, int32_t* status, cudaStream_t stream);
int launch_nbr_build(const int32_t* out_coors, const int32_t* out_num, int batch, int max_voxels, const ConvGeom& g,
                     const Table& in_table, int32_t* nbr, cudaStream_t stream);
// Strided layers: set the bit of every candidate output, then number the set bits in (z, y, x) order.
int launch_mark_outputs(const int32_t* in_coors, const int32_t* in_num, int batch, int max_voxels, const ConvGeom& g,
                        const BitGrid& out, cudaStream_t stream);
int launch_number_outputs(const BitGrid& out, int batch, int max_voxels, int32_t* chunk_counts, int32_t* out_coors,
                          int32_t* out_num, int32_t* status, cudaStream_t stream);
// Neighbour map + tile masks of a layer (any kernel up to 3x3x3, any stride) whose input level has an occupancy
// grid: output-stationary, one thread per output row.
int launch_map_rows(const int32_t* out_coors, const int32_t* out_num, int batch, int max_voxels, const ConvGeom& g,
                    const BitGrid& in, int32_t* nbr, uint32_t* tile_mask, cudaStream_t stream);
// The same for a strided layer whose input rows have no grid (voxeliser rows, caller's rows): input-stationary,
// every candidate of every input row finds its output row in the numbered output grid. Clears the map first.
int launch_scatter_rows(const int32_t* in_coors, const int32_t* in_num, const int32_t* out_num, int batch,
                        int max_voxels, const ConvGeom& g, const BitGrid& out, int32_t* nbr, uint32_t* tile_mask,
                        cudaStream_t stream);
int launch_bucket_build(const int32_t* coors, const int32_t* voxel_num, int batch, int max_voxels, const int shape[3],
                        const Buckets& t, int32_t* status, cudaStream_t stream);
// 3x3x3 / stride 1 / pad 1 neighbour map from a bucket table, plus the per-128-row-tile offset masks.
int launch_nbr_build_subm(const int32_t* coors, const int32_t* voxel_num, int batch, int max_voxels, const int shape[3],
                          const Buckets& t, int32_t* nbr, uint32_t* tile_mask, cudaStream_t stream);
int launch_tile_mask(const int32_t* nbr, const int32_t* out_num, int batch, int max_voxels, int kvol,
                     uint32_t* tile_mask, cudaStream_t stream);
// conv_simt.cu
struct ConvLaunch {
    const void* in;        // [B][max_voxels][Cin]
    void* out;             // [B][max_voxels][Cout]
    const int32_t* nbr;    // neighbour map, tile-major (nbr_index)
    const int32_t* out_num;// [B]
    const uint32_t* tile_mask; // [B][ceil(max_voxels/128)]: bit k set when offset k has a neighbour in the tile
    const void* weights;   // [kvol][Cin][Cout] in the feature dtype
    const void* umma_weights; // fp16 weights pre-tiled for the tensor-core kernel, or null
    const float* scale;    // [Cout] or null
    const float* shift;    // [Cout] or null
    int relu;
    int batch, max_voxels, kvol, cin, cout, dtype;
    // Optional fused BEV scatter (last layer): when dense != null the result row is also written to
    // dense[b][c*D + z][y][x] using out_coors.
    void* dense;
    const int32_t* out_coors;
    int D, H, W;
    int32_t* status;       // device status word (tensor-core path reports wait timeouts there)
    int debug_withhold_weights;   // tests only: the tensor-core kernel's weight streamer stays silent (waits run out)
    const float* scale_host;      // [Cout <= 64] host copies of scale / shift (ones / zeros without batch norm), or null
    const float* shift_host;
};
int launch_conv_simt(const ConvLaunch& c, cudaStream_t stream);
bool conv_simt_supported(int cin, int cout);

// conv_umma.cu (tcgen05 implicit GEMM, fp16 storage)
bool conv_umma_supported(int cin, int cout);
int conv_umma_pack_weights(const float* weights, int kvol, int cin, int cout, void** device_out);
int launch_conv_umma(const ConvLaunch& c, cudaStream_t stream);

// sparse2dense.cu
int launch_sparse2dense(const void* feat, const int32_t* coors, const int32_t* voxel_num, int batch, int max_voxels,
                        int C, int D, int H, int W, int top, int bottom, int left, int right, int dtype, void* dense,
                        cudaStream_t stream);
// [planes][H][W] -> [planes][top+H+bottom][left+W+right], zero border.
int launch_zero_pad2d(const void* in, void* out, size_t planes, int H, int W, int top, int bottom, int left, int right,
                      int dtype, cudaStream_t stream);

// voxelize.cu
struct VoxelWorkspace {
    int32_t* status;
    Table table;          // rank = per-slot sorted point list [cap][max_pts]
    int32_t* pt_slot;     // [B][max_points]
    int32_t* chunk_counts;// [B][chunks]
    int32_t* num_points;  // [B][max_voxels]
    int chunks;
    size_t table_bytes;   // bytes to set to 0xFF before a call (keys + point lists)
    void* table_base;
};
void voxel_workspace_layout(Bump& bump, const sessd_voxel_params* p, int batch, int max_points, VoxelWorkspace* w);
int voxelize_run(const sessd_voxel_params* p, int batch, int max_points, int out_dtype, const float* points,
                 const int32_t* points_size, void* voxels, int32_t* coors, int32_t* voxel_num, const VoxelWorkspace& w,
                 bool zero_tail, cudaStream_t stream, bool table_is_reset = false);   // table_is_reset: the caller has filled w.table_base

struct sessd_conv_weights_impl {
    void* w;        // device, [kvol][Cin][Cout] in dtype
    void* umma_w;   // device, tensor-core tiling of the same weights (fp16) or null
    float* scale;   // device or null
    float* shift;   // device or null
    int relu, dtype, kvol, cin, cout;
    int debug_withhold;   // tests of the time-out path: the tensor-core kernel's weight streamer stays silent
    // host copies of scale and shift (ones and zeros without batch norm) for kernels that take them as launch
    // parameters; filled for out_channel <= 64
    float host_scale[64], host_shift[64];
};

}  // namespace sessd
