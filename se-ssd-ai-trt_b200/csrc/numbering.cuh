// Ordered-unique numbering of table slots (device templates).
//
// Both the voxeliser (entries = points) and the strided convolution (entries = candidate outputs
// of every input row) must number the distinct cells they touch in the order a sequential pass
// would first meet them. Each slot keeps the smallest entry index that touched it (its rank); the
// entry with that index owns the slot. Numbering is then a prefix sum over owner flags in entry
// order: a counting pass per 1024-entry chunk, and an emitting pass that adds the counts of the
// preceding chunks. No block ever waits for another block.
#pragma once

#include "common.cuh"

namespace sessd {

__device__ __forceinline__ int numbering_entries(const NumberingArgs& a, int b) {
    int n = a.entry_count[b];
    n = n < 0 ? 0 : (n > a.entry_limit ? a.entry_limit : n);
    return n * a.entry_mul;
}

__device__ __forceinline__ bool numbering_is_owner(const NumberingArgs& a, const Table& t, int b, int e, int n,
                                                   int* slot_out) {
    if (e >= n) return false;
    int s = a.slot_of[(int64_t)b * a.entry_stride + e];
    if (s >= 0) s = (int)((uint32_t)s & a.slot_mask);
    *slot_out = s;
    if (s < 0) return false;
    return t.rank[((size_t)b * t.cap + (uint32_t)s) * t.rank_stride] == (uint32_t)e;
}

// Emit must provide:
//   __device__ void frame_total(int b, int total)            once per frame
//   __device__ void operator()(int b, int e, int slot, int id)  once per owner entry
template <class Emit>
__global__ void __launch_bounds__(kThreads) emit_owners_kernel(NumberingArgs a, Table t, Emit emit) {
    const int cpf = a.chunks_per_frame;
    const int items = a.batch * cpf;
    for (int g = blockIdx.x; g < items; g += gridDim.x) {
        const int b = g / cpf, c = g - b * cpf;
        const int n = numbering_entries(a, b);
        const int nchunks = (n + kChunk - 1) / kChunk;
        if (c >= nchunks && c != 0) continue;  // uniform over the block
        const int32_t* counts = a.chunk_counts + (size_t)b * cpf;
        if (c == 0) {
            int partial = 0;
            for (int j = threadIdx.x; j < nchunks; j += kThreads) partial += counts[j];
            const int total = block_sum(partial);
            if (threadIdx.x == 0) emit.frame_total(b, total);
            if (nchunks == 0) continue;
        }
        int partial = 0;
        for (int j = threadIdx.x; j < c; j += kThreads) partial += counts[j];
        const int base = block_sum(partial);
        const int e0 = c * kChunk + threadIdx.x * 4;
        int slots[4];
        bool own[4];
        int cnt = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            slots[j] = -1;
            own[j] = numbering_is_owner(a, t, b, e0 + j, n, &slots[j]);
            cnt += own[j] ? 1 : 0;
        }
        int unused;
        int id = base + block_exclusive_scan(cnt, &unused);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (own[j]) {
                emit(b, e0 + j, slots[j], id);
                ++id;
            }
        }
    }
}

}  // namespace sessd
