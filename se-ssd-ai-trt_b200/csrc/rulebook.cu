// Rulebook construction for submanifold and strided sparse convolutions.
//
// The reference builds, in every plugin call, a dense index grid (up to 369 MB, reset with
// cudaMemset), a candidate list per voxel and an input-stationary pair list per kernel offset
// (submConv3dlayer.cu:271-459, sparseConv3dlayer.cu:310-555). Here the rulebook is kept in
// output-stationary form: nbr[b][k][o] = input row that feeds output row o through kernel offset k,
// or -1. Pair (k, i, o) of the reference exists exactly when nbr[b][k][o] == i, because
// k = in - out*stride + pad per axis (submConv3dlayer.cu:328-329) and input rows are unique.
// nbr[b][k][o] names the entry; in memory the map is tile-major (nbr_index in common.cuh: the offsets of a
// 128-row tile side by side), so that the tensor-core kernel fetches a tile's offsets with one copy.
//
// Where the rows of a frame come from decides how a coordinate is turned back into its row:
//   - the voxeliser's rows (full resolution, 92 M cells, 80 K of them active) sit in an x-grouped
//     open-addressing table (32-byte buckets of four x-neighbours);
//   - the rows a strided layer produces are numbered through an occupancy grid of the output level: one
//     bit per cell, 64 x-neighbours per word, each word followed by the number of rows before it. Every
//     candidate output of every input row sets its bit (sparseConv3dlayer.cu:310-386 with the truncating
//     divisions kept); a count and a scan/emit pass then number the set bits in (z, y, x) order and write
//     the output coordinates. A cell's row is prefix + popcount(bits below), one 16-byte read, and the
//     three x-neighbours of a 3x3x3 kernel share that read. The grids are small (3 MB per frame at half
//     resolution, 0.4 MB at quarter resolution) and stay in L2. The reference numbers outputs in the
//     arrival order of an atomic over a dense scan (sparseConv3dlayer.cu:529-541); (z, y, x) order is
//     deterministic and keeps the rows of a 128-row tile close together in space;
//   - coordinates handed in by a caller (the stand-alone plugin entry points) go into a flat table.
#include "numbering.cuh"

namespace sessd {

namespace {

__global__ void __launch_bounds__(kThreads)
table_build_kernel(const int4* __restrict__ coors, const int32_t* __restrict__ voxel_num, int batch, int max_voxels,
                   int Z, int Y, int X, Table t, int32_t* status) {
    const int chunks = (max_voxels + kThreads - 1) / kThreads;
    const int items = batch * chunks;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / chunks;
        const int i = (it - b * chunks) * kThreads + threadIdx.x;
        int n = voxel_num[b];
        n = n > max_voxels ? max_voxels : n;
        if (i >= n) continue;
        const int4 c = __ldg(&coors[(size_t)b * max_voxels + i]);  // (b, z, y, x)
        if (c.y < 0 || c.y >= Z || c.z < 0 || c.z >= Y || c.w < 0 || c.w >= X) {
            atomicOr(status, SESSD_STATUS_BAD_COORD);
            continue;
        }
        const uint32_t key = ((uint32_t)c.y * Y + c.z) * X + c.w;
        const int slot = table_insert(t.keys + (size_t)b * t.cap, t.cap, t.shift, key);
        if (slot < 0) {
            atomicOr(status, SESSD_STATUS_HASH_FULL);
            continue;
        }
        // Duplicate coordinates (the reference's grid keeps whichever write lands last,
        // submConv3dlayer.cu:457) resolve to the highest row here.
        atomicMax(&t.vals[(size_t)b * t.cap + slot], i);
    }
}

// One thread per (offset k, output row o); threads of a warp share k and walk consecutive rows, so
// the writes to nbr[b][k][*] are coalesced.
__global__ void __launch_bounds__(kThreads)
nbr_build_kernel(const int4* __restrict__ out_coors, const int32_t* __restrict__ out_num, int batch, int max_voxels,
                 ConvGeom g, Table in_table, int32_t* __restrict__ nbr) {
    const int chunks = (max_voxels + kThreads - 1) / kThreads;
    const int items = batch * g.kvol * chunks;
    const int k12 = g.K[1] * g.K[2];
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / (g.kvol * chunks);
        const int r = it - b * (g.kvol * chunks);
        const int k = r / chunks;
        const int o = (r - k * chunks) * kThreads + threadIdx.x;
        int n = out_num[b];
        n = n > max_voxels ? max_voxels : n;
        if (o >= n) continue;
        const int4 c = __ldg(&out_coors[(size_t)b * max_voxels + o]);
        const int kz = k / k12, ky = (k - kz * k12) / g.K[2], kx = k - kz * k12 - ky * g.K[2];
        // in = out*stride - pad + k*dilation (inverse of the offset formula at submConv3dlayer.cu:328)
        const int iz = c.y * g.S[0] - g.P[0] + kz * g.dil;
        const int iy = c.z * g.S[1] - g.P[1] + ky * g.dil;
        const int ix = c.w * g.S[2] - g.P[2] + kx * g.dil;
        int row = -1;
        if (iz >= 0 && iz < g.in_shape[0] && iy >= 0 && iy < g.in_shape[1] && ix >= 0 && ix < g.in_shape[2]) {
            const uint32_t key = ((uint32_t)iz * g.in_shape[1] + iy) * g.in_shape[2] + ix;
            const int slot = table_find(in_table.keys + (size_t)b * in_table.cap, in_table.cap, in_table.shift, key);
            if (slot >= 0) row = in_table.vals[(size_t)b * in_table.cap + slot];
        }
        nbr[nbr_index(g.kvol, max_voxels, b, k, o)] = row;
    }
}

// Integer helpers for the candidate geometry. Strides and candidate spans are 1, 2 or 3; a division by a
// run-time divisor costs some 25 instructions on the GPU and these kernels are bound by instruction issue,
// so the common divisors get shifts.
__device__ __forceinline__ int div_trunc(int a, int s) {   // C division (rounds toward zero)
    if (s == 1) return a;
    if (s == 2) return (a + (a < 0 ? 1 : 0)) >> 1;
    return a / s;
}
__device__ __forceinline__ void split_small(int e, int m, int* q, int* r) {   // e = q * m + r, e >= 0
    if (m == 1) {
        *q = e;
        *r = 0;
    } else if (m == 2) {
        *q = e >> 1;
        *r = e & 1;
    } else {
        *q = e / m;
        *r = e - *q * m;
    }
}

// One block per kernel offset: compacts nbr[frame][k][*] into the reference's pair columns.
__global__ void __launch_bounds__(kThreads)
rulebook_export_kernel(const int32_t* __restrict__ nbr, const int32_t* __restrict__ out_num, int frame, int kvol,
                       int max_voxels, int32_t* __restrict__ pairs, uint32_t* __restrict__ pair_num) {
    const int k = blockIdx.x;
    int n = out_num[frame];
    n = n > max_voxels ? max_voxels : n;
    const int32_t* col = nbr + nbr_index(kvol, max_voxels, frame, k, 0);   // entry o of the column: col[(o >> 7) * kvol * kNbrRun + (o & 127)]
    int32_t* pin = pairs + ((size_t)k * 2 + 0) * max_voxels;
    int32_t* pout = pairs + ((size_t)k * 2 + 1) * max_voxels;
    int base = 0;
    for (int o0 = 0; o0 < n; o0 += kThreads) {
        const int o = o0 + threadIdx.x;
        const int v = o < n ? col[(size_t)(o >> 7) * kvol * kNbrRun + (o & 127)] : -1;
        int total;
        const int pos = base + block_exclusive_scan(v >= 0 ? 1 : 0, &total);
        if (v >= 0) {
            pin[pos] = v;
            pout[pos] = o;
        }
        base += total;
    }
    if (threadIdx.x == 0) pair_num[k] = (uint32_t)base;
}

// Number of present neighbours (= rulebook pairs) of one layer, added to *total.
__global__ void __launch_bounds__(kThreads)
count_pairs_kernel(const int32_t* __restrict__ nbr, const int32_t* __restrict__ out_num, int batch, int max_voxels,
                   int kvol, unsigned long long* total) {
    const int chunks = (max_voxels + kThreads - 1) / kThreads;
    const int items = batch * kvol * chunks;
    int local = 0;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / (kvol * chunks);
        const int r = it - b * (kvol * chunks);
        const int k = r / chunks;
        const int o = (r - k * chunks) * kThreads + threadIdx.x;
        int n = out_num[b];
        n = n > max_voxels ? max_voxels : n;
        if (o < n && nbr[nbr_index(kvol, max_voxels, b, k, o)] >= 0) ++local;
    }
    const int sum = block_sum(local);
    if (threadIdx.x == 0 && sum) atomicAdd(total, (unsigned long long)sum);
}

// ---- x-grouped coordinate table ---------------------------------------------------------------
// A bucket is one 32-byte sector: the rows of the 4 cells that share (z, y, x >> 2), then the group
// key. The three x-neighbours of a cell lie in at most two buckets, so a 3x3x3 neighbourhood costs 9-18
// sector reads instead of 27 probes of a flat table.

__global__ void __launch_bounds__(kThreads)
bucket_build_kernel(const int4* __restrict__ coors, const int32_t* __restrict__ voxel_num, int batch, int max_voxels,
                    int Z, int Y, int X, Buckets t, int32_t* status) {
    const int chunks = (max_voxels + kThreads - 1) / kThreads;
    const int items = batch * chunks;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / chunks;
        const int i = (it - b * chunks) * kThreads + threadIdx.x;
        int n = voxel_num[b];
        n = n > max_voxels ? max_voxels : n;
        if (i >= n) continue;
        const int4 c = __ldg(&coors[(size_t)b * max_voxels + i]);
        if (c.y < 0 || c.y >= Z || c.z < 0 || c.z >= Y || c.w < 0 || c.w >= X) {
            atomicOr(status, SESSD_STATUS_BAD_COORD);
            continue;
        }
        const uint32_t key = ((uint32_t)c.y * Y + c.z) * X + c.w;
        const uint32_t gkey = key >> 2;
        uint32_t* base = t.data + (size_t)b * t.cap * 8;
        uint32_t h = hash_slot(gkey, t.shift);
        bool done = false;
        for (uint32_t probe = 0; probe < t.cap && !done; ++probe) {
            uint32_t* bk = base + (size_t)h * 8;
            uint32_t cur = bk[4];
            if (cur == kEmpty) cur = atomicCAS(&bk[4], kEmpty, gkey);
            if (cur == kEmpty || cur == gkey) {
                atomicMax(reinterpret_cast<int32_t*>(&bk[key & 3u]), i);  // duplicates: highest row wins
                done = true;
            }
            h = (h + 1) & (t.cap - 1);
        }
        if (!done) atomicOr(status, SESSD_STATUS_HASH_FULL);
    }
}

__device__ __forceinline__ int pick4(const int4& v, uint32_t i) {
    return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// First probe of a bucket lookup, kept apart from its evaluation so that a thread can have the probes of
// several lookups in flight at once (the kernel below is bound by dependent round trips to L2, not by bytes).
struct BucketProbe {
    uint4 lo, hi;
    uint32_t h;
};
__device__ __forceinline__ void bucket_probe(const uint32_t* __restrict__ base, int shift, uint32_t gkey, bool on,
                                             BucketProbe* p) {
    p->h = hash_slot(gkey, shift);
    p->hi = make_uint4(kEmpty, 0u, 0u, 0u);
    p->lo = make_uint4(~0u, ~0u, ~0u, ~0u);
    if (on) {
        // the whole 32-byte bucket with one 256-bit load (one request to L1 instead of two)
        const uint32_t* bk = base + (size_t)p->h * 8;
        asm volatile("ld.global.nc.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(p->lo.x), "=r"(p->lo.y), "=r"(p->lo.z), "=r"(p->lo.w), "=r"(p->hi.x), "=r"(p->hi.y),
                       "=r"(p->hi.z), "=r"(p->hi.w)
                     : "l"(bk));
    }
}
__device__ __forceinline__ int4 bucket_finish(const uint32_t* __restrict__ base, uint32_t cap, uint32_t gkey,
                                              const BucketProbe& p) {
    if (p.hi.x == gkey) return make_int4((int)p.lo.x, (int)p.lo.y, (int)p.lo.z, (int)p.lo.w);
    int4 none = make_int4(-1, -1, -1, -1);
    if (p.hi.x == kEmpty) return none;
    uint32_t h = (p.h + 1) & (cap - 1);   // first slot taken by another group: keep probing
    for (uint32_t probe = 1; probe < cap; ++probe) {
        const uint4* bk = reinterpret_cast<const uint4*>(base + (size_t)h * 8);
        const uint4 hi = __ldg(bk + 1);
        const uint4 lo = __ldg(bk);
        if (hi.x == gkey) return make_int4((int)lo.x, (int)lo.y, (int)lo.z, (int)lo.w);
        if (hi.x == kEmpty) return none;
        h = (h + 1) & (cap - 1);
    }
    return none;
}

// Submanifold 3x3x3 neighbour map. One thread per output row: it reads its coordinates once and, for each
// kz, has the bucket probes of the three ky rows (one or two 32-byte buckets each) in flight together,
// then writes nbr[b][k][o] for the nine offsets of that kz. Threads of a warp cover 32 consecutive rows of
// one 128-row tile, so the writes are coalesced and the per-tile offset mask (which offsets have any
// neighbour) costs one ballot per offset and one atomic per warp.
__global__ void __launch_bounds__(kThreads, 4)
nbr_build_subm_kernel(const int4* __restrict__ coors, const int32_t* __restrict__ voxel_num, int batch,
                      int max_voxels, int Z, int Y, int X, Buckets t, int32_t* __restrict__ nbr,
                      uint32_t* __restrict__ tile_mask, int tiles_per_frame) {
    const int chunks = (max_voxels + kThreads - 1) / kThreads;
    const int items = batch * chunks;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / chunks;
        const int o0 = (it - b * chunks) * kThreads;
        int n = voxel_num[b];
        n = n > max_voxels ? max_voxels : n;
        if (o0 >= n) continue;
        const int o = o0 + threadIdx.x;
        const bool live = o < n;
        int4 c = make_int4(0, -4, -4, -4);
        if (live) c = __ldg(&coors[(size_t)b * max_voxels + o]);
        const int x = c.w;
        const bool x_ok = live && x >= 0 && x < X;
        const uint32_t* base = t.data + (size_t)b * t.cap * 8;
        int32_t* out = nbr + nbr_index(27, max_voxels, b, 0, o);
        uint32_t bits = 0;
#pragma unroll
        for (int kz = 0; kz < 3; ++kz) {
            const int z = c.y + kz - 1;
            BucketProbe pa[3], pb[3];
            uint32_t center[3], g_lo[3], g_hi[3];
            bool on[3];
#pragma unroll
            for (int ky = 0; ky < 3; ++ky) {
                const int y = c.z + ky - 1;
                on[ky] = x_ok && z >= 0 && z < Z && y >= 0 && y < Y;
                center[ky] = on[ky] ? ((uint32_t)z * Y + y) * X + x : 0u;
                g_lo[ky] = (x > 0 ? center[ky] - 1 : center[ky]) >> 2;
                g_hi[ky] = (x + 1 < X ? center[ky] + 1 : center[ky]) >> 2;
                bucket_probe(base, t.shift, g_lo[ky], on[ky], &pa[ky]);
                bucket_probe(base, t.shift, g_hi[ky], on[ky] && g_hi[ky] != g_lo[ky], &pb[ky]);
            }
#pragma unroll
            for (int ky = 0; ky < 3; ++ky) {
                int res[3] = {-1, -1, -1};
                if (on[ky]) {
                    const int4 va = bucket_finish(base, t.cap, g_lo[ky], pa[ky]);
                    const int4 vb = g_hi[ky] != g_lo[ky] ? bucket_finish(base, t.cap, g_hi[ky], pb[ky]) : va;
#pragma unroll
                    for (int d = 0; d < 3; ++d) {
                        const int xx = x + d - 1;
                        if (xx < 0 || xx >= X) continue;
                        const uint32_t key = center[ky] + d - 1;
                        res[d] = pick4((key >> 2) == g_lo[ky] ? va : vb, key & 3u);
                    }
                }
#pragma unroll
                for (int d = 0; d < 3; ++d) {
                    const int k = (kz * 3 + ky) * 3 + d;
                    if (live) out[k * kNbrRun] = res[d];
                    if (__ballot_sync(0xFFFFFFFFu, res[d] >= 0)) bits |= 1u << k;
                }
            }
        }
        if ((threadIdx.x & 31) == 0 && bits && live)
            atomicOr(&tile_mask[(size_t)b * tiles_per_frame + (o >> 7)], bits);
    }
}

// ---- occupancy grids -----------------------------------------------------------------------------

__device__ __forceinline__ unsigned long long rec_bits(const uint4& r) {
    return (unsigned long long)r.x | ((unsigned long long)r.y << 32);
}

// Marks the candidate outputs of every input row: the reference's enumeration (sparseConv3dlayer.cu:339-383),
// one thread per input row. Per axis the row has up to three candidate output positions (one or two for the
// stride-2 layers); the x candidates of one (z, y) pair are neighbouring bits, mostly of one 64-bit word, so
// they are tested and set together, and all words are read before any is updated (the reads are independent;
// most of them find their bits already set by a neighbouring row and nothing is written).
__global__ void __launch_bounds__(kThreads)
mark_outputs_kernel(const int4* __restrict__ in_coors, const int32_t* __restrict__ in_num, int batch, int max_voxels,
                    ConvGeom g, BitGrid out) {
    constexpr int MAXS = 3;   // span_max never exceeds the kernel size (<= 3)
    const int chunks = (max_voxels + kThreads - 1) / kThreads;
    const int items = batch * chunks;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / chunks;
        const int i0 = (it - b * chunks) * kThreads;
        int n = in_num[b];
        n = n > max_voxels ? max_voxels : n;
        if (i0 >= n) continue;   // uniform over the block
        const int i = i0 + threadIdx.x;
        if (i >= n) continue;
        const int4 c4 = __ldg(&in_coors[(size_t)b * max_voxels + i]);
        const int c[3] = {c4.y, c4.z, c4.w};
        // candidate positions per axis, upper corner downward; pos[j][e] < 0 marks an unusable candidate
        int pos[3][MAXS];
        bool in_ok = true;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            // C integer division, as in the reference (sparseConv3dlayer.cu:339-348); dilation is 1
            const int lo = div_trunc(c[j] - (g.K[j] - 1) - 1 + g.S[j] + g.P[j], g.S[j]);
            const int hi = div_trunc(c[j] + g.P[j], g.S[j]);
            in_ok = in_ok && c[j] >= 0 && c[j] < g.in_shape[j];
#pragma unroll
            for (int e = 0; e < MAXS; ++e) {
                const int o = hi - e;
                const int k = c[j] - o * g.S[j] + g.P[j];   // the offset this pair would get (:366)
                const bool ok = e < g.span_max[j] && e <= hi - lo && o >= 0 && o < g.out_shape[j] && k >= 0 && k < g.K[j];
                pos[j][e] = ok ? o : -1;
            }
        }
        if (!in_ok) continue;
        // the x candidates as bits of at most two neighbouring words
        int w0 = -1;
        unsigned long long bits0 = 0ull, bits1 = 0ull;
#pragma unroll
        for (int e = 0; e < MAXS; ++e) {
            const int ox = pos[2][e];
            if (ox < 0) continue;
            if (w0 < 0) w0 = ox >> 6;            // candidates descend, so the first valid one has the highest word
            if ((ox >> 6) == w0) bits0 |= 1ull << (ox & 63);
            else bits1 |= 1ull << (ox & 63);     // the word below (spans are at most three cells)
        }
        if (w0 < 0) continue;
        unsigned long long* base = reinterpret_cast<unsigned long long*>(out.rec + (size_t)b * out.words);
        unsigned long long cur0[MAXS * MAXS], cur1[MAXS * MAXS];
        size_t rec[MAXS * MAXS];
#pragma unroll
        for (int ez = 0; ez < MAXS; ++ez)
#pragma unroll
            for (int ey = 0; ey < MAXS; ++ey) {
                const int q = ez * MAXS + ey;
                const bool ok = pos[0][ez] >= 0 && pos[1][ey] >= 0;
                rec[q] = ok ? ((size_t)pos[0][ez] * out.Y + pos[1][ey]) * out.xw + w0 : (size_t)-1;
                // a record is 16 bytes: its bits are the first 8
                cur0[q] = ok ? *reinterpret_cast<volatile unsigned long long*>(base + 2 * rec[q]) : ~0ull;
                cur1[q] = (ok && bits1) ? *reinterpret_cast<volatile unsigned long long*>(base + 2 * (rec[q] - 1)) : ~0ull;
            }
#pragma unroll
        for (int q = 0; q < MAXS * MAXS; ++q) {
            if (rec[q] == (size_t)-1) continue;
            if ((cur0[q] & bits0) != bits0) atomicOr(base + 2 * rec[q], bits0);
            if (bits1 && (cur1[q] & bits1) != bits1) atomicOr(base + 2 * (rec[q] - 1), bits1);
        }
    }
}

// Set bits of every 1024-word chunk of every frame.
__global__ void __launch_bounds__(kThreads)
count_bits_kernel(BitGrid g, int batch, int32_t* __restrict__ chunk_counts) {
    const int items = batch * g.chunks;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / g.chunks, c = it - b * g.chunks;
        const uint4* rec = g.rec + (size_t)b * g.words;
        int cnt = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int w = c * kChunk + threadIdx.x * 4 + j;
            if (w < g.words) cnt += __popcll(rec_bits(rec[w]));
        }
        const int total = block_sum(cnt);
        if (threadIdx.x == 0) chunk_counts[(size_t)b * g.chunks + c] = total;
    }
}

// Numbers the set bits of a frame in word order (= (z, y, x) order): writes every word's prefix, the output
// coordinates (sparseConv3dlayer.cu:436-441 writes them per pair) and the frame's row count. Rows past
// max_voxels are dropped (their bits stay set; look-ups reject ids >= max_voxels) and reported.
__global__ void __launch_bounds__(kThreads)
number_outputs_kernel(BitGrid g, int batch, int max_voxels, const int32_t* __restrict__ chunk_counts,
                      int4* __restrict__ out_coors, int32_t* __restrict__ out_num, int32_t* status) {
    const int items = batch * g.chunks;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / g.chunks, c = it - b * g.chunks;
        const int32_t* counts = chunk_counts + (size_t)b * g.chunks;
        if (c == 0) {
            int partial = 0;
            for (int j = threadIdx.x; j < g.chunks; j += kThreads) partial += counts[j];
            const int total = block_sum(partial);
            if (threadIdx.x == 0) {
                out_num[b] = total > max_voxels ? max_voxels : total;
                if (total > max_voxels) atomicOr(status, SESSD_STATUS_VOXEL_OVERFLOW);
            }
        }
        int partial = 0;
        for (int j = threadIdx.x; j < c; j += kThreads) partial += counts[j];
        const int base = block_sum(partial);
        uint4* rec = g.rec + (size_t)b * g.words;
        unsigned long long bits[4];
        int cnt = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int w = c * kChunk + threadIdx.x * 4 + j;
            bits[j] = w < g.words ? rec_bits(rec[w]) : 0ull;
            cnt += __popcll(bits[j]);
        }
        int unused;
        int id = base + block_exclusive_scan(cnt, &unused);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int w = c * kChunk + threadIdx.x * 4 + j;
            if (w >= g.words) continue;
            rec[w].z = (uint32_t)id;
            unsigned long long rem = bits[j];
            if (!rem) continue;
            const int row = w / g.xw;                 // z * Y + y
            const int x0 = (w - row * g.xw) << 6;
            const int z = row / g.Y, y = row - z * g.Y;
            while (rem) {
                const int bit = __ffsll((long long)rem) - 1;
                rem &= rem - 1ull;
                if (id < max_voxels) out_coors[(size_t)b * max_voxels + id] = make_int4(b, z, y, x0 + bit);
                ++id;
            }
        }
    }
}

// Rows of up to three x-neighbours (x0, x0+1, x0+2; `count` of them) of one (z, y) line of the input level.
struct BitsIndex {
    BitGrid g;
    int max_rows;
    struct Probe { uint4 a, b; int w; bool two; };
    __device__ __forceinline__ void probe(int b, int z, int y, int x0, int count, bool on, Probe* p) const {
        p->a = p->b = make_uint4(0u, 0u, 0u, 0u);
        p->two = false;
        p->w = 0;
        if (!on) return;
        const int lo = x0 < 0 ? 0 : x0, hi = x0 + count - 1 >= g.X ? g.X - 1 : x0 + count - 1;
        if (lo > hi) return;
        const uint4* rec = g.rec + (size_t)b * g.words + ((size_t)z * g.Y + y) * g.xw;
        p->w = lo >> 6;
        p->a = __ldg(rec + p->w);
        p->two = (hi >> 6) != p->w;
        if (p->two) p->b = __ldg(rec + p->w + 1);
    }
    __device__ __forceinline__ int finish(const Probe& p, int x) const {
        if (x < 0 || x >= g.X) return -1;
        const uint4& r = (x >> 6) == p.w ? p.a : p.b;
        if ((x >> 6) != p.w && !p.two) return -1;
        const unsigned long long bits = rec_bits(r);
        const int bit = x & 63;
        if (!((bits >> bit) & 1ull)) return -1;
        const int id = (int)r.z + __popcll(bits & ((1ull << bit) - 1ull));
        return id < max_rows ? id : -1;
    }
    // The rows of the cells x0 .. x0 + count - 1 (count <= 3) of a probed line at once: the cells are neighbouring
    // bits of a window that may straddle two records, and rows are numbered along the line, so the row of a set
    // cell is the row of the window's first cell plus the set cells before it.
    __device__ __forceinline__ void finish_line(const Probe& p, int x0, int count, int (&rows)[3]) const {
        const int lo = x0 < 0 ? 0 : x0;
        const int sh = lo & 63;
        const unsigned long long a = rec_bits(p.a), b = p.two ? rec_bits(p.b) : 0ull;
        const unsigned long long window = sh ? (a >> sh) | (b << (64 - sh)) : a;
        const int base = (int)p.a.z + __popcll(a & ((1ull << sh) - 1ull));
#pragma unroll
        for (int e = 0; e < 3; ++e) {
            const int x = x0 + e, pos = x - lo;
            int row = -1;
            if (e < count && x >= 0 && x < g.X && ((window >> pos) & 1ull)) {
                const int id = base + __popcll(window & ((1ull << pos) - 1ull));
                row = id < max_rows ? id : -1;
            }
            rows[e] = row;
        }
    }
};

// Neighbour map of a layer whose input level has an occupancy grid: one thread per output row walks the
// K0 x K1 lines of its receptive field, has the grid reads of a kz plane in flight together, and writes
// nbr[b][k][o] (coalesced over o) plus the per-128-row-tile offset mask (one ballot per offset, one atomic
// per warp). in = out*stride - pad + k, the inverse of the offset formula at submConv3dlayer.cu:328.
__global__ void __launch_bounds__(kThreads, 4)
map_rows_kernel(const int4* __restrict__ out_coors, const int32_t* __restrict__ out_num, int batch, int max_voxels,
                ConvGeom g, BitsIndex in, int32_t* __restrict__ nbr, uint32_t* __restrict__ tile_mask,
                int tiles_per_frame) {
    const int chunks = (max_voxels + kThreads - 1) / kThreads;
    const int items = batch * chunks;
    const int K0 = g.K[0], K1 = g.K[1], K2 = g.K[2];
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / chunks;
        const int o0 = (it - b * chunks) * kThreads;
        int n = out_num[b];
        n = n > max_voxels ? max_voxels : n;
        if (o0 >= n) continue;
        const int o = o0 + threadIdx.x;
        const bool live = o < n;
        int4 c = make_int4(0, 0, 0, 0);
        if (live) c = __ldg(&out_coors[(size_t)b * max_voxels + o]);
        const int bz = c.y * g.S[0] - g.P[0], by = c.z * g.S[1] - g.P[1], bx = c.w * g.S[2] - g.P[2];
        int32_t* out = nbr + nbr_index(g.kvol, max_voxels, b, 0, o);
        uint32_t bits = 0;
#pragma unroll
        for (int kz = 0; kz < 3; ++kz) {
            if (kz >= K0) break;
            const int z = bz + kz;
            const bool z_ok = live && z >= 0 && z < g.in_shape[0];
            BitsIndex::Probe pb[3];
#pragma unroll
            for (int ky = 0; ky < 3; ++ky) {
                if (ky >= K1) break;
                const int y = by + ky;
                in.probe(b, z, y, bx, K2, z_ok && y >= 0 && y < g.in_shape[1], &pb[ky]);
            }
#pragma unroll
            for (int ky = 0; ky < 3; ++ky) {
                if (ky >= K1) break;
                const int y = by + ky;
                const bool on = z_ok && y >= 0 && y < g.in_shape[1];
                int rows3[3] = {-1, -1, -1};
                if (on) in.finish_line(pb[ky], bx, K2, rows3);
#pragma unroll
                for (int kx = 0; kx < 3; ++kx) {
                    if (kx >= K2) break;
                    const int row = rows3[kx];
                    const int k = (kz * K1 + ky) * K2 + kx;
                    if (live) out[k * kNbrRun] = row;
                    if (__ballot_sync(0xFFFFFFFFu, row >= 0)) bits |= 1u << k;
                }
            }
        }
        if ((threadIdx.x & 31) == 0 && bits && live)
            atomicOr(&tile_mask[(size_t)b * tiles_per_frame + (o >> 7)], bits);
    }
}

// Fills the map entries of the tiles that hold rows 0 .. out_num[b] with -1, one int4 per thread (a tile's block of
// kvol x kNbrRun words is contiguous and 16-byte aligned; the padding words are written too).
__global__ void __launch_bounds__(kThreads)
nbr_clear_kernel(int32_t* __restrict__ nbr, const int32_t* __restrict__ out_num, int batch, int max_voxels, int kvol) {
    const size_t frame_words = nbr_frame_words(kvol, max_voxels);
    const int chunks = (int)((frame_words / 4 + kThreads - 1) / kThreads);
    const int items = batch * chunks;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / chunks;
        int n = out_num[b];
        n = n > max_voxels ? max_voxels : n;
        const size_t used_words = (size_t)((n + 127) / 128) * kvol * kNbrRun;   // a multiple of 4
        const size_t w = ((size_t)(it - b * chunks) * kThreads + threadIdx.x) * 4;
        if (w >= used_words) continue;
        *reinterpret_cast<int4*>(nbr + (size_t)b * frame_words + w) = make_int4(-1, -1, -1, -1);
    }
}

// Neighbour map of a strided layer whose input rows have no occupancy grid (the voxeliser's rows, or rows handed
// in by a caller): input-stationary. Thread = (input row i, candidate e) as in mark_outputs_kernel; the candidate's
// row in the numbered output grid is one read, and the pair lands as nbr[b][k][out] = i with
// k = in - out*stride + pad per axis (sparseConv3dlayer.cu:366). Each (k, out) has at most one input, so the
// writes never collide. The map must hold -1 for rows < out_num beforehand.
__global__ void __launch_bounds__(kThreads)
scatter_rows_kernel(const int4* __restrict__ in_coors, const int32_t* __restrict__ in_num, int batch, int max_voxels,
                    ConvGeom g, BitsIndex out, int32_t* __restrict__ nbr, uint32_t* __restrict__ tile_mask,
                    int tiles_per_frame) {
    const int64_t per_frame = (int64_t)max_voxels * g.ncand;
    const int chunks = (int)((per_frame + kThreads - 1) / kThreads);
    const int items = batch * chunks;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / chunks;
        const int t = (it - b * chunks) * kThreads + threadIdx.x;
        int n = in_num[b];
        n = n > max_voxels ? max_voxels : n;
        if ((it - b * chunks) * kThreads >= n * g.ncand) continue;   // uniform over the block
        if (t >= n * g.ncand) continue;
        const int i = g.cand_shift >= 0 ? (t >> g.cand_shift) : t / g.ncand;
        const int e = t - i * g.ncand;
        int cz, cy, cx, rest;
        split_small(e, g.span_max[2], &rest, &cx);
        split_small(rest, g.span_max[1], &cz, &cy);
        const int4 c4 = __ldg(&in_coors[(size_t)b * max_voxels + i]);
        const int c[3] = {c4.y, c4.z, c4.w};
        const int cj[3] = {cz, cy, cx};
        int o[3];
        bool ok = true;
        int k = 0;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            const int lo = div_trunc(c[j] - (g.K[j] - 1) - 1 + g.S[j] + g.P[j], g.S[j]);
            const int hi = div_trunc(c[j] + g.P[j], g.S[j]);
            o[j] = hi - cj[j];
            const int kj = c[j] - o[j] * g.S[j] + g.P[j];
            ok = ok && cj[j] <= hi - lo && o[j] >= 0 && o[j] < g.out_shape[j] && kj >= 0 && kj < g.K[j] &&
                 c[j] >= 0 && c[j] < g.in_shape[j];
            k = k * g.K[j] + kj;
        }
        if (!ok) continue;
        BitsIndex::Probe p;
        out.probe(b, o[0], o[1], o[2], 1, true, &p);
        const int id = out.finish(p, o[2]);
        if (id < 0) continue;   // output dropped by the max_voxels cap
        nbr[nbr_index(g.kvol, max_voxels, b, k, id)] = i;
        uint32_t* m = &tile_mask[(size_t)b * tiles_per_frame + (id >> 7)];
        if (!((*reinterpret_cast<volatile uint32_t*>(m) >> k) & 1u)) atomicOr(m, 1u << k);
    }
}

// Generic variant of the tile mask for maps built by nbr_build_kernel: one warp per (tile, k).
__global__ void __launch_bounds__(kThreads)
tile_mask_kernel(const int32_t* __restrict__ nbr, const int32_t* __restrict__ out_num, int batch, int max_voxels,
                 int kvol, uint32_t* __restrict__ tile_mask, int tiles_per_frame) {
    const int warps_per_block = kThreads / 32;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int64_t items = (int64_t)batch * tiles_per_frame * kvol;
    for (int64_t it = (int64_t)blockIdx.x * warps_per_block + w; it < items; it += (int64_t)gridDim.x * warps_per_block) {
        const int k = (int)(it % kvol);
        const int64_t bt = it / kvol;
        const int tile = (int)(bt % tiles_per_frame), b = (int)(bt / tiles_per_frame);
        int n = out_num[b];
        n = n > max_voxels ? max_voxels : n;
        bool any = false;
        for (int q = 0; q < 4; ++q) {
            const int o = tile * 128 + q * 32 + lane;
            if (o < n && nbr[nbr_index(kvol, max_voxels, b, k, o)] >= 0) any = true;
        }
        if (__ballot_sync(0xFFFFFFFFu, any) && lane == 0) atomicOr(&tile_mask[(size_t)b * tiles_per_frame + tile], 1u << k);
    }
}

}  // namespace

int launch_bucket_build(const int32_t* coors, const int32_t* voxel_num, int batch, int max_voxels, const int shape[3],
                        const Buckets& t, int32_t* status, cudaStream_t stream) {
    SESSD_LAUNCH(bucket_build_kernel, persistent_grid(8), kThreads, 0, stream, reinterpret_cast<const int4*>(coors),
                 voxel_num, batch, max_voxels, shape[0], shape[1], shape[2], t, status);
    return SESSD_OK;
}

int launch_nbr_build_subm(const int32_t* coors, const int32_t* voxel_num, int batch, int max_voxels, const int shape[3],
                          const Buckets& t, int32_t* nbr, uint32_t* tile_mask, cudaStream_t stream) {
    SESSD_LAUNCH(nbr_build_subm_kernel, persistent_grid(8), kThreads, 0, stream, reinterpret_cast<const int4*>(coors),
                 voxel_num, batch, max_voxels, shape[0], shape[1], shape[2], t, nbr, tile_mask,
                 (max_voxels + 127) / 128);
    return SESSD_OK;
}

int launch_tile_mask(const int32_t* nbr, const int32_t* out_num, int batch, int max_voxels, int kvol,
                     uint32_t* tile_mask, cudaStream_t stream) {
    SESSD_LAUNCH(tile_mask_kernel, persistent_grid(8), kThreads, 0, stream, nbr, out_num, batch, max_voxels, kvol,
                 tile_mask, (max_voxels + 127) / 128);
    return SESSD_OK;
}

int launch_count_pairs(const int32_t* nbr, const int32_t* out_num, int batch, int max_voxels, int kvol,
                       unsigned long long* total, cudaStream_t stream) {
    SESSD_LAUNCH(count_pairs_kernel, persistent_grid(8), kThreads, 0, stream, nbr, out_num, batch, max_voxels, kvol,
                 total);
    return SESSD_OK;
}

int conv_geom_from_params(const sessd_conv_params* p, ConvGeom* g) {
    for (int j = 0; j < 3; ++j) {
        g->K[j] = p->ksize[j];
        g->S[j] = p->subm ? 1 : p->stride[j];
        g->P[j] = p->padding[j];
        if (g->K[j] < 1 || g->K[j] > 3 || g->S[j] < 1 || g->S[j] > 3 || g->P[j] < 0 || g->P[j] > 2) return SESSD_ERR_PARAM;
    }
    g->dil = p->dilation < 1 ? 1 : p->dilation;
    if (g->dil != 1) return SESSD_ERR_UNSUPPORTED;  // the reference only ever passes 1 (se-ssd-ai-trt.cpp:704)
    g->out_shape[0] = p->out_shape_z; g->out_shape[1] = p->out_shape_y; g->out_shape[2] = p->out_shape_x;
    if (p->subm) {
        // SubM layers carry only out_shape in the reference (submConv3dlayer.cu:596-603).
        for (int j = 0; j < 3; ++j) g->in_shape[j] = g->out_shape[j];
    } else {
        g->in_shape[0] = p->spatial_shape_z; g->in_shape[1] = p->spatial_shape_y; g->in_shape[2] = p->spatial_shape_x;
    }
    g->kvol = g->K[0] * g->K[1] * g->K[2];
    g->ncand = 1;
    for (int j = 0; j < 3; ++j) {
        if (g->in_shape[j] < 1 || g->out_shape[j] < 1) return SESSD_ERR_PARAM;
        g->span_max[j] = (g->K[j] - 1) / g->S[j] + 1;
        g->ncand *= g->span_max[j];
    }
    g->cand_shift = -1;
    for (int sh = 0; sh < 6; ++sh)
        if (g->ncand == (1 << sh)) g->cand_shift = sh;
    const uint64_t vin = (uint64_t)g->in_shape[0] * g->in_shape[1] * g->in_shape[2];
    const uint64_t vout = (uint64_t)g->out_shape[0] * g->out_shape[1] * g->out_shape[2];
    if (vin >= 0xFFFFFFFFull || vout >= 0xFFFFFFFFull) return SESSD_ERR_PARAM;  // keys are 32-bit cell indices
    return SESSD_OK;
}

int launch_table_build(const int32_t* coors, const int32_t* voxel_num, int batch, int max_voxels, const int shape[3],
                       const Table& t, int32_t* status, cudaStream_t stream) {
    SESSD_LAUNCH(table_build_kernel, persistent_grid(8), kThreads, 0, stream, reinterpret_cast<const int4*>(coors),
                 voxel_num, batch, max_voxels, shape[0], shape[1], shape[2], t, status);
    return SESSD_OK;
}

int launch_nbr_build(const int32_t* out_coors, const int32_t* out_num, int batch, int max_voxels, const ConvGeom& g,
                     const Table& in_table, int32_t* nbr, cudaStream_t stream) {
    SESSD_LAUNCH(nbr_build_kernel, persistent_grid(8), kThreads, 0, stream, reinterpret_cast<const int4*>(out_coors),
                 out_num, batch, max_voxels, g, in_table, nbr);
    return SESSD_OK;
}

int launch_mark_outputs(const int32_t* in_coors, const int32_t* in_num, int batch, int max_voxels, const ConvGeom& g,
                        const BitGrid& out, cudaStream_t stream) {
    SESSD_LAUNCH(mark_outputs_kernel, persistent_grid(8), kThreads, 0, stream, reinterpret_cast<const int4*>(in_coors),
                 in_num, batch, max_voxels, g, out);
    return SESSD_OK;
}

int launch_number_outputs(const BitGrid& out, int batch, int max_voxels, int32_t* chunk_counts, int32_t* out_coors,
                          int32_t* out_num, int32_t* status, cudaStream_t stream) {
    SESSD_LAUNCH(count_bits_kernel, persistent_grid(8), kThreads, 0, stream, out, batch, chunk_counts);
    SESSD_LAUNCH(number_outputs_kernel, persistent_grid(8), kThreads, 0, stream, out, batch, max_voxels, chunk_counts,
                 reinterpret_cast<int4*>(out_coors), out_num, status);
    return SESSD_OK;
}

int launch_map_rows(const int32_t* out_coors, const int32_t* out_num, int batch, int max_voxels, const ConvGeom& g,
                    const BitGrid& in, int32_t* nbr, uint32_t* tile_mask, cudaStream_t stream) {
    SESSD_LAUNCH(map_rows_kernel, persistent_grid(8), kThreads, 0, stream, reinterpret_cast<const int4*>(out_coors),
                 out_num, batch, max_voxels, g, BitsIndex{in, max_voxels}, nbr, tile_mask, (max_voxels + 127) / 128);
    return SESSD_OK;
}

int launch_scatter_rows(const int32_t* in_coors, const int32_t* in_num, const int32_t* out_num, int batch,
                        int max_voxels, const ConvGeom& g, const BitGrid& out, int32_t* nbr, uint32_t* tile_mask,
                        cudaStream_t stream) {
    SESSD_LAUNCH(nbr_clear_kernel, persistent_grid(8), kThreads, 0, stream, nbr, out_num, batch, max_voxels, g.kvol);
    SESSD_LAUNCH(scatter_rows_kernel, persistent_grid(8), kThreads, 0, stream, reinterpret_cast<const int4*>(in_coors),
                 in_num, batch, max_voxels, g, BitsIndex{out, max_voxels}, nbr, tile_mask, (max_voxels + 127) / 128);
    return SESSD_OK;
}

int launch_rulebook_export(const int32_t* nbr, const int32_t* out_num, int frame, int kvol, int max_voxels,
                           int32_t* pairs, uint32_t* pair_num, cudaStream_t stream) {
    SESSD_CUDA(cudaMemsetAsync(pairs, 0xFF, sizeof(int32_t) * 2 * (size_t)kvol * max_voxels, stream));
    SESSD_LAUNCH(rulebook_export_kernel, kvol, kThreads, 0, stream, nbr, out_num, frame, kvol, max_voxels, pairs,
                 pair_num);
    return SESSD_OK;
}

}  // namespace sessd
