// Point cloud -> voxels with a mean voxel feature, for B independent frames per call.
//
// Replaces the reference's dense-grid voxeliser (voxelGenerator.cu:348-451, 255-321), which zeroes
// a 739 MB coordinate table every frame and lets a thread spin until another thread has published a
// voxel id. Here each frame owns a small open-addressing table keyed by the linear cell index:
//   pass 1 (insert)  every point claims/finds its cell's slot and pushes its index through the
//                    slot's ascending list of the max_points_per_voxel smallest point indices
//                    (a cascade of atomicMin, so the list content does not depend on timing);
//   pass 2 (count)   owner points (index == smallest index of the slot) are counted per chunk;
//   pass 3 (emit)    voxel ids = rank of the owner in point order; the owner writes coordinates,
//                    count and the mean of the listed points, summed in ascending index order.
// Results are therefore bit-reproducible, and no thread waits on another.
#include "numbering.cuh"

namespace sessd {

namespace {

struct VoxGeom {
    float x_min, x_max, y_min, y_max, z_min, z_max;
    float vx, vy, vz;
    int gx, gy, gz;
};

__global__ void __launch_bounds__(kThreads)
voxel_insert_kernel(const float4* __restrict__ points, const int32_t* __restrict__ points_size, int batch,
                    int max_points, VoxGeom g, Table t, int max_pts, int32_t* __restrict__ pt_slot,
                    int32_t* status) {
    const int chunks = (max_points + kThreads - 1) / kThreads;
    const int items = batch * chunks;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / chunks;
        const int p = (it - b * chunks) * kThreads + threadIdx.x;
        int n = points_size[b];
        n = n > max_points ? max_points : n;
        if (p >= n) continue;
        const float4 pt = __ldg(&points[(size_t)b * max_points + p]);
        int slot = -1;
        // Same tests and fp32 arithmetic as voxelGenerator.cu:363-375.
        if (pt.x >= g.x_min && pt.x < g.x_max && pt.y >= g.y_min && pt.y < g.y_max && pt.z >= g.z_min &&
            pt.z < g.z_max) {
            const int ix = (int)floorf(__fdiv_rn(__fsub_rn(pt.x, g.x_min), g.vx));
            const int iy = (int)floorf(__fdiv_rn(__fsub_rn(pt.y, g.y_min), g.vy));
            const int iz = (int)floorf(__fdiv_rn(__fsub_rn(pt.z, g.z_min), g.vz));
            if (ix >= 0 && ix < g.gx && iy >= 0 && iy < g.gy && iz >= 0 && iz < g.gz) {
                const uint32_t key = ((uint32_t)iz * g.gy + iy) * g.gx + ix;
                uint32_t* keys = t.keys + (size_t)b * t.cap;
                slot = table_insert(keys, t.cap, t.shift, key);
                if (slot < 0) {
                    atomicOr(status, SESSD_STATUS_HASH_FULL);
                } else {
                    // Keep the max_pts smallest point indices of the cell, ascending: offer the index to
                    // position 0; whatever loses a position (the larger value) is offered to the next.
                    uint32_t* list = t.rank + ((size_t)b * t.cap + (uint32_t)slot) * max_pts;
                    uint32_t carry = (uint32_t)p;
                    for (int j = 0; j < max_pts; ++j) {
                        const uint32_t old = atomicMin(&list[j], carry);
                        if (old == kEmpty) break;
                        carry = old > carry ? old : carry;
                    }
                }
            }
        }
        pt_slot[(size_t)b * max_points + p] = slot;
    }
}

template <typename T>
struct VoxelEmit {
    const float4* points;
    Table t;
    VoxGeom g;
    int max_points, max_pts, max_voxels;
    T* voxels;
    int32_t* coors;
    int32_t* num_points;
    int32_t* voxel_num;
    int32_t* status;

    __device__ void frame_total(int b, int total) const {
        voxel_num[b] = total > max_voxels ? max_voxels : total;
        if (total > max_voxels) atomicOr(status, SESSD_STATUS_VOXEL_OVERFLOW);
    }
    __device__ void operator()(int b, int /*e*/, int slot, int id) const {
        const size_t gslot = (size_t)b * t.cap + (uint32_t)slot;
        if (id >= max_voxels) {
            t.vals[gslot] = -1;
            return;
        }
        t.vals[gslot] = id;
        const uint32_t key = t.keys[gslot];
        const int plane = g.gy * g.gx;
        const int iz = key / plane, rem = key - iz * plane;
        const int iy = rem / g.gx, ix = rem - iy * g.gx;
        const size_t row = (size_t)b * max_voxels + id;
        reinterpret_cast<int4*>(coors)[row] = make_int4(b, iz, iy, ix);
        // Mean as generateAverage_kernel (voxelGenerator.cu:274-296): left-to-right sum over all
        // max_pts slots (unused slots contribute +0), divided by the clamped count.
        const uint32_t* list = t.rank + gslot * max_pts;
        float sx = 0.f, sy = 0.f, sz = 0.f, sw = 0.f;
        int cnt = 0;
        for (int j = 0; j < max_pts; ++j) {
            const uint32_t pi = list[j];
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (pi != kEmpty) {
                v = __ldg(&points[(size_t)b * max_points + pi]);
                ++cnt;
            }
            if (j == 0) {
                sx = v.x; sy = v.y; sz = v.z; sw = v.w;
            } else {
                sx = __fadd_rn(sx, v.x); sy = __fadd_rn(sy, v.y); sz = __fadd_rn(sz, v.z); sw = __fadd_rn(sw, v.w);
            }
        }
        const float fn = (float)cnt;
        const float mx = __fdiv_rn(sx, fn), my = __fdiv_rn(sy, fn), mz = __fdiv_rn(sz, fn), mw = __fdiv_rn(sw, fn);
        if constexpr (sizeof(T) == 4) {
            reinterpret_cast<float4*>(voxels)[row] = make_float4(mx, my, mz, mw);
        } else {
            __half2 lo = __floats2half2_rn(mx, my), hi = __floats2half2_rn(mz, mw);
            uint2 packed;
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
            reinterpret_cast<uint2*>(voxels)[row] = packed;
        }
        num_points[row] = cnt;
    }
};

__global__ void __launch_bounds__(kThreads) count_owners_kernel(NumberingArgs a, Table t) {
    const int cpf = a.chunks_per_frame;
    const int items = a.batch * cpf;
    for (int g = blockIdx.x; g < items; g += gridDim.x) {
        const int b = g / cpf, c = g - b * cpf;
        const int n = numbering_entries(a, b);
        if (c * kChunk >= n) continue;
        const int e0 = c * kChunk + threadIdx.x * 4;
        int cnt = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int s;
            cnt += numbering_is_owner(a, t, b, e0 + j, n, &s) ? 1 : 0;
        }
        const int total = block_sum(cnt);
        if (threadIdx.x == 0) a.chunk_counts[(size_t)b * cpf + c] = total;
    }
}

template <typename V>
__global__ void __launch_bounds__(kThreads)
zero_tail_kernel(V* __restrict__ tensor, int row_units, const int32_t* __restrict__ voxel_num, int batch,
                 int max_voxels) {
    const int64_t per_frame = (int64_t)max_voxels * row_units;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    V zero;
    memset(&zero, 0, sizeof(V));
    for (int b = 0; b < batch; ++b) {
        int n = voxel_num[b];
        n = n < 0 ? 0 : (n > max_voxels ? max_voxels : n);
        V* base = tensor + (int64_t)b * per_frame;
        for (int64_t i = (int64_t)n * row_units + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < per_frame; i += stride)
            base[i] = zero;
    }
}

__global__ void __launch_bounds__(kThreads) fill_zero_kernel(uint4* __restrict__ p, size_t n16) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16; i += stride) p[i] = make_uint4(0, 0, 0, 0);
}

__global__ void __launch_bounds__(kThreads) fill_ones_kernel(uint4* __restrict__ p, size_t n16) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16; i += stride)
        p[i] = make_uint4(kEmpty, kEmpty, kEmpty, kEmpty);
}

// Up to four ranges filled by one launch (r = range, 16-byte words; value 0 or kEmpty in every word): the resets a
// call of the fused front end needs (voxel table and bucket table to 0xFF, grids + masks and the BEV map to 0).
__global__ void __launch_bounds__(kThreads) fill_ranges_kernel(FillRanges f) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t first = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const uint32_t v = f.ones[r] ? kEmpty : 0u;
        uint4* p = f.ptr[r];
        const size_t n = f.n16[r];
        for (size_t i = first; i < n; i += stride) p[i] = make_uint4(v, v, v, v);
    }
}

}  // namespace

int launch_fill_ranges(const FillRanges& f, cudaStream_t stream) {
    SESSD_LAUNCH(fill_ranges_kernel, persistent_grid(8), kThreads, 0, stream, f);
    return SESSD_OK;
}

int launch_count_owners(const NumberingArgs& a, const Table& t, cudaStream_t stream) {
    SESSD_LAUNCH(count_owners_kernel, persistent_grid(8), kThreads, 0, stream, a, t);
    return SESSD_OK;
}

int launch_zero_tail(void* tensor, int row_bytes, const int32_t* voxel_num, int batch, int max_voxels,
                     cudaStream_t stream) {
    const int grid = persistent_grid(8);
    if (row_bytes % 16 == 0) {
        SESSD_LAUNCH(zero_tail_kernel<uint4>, grid, kThreads, 0, stream, static_cast<uint4*>(tensor), row_bytes / 16,
                     voxel_num, batch, max_voxels);
    } else if (row_bytes % 8 == 0) {
        SESSD_LAUNCH(zero_tail_kernel<uint2>, grid, kThreads, 0, stream, static_cast<uint2*>(tensor), row_bytes / 8,
                     voxel_num, batch, max_voxels);
    } else {
        SESSD_LAUNCH(zero_tail_kernel<uint32_t>, grid, kThreads, 0, stream, static_cast<uint32_t*>(tensor),
                     row_bytes / 4, voxel_num, batch, max_voxels);
    }
    return SESSD_OK;
}

int launch_fill_zero(void* ptr, size_t bytes, cudaStream_t stream) {
    if (bytes == 0) return SESSD_OK;
    SESSD_LAUNCH(fill_zero_kernel, persistent_grid(8), kThreads, 0, stream, static_cast<uint4*>(ptr), bytes / 16);
    return SESSD_OK;
}

int launch_fill_ones(void* ptr, size_t bytes, cudaStream_t stream) {
    if (bytes == 0) return SESSD_OK;
    SESSD_LAUNCH(fill_ones_kernel, persistent_grid(8), kThreads, 0, stream, static_cast<uint4*>(ptr), bytes / 16);
    return SESSD_OK;
}

void voxel_workspace_layout(Bump& bump, const sessd_voxel_params* p, int batch, int max_points, VoxelWorkspace* w) {
    const uint32_t cap = pow2_at_least(2ull * (uint64_t)max_points);
    w->chunks = (max_points + kChunk - 1) / kChunk;
    // keys and point lists are contiguous so that one fill resets both.
    const size_t key_elems = (size_t)batch * cap;
    const size_t list_elems = key_elems * p->max_points_per_voxel;
    uint32_t* block = bump.take<uint32_t>(key_elems + list_elems);
    w->table_base = block;
    w->table_bytes = (key_elems + list_elems) * sizeof(uint32_t);
    w->table.keys = block;
    w->table.rank = block ? block + key_elems : nullptr;
    w->table.vals = bump.take<int32_t>(key_elems);
    w->table.cap = cap;
    w->table.shift = 32 - ilog2(cap);
    w->table.rank_stride = p->max_points_per_voxel;
    w->table.key_stride = 1;
    w->pt_slot = bump.take<int32_t>((size_t)batch * max_points);
    w->chunk_counts = bump.take<int32_t>((size_t)batch * w->chunks);
    w->num_points = bump.take<int32_t>((size_t)batch * p->max_voxels);
}

int voxelize_run(const sessd_voxel_params* p, int batch, int max_points, int out_dtype, const float* points,
                 const int32_t* points_size, void* voxels, int32_t* coors, int32_t* voxel_num, const VoxelWorkspace& w,
                 bool zero_tail, cudaStream_t stream, bool table_is_reset) {
    VoxGeom g{p->x_min, p->x_max, p->y_min, p->y_max, p->z_min, p->z_max, p->voxel_x, p->voxel_y, p->voxel_z,
              p->grid_x, p->grid_y, p->grid_z};
    int rc = table_is_reset ? SESSD_OK : launch_fill_ones(w.table_base, w.table_bytes, stream);
    if (rc) return rc;
    const float4* pts = reinterpret_cast<const float4*>(points);
    SESSD_LAUNCH(voxel_insert_kernel, persistent_grid(8), kThreads, 0, stream, pts, points_size, batch, max_points, g,
                 w.table, p->max_points_per_voxel, w.pt_slot, w.status);
    NumberingArgs a{};
    a.slot_of = w.pt_slot;
    a.entry_stride = max_points;
    a.entry_count = points_size;
    a.entry_mul = 1;
    a.slot_mask = 0x7FFFFFFFu;
    a.entry_limit = max_points;
    a.chunk_counts = w.chunk_counts;
    a.chunks_per_frame = w.chunks;
    a.batch = batch;
    rc = launch_count_owners(a, w.table, stream);
    if (rc) return rc;
    if (out_dtype == SESSD_F32) {
        VoxelEmit<float> e{pts, w.table, g, max_points, p->max_points_per_voxel, p->max_voxels,
                           static_cast<float*>(voxels), coors, w.num_points, voxel_num, w.status};
        SESSD_LAUNCH(emit_owners_kernel<VoxelEmit<float>>, persistent_grid(8), kThreads, 0, stream, a, w.table, e);
    } else {
        VoxelEmit<__half> e{pts, w.table, g, max_points, p->max_points_per_voxel, p->max_voxels,
                            static_cast<__half*>(voxels), coors, w.num_points, voxel_num, w.status};
        SESSD_LAUNCH(emit_owners_kernel<VoxelEmit<__half>>, persistent_grid(8), kThreads, 0, stream, a, w.table, e);
    }
    if (zero_tail) {
        rc = launch_zero_tail(voxels, out_dtype == SESSD_F32 ? 16 : 8, voxel_num, batch, p->max_voxels, stream);
        if (rc) return rc;
        rc = launch_zero_tail(coors, 16, voxel_num, batch, p->max_voxels, stream);
        if (rc) return rc;
        rc = launch_zero_tail(w.num_points, 4, voxel_num, batch, p->max_voxels, stream);
        if (rc) return rc;
    }
    return SESSD_OK;
}

}  // namespace sessd
