// Sparse rows -> dense BEV map [B][C*D][H][W].
//
// Replaces Sparse2DensePlugin::enqueue (sparse2Dense.cu:224-249): the reference clears the map with
// cudaMemset and lets one thread per voxel loop over the C channels with stores H*W*D elements
// apart. Here the map is cleared by a vectorised fill and the scatter uses one thread per
// (row, channel) with the row's channels read coalesced; the map (9 MB in fp16) stays in L2
// between the fill and the scatter.
#include "common.cuh"

namespace sessd {

namespace {

template <typename T>
__global__ void __launch_bounds__(kThreads)
sparse2dense_kernel(const T* __restrict__ feat, const int4* __restrict__ coors, const int32_t* __restrict__ voxel_num,
                    int batch, int max_voxels, int C, int D, int H, int W, T* __restrict__ dense) {
    const int64_t per_frame = (int64_t)max_voxels * C;
    const int chunks = (int)((per_frame + kThreads - 1) / kThreads);
    const int items = batch * chunks;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int b = it / chunks;
        const int64_t t = (int64_t)(it - b * chunks) * kThreads + threadIdx.x;
        int n = voxel_num[b];
        n = n > max_voxels ? max_voxels : n;
        if (t >= (int64_t)n * C) continue;
        const int i = (int)(t / C), c = (int)(t - (int64_t)i * C);
        const int4 c4 = __ldg(&coors[(size_t)b * max_voxels + i]);  // (b, z, y, x)
        if (c4.y < 0 || c4.y >= D || c4.z < 0 || c4.z >= H || c4.w < 0 || c4.w >= W) continue;
        // dense[b][c*D + z][y][x] (sparse2Dense.cu:201-206)
        dense[(((size_t)b * C * D + (size_t)c * D + c4.y) * H + c4.z) * W + c4.w] = feat[(size_t)b * per_frame + t];
    }
}

}  // namespace

int launch_sparse2dense(const void* feat, const int32_t* coors, const int32_t* voxel_num, int batch, int max_voxels,
                        int C, int D, int H, int W, int dtype, void* dense, cudaStream_t stream) {
    const size_t esize = dtype == SESSD_F32 ? 4 : 2;
    const size_t bytes = (size_t)batch * C * D * H * W * esize;
    if (bytes % 16 != 0) {
        SESSD_CUDA(cudaMemsetAsync(dense, 0, bytes, stream));
    } else {
        int rc = launch_fill_zero(dense, bytes, stream);
        if (rc) return rc;
    }
    if (dtype == SESSD_F32) {
        SESSD_LAUNCH(sparse2dense_kernel<float>, persistent_grid(8), kThreads, 0, stream,
                     static_cast<const float*>(feat), reinterpret_cast<const int4*>(coors), voxel_num, batch,
                     max_voxels, C, D, H, W, static_cast<float*>(dense));
    } else {
        SESSD_LAUNCH(sparse2dense_kernel<__half>, persistent_grid(8), kThreads, 0, stream,
                     static_cast<const __half*>(feat), reinterpret_cast<const int4*>(coors), voxel_num, batch,
                     max_voxels, C, D, H, W, static_cast<__half*>(dense));
    }
    return SESSD_OK;
}

}  // namespace sessd
