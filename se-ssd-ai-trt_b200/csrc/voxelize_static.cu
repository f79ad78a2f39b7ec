// Voxel generator entry point for callers that are not allowed to allocate device memory.
//
// Some hosts of this library hand out no workspace and must not call cudaMalloc themselves: code
// running inside a stream capture, a real-time inference loop whose memory was fixed at start-up, or
// a plugin host that sizes its arena before this library is loaded. For them the voxeliser's scratch
// (coordinate table, per-point slots, chunk counts, point counts, status block) lives in one
// file-scope device array that is part of the library image; every GPU that loads the library holds
// it until the process exits.
//
// The array's name is only a host-side handle here, so its device address is looked up once per
// device with cudaGetSymbolAddress (while that device is current) and then passed to the same
// kernels the regular entry point uses.
#include <mutex>

#include "common.cuh"

namespace {

// 4 MiB: enough for one frame of up to 32768 points with max_voxels up to 32768 and 5 points per voxel
// (about 2.3 MiB); anything larger is rejected.
constexpr size_t kStaticScratchBytes = 4u << 20;

static __device__ __align__(256) unsigned char g_voxel_scratch[kStaticScratchBytes];

std::mutex g_setup_mutex;
void* g_scratch_addr[64] = {nullptr};

}  // namespace

extern "C" int sessd_voxelize_enqueue_static(const sessd_voxel_params* p, int batch, int max_points, int out_dtype,
                                              const void* const* inputs, void* const* outputs, void* stream) {
    if (!p || !inputs || !outputs) return SESSD_ERR_NULL;
    const size_t need = sessd_voxelize_workspace_bytes(p, batch, max_points);
    if (need == 0) return SESSD_ERR_PARAM;
    if (need > kStaticScratchBytes) {
        sessd::set_cuda_error(cudaErrorInvalidValue,
                              "sessd_voxelize_enqueue_static: batch/max_points/max_voxels need more than the 4 MiB "
                              "built-in scratch; use sessd_voxelize_enqueue with a caller workspace");
        return SESSD_ERR_WORKSPACE;
    }
    int dev = 0;
    SESSD_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SESSD_ERR_PARAM;
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (!g_scratch_addr[dev]) {
            // first call on this device: resolve the device address of the array (device `dev` is current)
            void* addr = nullptr;
            SESSD_CUDA(cudaGetSymbolAddress(&addr, g_voxel_scratch));
            g_scratch_addr[dev] = addr;
        }
        scratch = g_scratch_addr[dev];
    }
    return sessd_voxelize_enqueue(p, batch, max_points, out_dtype, inputs, outputs, scratch, kStaticScratchBytes,
                                  stream);
}

// Status word of the last sessd_voxelize_enqueue_static call on the current device (the word sits at the start of
// the built-in array): synchronises `stream`, copies the word to the host and returns it (>= 0), or a negative
// sessd_error (SESSD_ERR_PARAM when no call has been made on this device yet). Allocates nothing.
extern "C" int sessd_voxelize_static_status(void* stream) {
    int dev = 0;
    SESSD_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SESSD_ERR_PARAM;
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        scratch = g_scratch_addr[dev];
    }
    if (!scratch) return SESSD_ERR_PARAM;
    return sessd_read_status(scratch, stream);
}
