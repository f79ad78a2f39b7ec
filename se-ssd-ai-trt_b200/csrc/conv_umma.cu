// Tensor-core (tcgen05 / TMEM) implicit-GEMM sparse convolution: placeholder until the kernel lands.
#include "common.cuh"

namespace sessd {

bool conv_umma_supported(int, int) { return false; }
int conv_umma_pack_weights(const float*, int, int, int, void** device_out) {
    *device_out = nullptr;
    return SESSD_OK;
}
int launch_conv_umma(const ConvLaunch&, cudaStream_t) { return SESSD_ERR_UNSUPPORTED; }

}  // namespace sessd
