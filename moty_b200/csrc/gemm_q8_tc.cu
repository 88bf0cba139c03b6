// gemm_q8_tc.cu -- tcgen05 int8 GEMM (placeholder until the kernel lands: reports
// "not supported" so that the drivers keep using the dp4a kernels).
#include "kernels.cuh"

bool q8_tc_supported(int, int, int) { return false; }
int q8_tc_make_tmap(MotyCudaMat *m) { m->has_tmap = false; return 0; }
int launch_q8_tc(const MotyCudaMat *, const int8_t *, const float *, float *, int32_t *, int, DevCtx *, cudaStream_t) {
    return moty_set_error(MOTY_CUDA_EARG, "tensor-core path not built");
}
