// Layer boundary of a stack of MoE layers: x <- x + update (fp32 residual stream, in place), then
// the next layer's input RMSNorm(x) with unit gain, written in the activation dtype.
// One block per token.  Oracle: oracle/moe_oracle.py moe_stack (x_{l+1} = x_l + MoE_l(RMSNorm(x_l))).

#include "common.cuh"
#include "kernels.cuh"

namespace fk {

__global__ void __launch_bounds__(256) residual_norm_kernel(float* __restrict__ x, const float* __restrict__ update,
                                                            void* __restrict__ normed, int out_dtype, int H, float eps) {
    __shared__ float red[8];
    pdl_trigger();
    pdl_wait();
    float* row = x + (size_t)blockIdx.x * H;
    const float* up = update ? update + (size_t)blockIdx.x * H : nullptr;
    float ss = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float v = row[h];
        if (up) { v += up[h]; row[h] = v; }
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) total += red[i];
    const float inv = rsqrtf(total / (float)H + eps);
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float v = row[h] * inv;
        const size_t o = (size_t)blockIdx.x * H + h;
        if (out_dtype == FK_BF16) reinterpret_cast<__nv_bfloat16*>(normed)[o] = __float2bfloat16_rn(v);
        else if (out_dtype == FK_F16) reinterpret_cast<__half*>(normed)[o] = __float2half_rn(v);
        else reinterpret_cast<float*>(normed)[o] = v;
    }
}

int launch_residual_norm(float* x, const float* update, void* normed, int out_dtype, int T, int H, float eps, cudaStream_t stream) {
    if (T <= 0) return FK_OK;
    FK_CUDA_OK(launch_pdl(residual_norm_kernel, dim3(T), dim3(256), 0, stream, x, update, normed, out_dtype, H, eps), "residual norm launch");
    FK_LAUNCH_OK("residual norm launch");
    return FK_OK;
}

}  // namespace fk
