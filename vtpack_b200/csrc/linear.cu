// vtp_linear: argument checks and the choice between the tcgen05 and CUDA-core kernels.
#include "linear.h"

namespace vtp {

int linear_validate(const LinearArgs& p) {
    VTP_REQUIRE(p.a && p.w && p.y, VTP_ERR_NULL, "linear: null pointer");
    VTP_REQUIRE(p.dtype == VTP_F32 || p.dtype == VTP_BF16, VTP_ERR_DTYPE, "linear: dtype %d", p.dtype);
    VTP_REQUIRE(p.m_max >= 0 && p.N > 0 && p.K > 0, VTP_ERR_SHAPE, "linear: bad shape M=%d N=%d K=%d",
                p.m_max, p.N, p.K);
    VTP_REQUIRE(p.lda >= p.K && p.ldy >= p.N && (!p.res || p.ldr >= p.N), VTP_ERR_SHAPE,
                "linear: row stride shorter than the row");
    VTP_REQUIRE(aligned16(p.a) && aligned16(p.w) && aligned16(p.y) && aligned16(p.res) && aligned16(p.bias),
                VTP_ERR_ALIGN, "linear: pointers must be 16-byte aligned");
    return VTP_OK;
}

int linear(const LinearArgs& p, cudaStream_t st) {
    if (int rc = linear_validate(p)) return rc;
    // the tensor-core kernel takes K in 64-element TMA boxes; a narrower reduction (PVT's 4x4x3 patch
    // embedding, K = 48) is small enough for the CUDA-core kernel
    // and so does an output width that is not a whole number of 16-byte chunks (e.g. a 10-class head)
    const bool tc_shape = (p.K % 64 == 0 && p.N % 8 == 0 && p.lda % 8 == 0 && p.ldy % 8 == 0 &&
                           (!p.res || p.ldr % 8 == 0)) || p.ln_mode != 0 || p.emit_stats;
    if (p.dtype == VTP_BF16 && !(p.flags & VTP_FLAG_CUDA_CORES) && tc_shape) return linear_tcgen05(p, st);
    VTP_REQUIRE(p.ln_mode == 0 && !p.emit_stats, VTP_ERR_UNSUPPORTED,
                "linear (CUDA cores): folded LayerNorm is a feature of the tcgen05 kernel");
    return linear_cuda_cores(p, st);
}

// One warp per output row n of W [N,K]:
//   w_out[n,k] = round(W[n,k] * gamma[k]),  s[n] = sum_k w_out[n,k],  c[n] = sum_k beta[k] W[n,k] + bias[n]
template <typename T>
__global__ void __launch_bounds__(256)
fold_ln_kernel(const T* __restrict__ w, int N, int K, const float* __restrict__ gamma,
               const float* __restrict__ beta, const float* __restrict__ bias, T* __restrict__ w_out,
               float* __restrict__ s_out, float* __restrict__ c_out) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= N) return;
    float s = 0.f, c = 0.f;
    for (int k = lane; k < K; k += 32) {
        const float wv = to_f32(w[(size_t)n * K + k]);
        const T folded = from_f32<T>(wv * __ldg(gamma + k));
        w_out[(size_t)n * K + k] = folded;
        s += to_f32(folded);
        c = fmaf(__ldg(beta + k), wv, c);
    }
    s = warp_sum(s);
    c = warp_sum(c);
    if (lane == 0) {
        s_out[n] = s;
        c_out[n] = c + (bias ? __ldg(bias + n) : 0.f);
    }
}

}  // namespace vtp

extern "C" int vtp_fold_layernorm(const void* w, int dtype, int N, int K, const float* gamma, const float* beta,
                                  const float* bias, void* w_out, float* s_out, float* c_out, void* stream) {
    VTP_REQUIRE(w && gamma && beta && w_out && s_out && c_out, VTP_ERR_NULL, "fold_layernorm: null pointer");
    VTP_REQUIRE(dtype == VTP_F32 || dtype == VTP_BF16, VTP_ERR_DTYPE, "fold_layernorm: dtype %d", dtype);
    VTP_REQUIRE(N > 0 && K > 0, VTP_ERR_SHAPE, "fold_layernorm: bad shape");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = vtp::ceil_div(N, 8);
    if (dtype == VTP_F32)
        vtp::fold_ln_kernel<float><<<grid, 256, 0, st>>>((const float*)w, N, K, gamma, beta, bias, (float*)w_out, s_out, c_out);
    else
        vtp::fold_ln_kernel<vtp::bf16><<<grid, 256, 0, st>>>((const vtp::bf16*)w, N, K, gamma, beta, bias,
                                                             (vtp::bf16*)w_out, s_out, c_out);
    return vtp::check_launch("fold_layernorm");
}

extern "C" int vtp_linear(const void* a, long long lda, const void* w, const float* bias,
                          const void* residual, long long ldr, void* y, long long ldy, int dtype, int m_max,
                          const int32_t* m_dev, int N, int K, unsigned flags, void* stream) {
    vtp::LinearArgs p;
    p.a = a; p.lda = lda; p.w = w; p.bias = bias; p.res = residual; p.ldr = ldr; p.y = y; p.ldy = ldy;
    p.dtype = dtype; p.m_max = m_max; p.m_dev = m_dev; p.N = N; p.K = K; p.flags = flags;
    return vtp::linear(p, static_cast<cudaStream_t>(stream));
}
