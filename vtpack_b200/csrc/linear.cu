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
    if (p.dtype == VTP_BF16 && !(p.flags & VTP_FLAG_CUDA_CORES)) return linear_tcgen05(p, st);
    return linear_cuda_cores(p, st);
}

}  // namespace vtp

extern "C" int vtp_linear(const void* a, long long lda, const void* w, const float* bias,
                          const void* residual, long long ldr, void* y, long long ldy, int dtype, int m_max,
                          const int32_t* m_dev, int N, int K, unsigned flags, void* stream) {
    vtp::LinearArgs p;
    p.a = a; p.lda = lda; p.w = w; p.bias = bias; p.res = residual; p.ldr = ldr; p.y = y; p.ldy = ldy;
    p.dtype = dtype; p.m_max = m_max; p.m_dev = m_dev; p.N = N; p.K = K; p.flags = flags;
    return vtp::linear(p, static_cast<cudaStream_t>(stream));
}
