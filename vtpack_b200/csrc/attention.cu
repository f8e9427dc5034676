// vtp_sparse_attention: argument checks and the choice between the tcgen05 and CUDA-core kernels.
#include "attention.h"

namespace vtp {

int attention(const AttnArgs& p, cudaStream_t st) {
    VTP_REQUIRE(p.q && p.k && p.v && p.out && p.offsets, VTP_ERR_NULL, "attention: null pointer");
    VTP_REQUIRE(p.dtype == VTP_F32 || p.dtype == VTP_BF16, VTP_ERR_DTYPE, "attention: dtype %d", p.dtype);
    VTP_REQUIRE(p.B > 0 && p.n_keys > 0 && p.heads > 0 && p.head_dim > 0 && p.l_max >= 0 && p.max_q >= 0,
                VTP_ERR_SHAPE, "attention: bad shape");
    if (p.l_max == 0 || p.max_q == 0) return VTP_OK;
    // the tensor-core kernel is written for 64-wide heads and at least one 16-key MMA step; other
    // shapes (and fp32) take the CUDA-core kernel
    const bool tc_shape = p.head_dim == 64 && p.n_keys >= 16 && p.B <= attention_tcgen05_max_images();
    if (p.dtype == VTP_BF16 && !(p.flags & VTP_FLAG_CUDA_CORES) && tc_shape) return attention_tcgen05(p, st);
    return attention_cuda_cores(p, st);
}

}  // namespace vtp

extern "C" int vtp_sparse_attention(const void* q, long long q_row_stride, long long q_head_stride,
                                    const void* k, const void* v, long long kv_batch_stride,
                                    long long kv_row_stride, long long kv_head_stride, void* out,
                                    long long o_row_stride, long long o_head_stride, int dtype, int B,
                                    int n_keys, int heads, int head_dim, const int32_t* offsets, int l_max,
                                    int max_q_per_image, float scale, unsigned flags, void* stream) {
    vtp::AttnArgs p;
    p.q = q; p.q_rs = q_row_stride; p.q_hs = q_head_stride;
    p.k = k; p.v = v; p.kv_bs = kv_batch_stride; p.kv_rs = kv_row_stride; p.kv_hs = kv_head_stride;
    p.out = out; p.o_rs = o_row_stride; p.o_hs = o_head_stride;
    p.dtype = dtype; p.B = B; p.n_keys = n_keys; p.heads = heads; p.head_dim = head_dim;
    p.offsets = offsets; p.l_max = l_max; p.max_q = max_q_per_image < l_max ? max_q_per_image : l_max;
    p.scale = scale; p.flags = flags;
    return vtp::attention(p, static_cast<cudaStream_t>(stream));
}
