// Internal interface of the Linear (GEMM + epilogue) kernels.
#pragma once

#include "common.cuh"

namespace vtp {

// y[out_row(m), n] = act(sum_k a[m,k] w[n,k] + bias[n]) + res[res_row(m), n]
//   out_row(m) = m + (m / out_grp + 1) * out_skip   when out_grp > 0, else m
//   res_row(m) = m % res_mod + res_off              when res_mod > 0, else m
// The row maps exist for the patch embedding, whose GEMM rows (b, t) land on token
// rows (b, 1 + t) and add the position embedding of token 1 + t.
struct LinearArgs {
    const void* a = nullptr; long long lda = 0;
    const void* w = nullptr;
    const float* bias = nullptr;
    const void* res = nullptr; long long ldr = 0;
    void* y = nullptr; long long ldy = 0;
    int dtype = VTP_F32;
    int m_max = 0; const int32_t* m_dev = nullptr;
    int N = 0, K = 0;
    unsigned flags = 0;
    int out_grp = 0, out_skip = 0;
    int res_mod = 0, res_off = 0;
};

int linear_validate(const LinearArgs& p);
int linear_cuda_cores(const LinearArgs& p, cudaStream_t st);   // fp32 or bf16 inputs, CUDA cores
int linear_tcgen05(const LinearArgs& p, cudaStream_t st);      // bf16 inputs, tcgen05 + TMA
int linear(const LinearArgs& p, cudaStream_t st);              // picks by dtype / flags

struct RowMap { int out_grp, out_skip, res_mod, res_off; };
__device__ __forceinline__ long long map_out_row(const RowMap& r, int m) {
    return r.out_grp > 0 ? (long long)m + (long long)(m / r.out_grp + 1) * r.out_skip : (long long)m;
}
__device__ __forceinline__ long long map_res_row(const RowMap& r, int m) {
    return r.res_mod > 0 ? (long long)(m % r.res_mod + r.res_off) : (long long)m;
}

}  // namespace vtp
