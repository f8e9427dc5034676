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
    // LayerNorm folded into the GEMM (tcgen05 kernel only): `a` holds the raw rows, `w` holds
    // W*diag(gamma), ln_s[n] = sum_k w[n,k], bias[n] = sum_k beta[k] W[n,k] + b[n]; then
    //   LN(a) W^T + b = rstd[m] * (acc[m,n] - mean[m] * ln_s[n]) + bias[n].
    // ln_mode 1: ln_stats[m] = (mean, rstd).  ln_mode 2: ln_stats[m * STAT_SLOTS + i], i < ln_slots,
    // are partial (sum, sum of squares) over ln_dim elements in total (written by the GEMM that
    // produced the rows, see emit_stats); variance = E[x^2] - mean^2, rstd = rsqrt(var + ln_eps).
    const float2* ln_stats = nullptr; const float* ln_s = nullptr;
    int ln_mode = 0, ln_dim = 0, ln_slots = 0; float ln_eps = 0.f;
    // When set, every stored row leaves (sum, sum of squares) of its outputs here, one slot per
    // (column tile, epilogue warp): plain stores, so the result does not depend on timing.
    // linear_stat_slots(N) tells the consumer how many slots the producer fills.
    float2* emit_stats = nullptr;
};

constexpr int STAT_SLOTS = 16;      // float2 slots per row in a row-statistics buffer
int linear_stat_slots(int N);       // slots a tcgen05 GEMM with N output columns fills

struct LnFold { const float2* stats; const float* s; int mode, dim; float eps; float2* emit; int slots; };

int linear_validate(const LinearArgs& p);
int linear_cuda_cores(const LinearArgs& p, cudaStream_t st);   // fp32 or bf16 inputs, CUDA cores
int linear_tcgen05(const LinearArgs& p, cudaStream_t st);      // bf16 inputs, tcgen05 + TMA
int linear(const LinearArgs& p, cudaStream_t st);              // picks by dtype / flags
bool linear_pair_supported(const LinearArgs& a, const LinearArgs& b);
int linear_tcgen05_pair(const LinearArgs& a, const LinearArgs& b, cudaStream_t st);   // two problems, one launch

struct RowMap { int out_grp, out_skip, res_mod, res_off; };
__device__ __forceinline__ long long map_out_row(const RowMap& r, int m) {
    return r.out_grp > 0 ? (long long)m + (long long)(m / r.out_grp + 1) * r.out_skip : (long long)m;
}
__device__ __forceinline__ long long map_res_row(const RowMap& r, int m) {
    return r.res_mod > 0 ? (long long)(m % r.res_mod + r.res_off) : (long long)m;
}

}  // namespace vtp
