// Linear layer on CUDA cores: fp32 accumulate, fp32 or bf16 operands.  This is the fp32
// product path (the reference evaluates in fp32, vtpack/engine/engine.py:102-118) and an
// independent check of the tcgen05 kernel for bf16.
//
// Replaces nn.Linear + GELU + residual add (vtpack/models/dge/deit_dge.py:38-44,72-74,96,127-128).
#include "linear.h"

namespace vtp {

constexpr int SBM = 64, SBN = 64, SBK = 16;

template <typename T, typename OutT>
__global__ void __launch_bounds__(256)
linear_simt_kernel(const T* __restrict__ a, long long lda, const T* __restrict__ w,
                   const float* __restrict__ bias, const T* __restrict__ res, long long ldr,
                   OutT* __restrict__ y, long long ldy, int m_max, const int32_t* __restrict__ m_dev,
                   int N, int K, unsigned flags, RowMap rm) {
    __shared__ float As[SBK][SBM + 4];
    __shared__ float Bs[SBK][SBN + 4];
    int M = m_max;
    if (m_dev) M = min(__ldg(m_dev), m_max);
    const int m0 = blockIdx.y * SBM;
    const int n0 = blockIdx.x * SBN;
    if (m0 >= M) return;
    const int tid = threadIdx.x;
    const int lr = tid >> 2;          // tile row loaded by this thread
    const int lk = (tid & 3) * 4;     // first k of its 4-element slice
    const int ty = tid >> 4, tx = tid & 15;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += SBK) {
        float av[4] = {0.f, 0.f, 0.f, 0.f}, bv[4] = {0.f, 0.f, 0.f, 0.f};
        if (m0 + lr < M) {
            const T* p = a + (size_t)(m0 + lr) * lda + k0 + lk;
#pragma unroll
            for (int i = 0; i < 4; ++i) if (k0 + lk + i < K) av[i] = to_f32(p[i]);
        }
        if (n0 + lr < N) {
            const T* p = w + (size_t)(n0 + lr) * K + k0 + lk;
#pragma unroll
            for (int i = 0; i < 4; ++i) if (k0 + lk + i < K) bv[i] = to_f32(p[i]);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) { As[lk + i][lr] = av[i]; Bs[lk + i][lr] = bv[i]; }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < SBK; ++k) {
            const float4 a4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 b4 = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
            const float ar[4] = {a4.x, a4.y, a4.z, a4.w};
            const float br[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
        const long long orow = map_out_row(rm, m);
        const long long rrow = map_res_row(rm, m);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += __ldg(bias + n);
            if (flags & VTP_FLAG_GELU) v = gelu_erf(v);
            if (res) v += to_f32(res[rrow * ldr + n]);
            y[orow * ldy + n] = from_f32<OutT>(v);
        }
    }
}

int linear_cuda_cores(const LinearArgs& p, cudaStream_t st) {
    if (p.m_max == 0) return VTP_OK;
    const dim3 grid(ceil_div(p.N, SBN), ceil_div(p.m_max, SBM));
    const RowMap rm{p.out_grp, p.out_skip, p.res_mod, p.res_off};
    if (p.dtype == VTP_F32) {
        linear_simt_kernel<float, float><<<grid, 256, 0, st>>>(
            (const float*)p.a, p.lda, (const float*)p.w, p.bias, (const float*)p.res, p.ldr,
            (float*)p.y, p.ldy, p.m_max, p.m_dev, p.N, p.K, p.flags, rm);
    } else if (p.flags & VTP_FLAG_OUT_F32) {
        linear_simt_kernel<bf16, float><<<grid, 256, 0, st>>>(
            (const bf16*)p.a, p.lda, (const bf16*)p.w, p.bias, (const bf16*)p.res, p.ldr,
            (float*)p.y, p.ldy, p.m_max, p.m_dev, p.N, p.K, p.flags, rm);
    } else {
        linear_simt_kernel<bf16, bf16><<<grid, 256, 0, st>>>(
            (const bf16*)p.a, p.lda, (const bf16*)p.w, p.bias, (const bf16*)p.res, p.ldr,
            (bf16*)p.y, p.ldy, p.m_max, p.m_dev, p.N, p.K, p.flags, rm);
    }
    return check_launch("linear (CUDA cores)");
}

}  // namespace vtp
