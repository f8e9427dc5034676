// Variable-length-query attention on CUDA cores, fp32 arithmetic (fp32 or bf16 storage).
// The fp32 product path, and an independent check of the tcgen05 kernel.
//
// One CTA owns 16 packed queries of one (image, head): scores for all keys are built in
// shared memory 64 keys at a time, a max-subtracted softmax runs over the whole row, then
// the probabilities are contracted with V 64 keys at a time.  Images with fewer queries
// simply launch CTAs that exit.
//
// Replaces batched_sparse_attention_forward
// (vtpack/layers/csrc/batched_sparse_gemm/batched_sparse_gemm.cu:219-305): scale is applied
// to Q K^T before the softmax exactly as the reference passes it as the GEMM alpha (:275).
#include "attention.h"
#include "runtime.h"

namespace vtp {

constexpr int AQ = 16;     // queries per CTA
constexpr int AD = 64;     // head dim
constexpr int AKC = 64;    // keys per chunk

template <typename T>
__global__ void __launch_bounds__(128)
attn_simt_kernel(const T* __restrict__ q, long long q_rs, long long q_hs, const T* __restrict__ k,
                 const T* __restrict__ v, long long kv_bs, long long kv_rs, long long kv_hs,
                 T* __restrict__ out, long long o_rs, long long o_hs, int n_keys, int n_keys_pad,
                 const int32_t* __restrict__ offsets, int l_max, float scale, int* status) {
    extern __shared__ float smem[];
    float* Qs = smem;                       // [AQ][AD]
    float* KV = Qs + AQ * AD;               // [AKC][AD + 1]
    float* S = KV + AKC * (AD + 1);         // [AQ][n_keys_pad]
    __shared__ float s_inv[AQ];

    const int b = blockIdx.z, h = blockIdx.y;
    const int row0 = __ldg(offsets + b) + blockIdx.x * AQ;
    int row_end = __ldg(offsets + b + 1);
#if VTP_INDEX_GUARDS
    // caller-supplied offsets: rows outside [0, l_max) are not touched
    if (row0 < 0 || row_end > l_max) {
        if (threadIdx.x == 0 && status) atomicOr(status, STATUS_BAD_INDEX);
        if (row0 < 0) return;
        row_end = l_max;
    }
#endif
    if (row0 >= row_end) return;
    const int nq = min(AQ, row_end - row0);
    const int tid = threadIdx.x;

    for (int e = tid; e < AQ * AD; e += 128) {
        const int i = e / AD, dd = e % AD;
        Qs[e] = i < nq ? to_f32(q[(size_t)(row0 + i) * q_rs + h * q_hs + dd]) : 0.f;
    }
    const T* kb = k + (size_t)b * kv_bs + h * kv_hs;
    const T* vb = v + (size_t)b * kv_bs + h * kv_hs;
    const int j = tid & 63, ig = tid >> 6;

    for (int c0 = 0; c0 < n_keys; c0 += AKC) {
        __syncthreads();
        for (int e = tid; e < AKC * AD; e += 128) {
            const int r = e / AD, dd = e % AD;
            KV[r * (AD + 1) + dd] = (c0 + r < n_keys) ? to_f32(kb[(size_t)(c0 + r) * kv_rs + dd]) : 0.f;
        }
        __syncthreads();
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
        for (int dd = 0; dd < AD; ++dd) {
            const float kv = KV[j * (AD + 1) + dd];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(Qs[(ig * 8 + i) * AD + dd], kv, acc[i]);
        }
        if (c0 + j < n_keys) {
#pragma unroll
            for (int i = 0; i < 8; ++i) S[(ig * 8 + i) * n_keys_pad + c0 + j] = acc[i] * scale;
        }
    }
    __syncthreads();
    {
        const int warp = tid >> 5, lane = tid & 31;
        for (int i = warp * 4; i < warp * 4 + 4; ++i) {
            float* row = S + (size_t)i * n_keys_pad;
            float mx = -INFINITY;
            for (int c = lane; c < n_keys; c += 32) mx = fmaxf(mx, row[c]);
            mx = warp_max(mx);
            float sum = 0.f;
            for (int c = lane; c < n_keys; c += 32) {
                const float p = expf(row[c] - mx);
                row[c] = p;
                sum += p;
            }
            sum = warp_sum(sum);
            if (lane == 0) s_inv[i] = 1.f / sum;
        }
    }
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int c0 = 0; c0 < n_keys; c0 += AKC) {
        __syncthreads();
        for (int e = tid; e < AKC * AD; e += 128) {
            const int r = e / AD, dd = e % AD;
            KV[r * (AD + 1) + dd] = (c0 + r < n_keys) ? to_f32(vb[(size_t)(c0 + r) * kv_rs + dd]) : 0.f;
        }
        __syncthreads();
        const int lim = min(AKC, n_keys - c0);
        for (int r = 0; r < lim; ++r) {
            const float vv = KV[r * (AD + 1) + j];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(S[(ig * 8 + i) * n_keys_pad + c0 + r], vv, acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int qi = ig * 8 + i;
        if (qi < nq) out[(size_t)(row0 + qi) * o_rs + h * o_hs + j] = from_f32<T>(acc[i] * s_inv[qi]);
    }
}

int attention_cuda_cores(const AttnArgs& p, cudaStream_t st) {
    VTP_REQUIRE(p.head_dim == AD, VTP_ERR_UNSUPPORTED, "attention: head_dim %d (only %d)", p.head_dim, AD);
    VTP_REQUIRE(p.B <= 65535 && p.heads <= 65535, VTP_ERR_SHAPE, "attention (CUDA cores): %d images x %d heads exceed the grid", p.B, p.heads);
    const int n_pad = (int)round_up(p.n_keys, 4) + 1;
    const size_t smem = (size_t)(AQ * AD + AKC * (AD + 1) + AQ * n_pad) * sizeof(float);
    VTP_REQUIRE(smem <= 200 * 1024, VTP_ERR_SHAPE, "attention: %d keys do not fit in shared memory", p.n_keys);
    // a query tile never straddles images; images with fewer queries launch CTAs that exit
    const dim3 grid(ceil_div(p.max_q, AQ), p.heads, p.B);
    cudaError_t e;
    if (p.dtype == VTP_F32) {
        e = cudaFuncSetAttribute(attn_simt_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            attn_simt_kernel<float><<<grid, 128, smem, st>>>(
                (const float*)p.q, p.q_rs, p.q_hs, (const float*)p.k, (const float*)p.v, p.kv_bs, p.kv_rs,
                p.kv_hs, (float*)p.out, p.o_rs, p.o_hs, p.n_keys, n_pad, p.offsets, p.l_max, p.scale, device_status_ptr());
    } else {
        e = cudaFuncSetAttribute(attn_simt_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            attn_simt_kernel<bf16><<<grid, 128, smem, st>>>(
                (const bf16*)p.q, p.q_rs, p.q_hs, (const bf16*)p.k, (const bf16*)p.v, p.kv_bs, p.kv_rs,
                p.kv_hs, (bf16*)p.out, p.o_rs, p.o_hs, p.n_keys, n_pad, p.offsets, p.l_max, p.scale, device_status_ptr());
    }
    if (e != cudaSuccess) {
        set_error("attention (CUDA cores): %s", cudaGetErrorString(e));
        return (int)e;
    }
    return check_launch("attention (CUDA cores)");
}

}  // namespace vtp
