// Ragged batched matrix product of the training path: for every image i and head h
//     out_i = op(a_i) * op(b_i),   a_i = a[h, a_off[i] : a_off[i+1], :],  b_i likewise,
// op = transpose when the matching flag is set, and the out_i stacked along the row axis.
// Replaces batched_sparse_gemm_forward (vtpack/layers/csrc/batched_sparse_gemm/
// batched_sparse_gemm.cu:150-196: a host loop of one bmm per image on pooled streams, then a
// concatenation) with one launch over (tile, image, head); the same entry point serves the
// backward products, which the reference also spells as forward calls with other transpose flags
// (vtpack/layers/sparse_ops.py:30-55).
//
// bf16 operands go to the tcgen05 kernel of ragged_gemm_tc.cu; fp32 operands (full-precision products)
// take the kernel in this file.  Shapes per (image, head) are small (about 113 x 257 x 64 in
// DeiT-S+DGE): a shared-memory tiled CUDA-core kernel: 64 x 64 output tile, 16-deep slices, 256 threads with a
// 4 x 4 accumulator block each, fp32 accumulation in slice order.  The loads walk whichever axis is
// contiguous in memory for the given transpose flag; row lengths need no alignment.
#include "common.cuh"

namespace vtp {

// bf16: the tensor-core kernel (ragged_gemm_tc.cu)
int ragged_gemm_tcgen05(const void* a, const void* b, void* out, int heads, int n_images, long long a_rows,
                        int a_cols, long long b_rows, int b_cols, const int32_t* a_off, const int32_t* b_off,
                        int max_m, int max_n, int ta, int tb, long long out_rows, int out_cols, cudaStream_t st);

constexpr int RG_TM = 64, RG_TN = 64, RG_TK = 16, RG_THREADS = 256;

struct RaggedGemmArgs {
    const void* a;
    const void* b;
    void* out;
    long long a_rows, b_rows, out_rows;
    int a_cols, b_cols, out_cols;
    const int32_t* a_off;
    const int32_t* b_off;
    int ta, tb;
    int tiles_n;
};

template <typename T>
__global__ void __launch_bounds__(RG_THREADS)
ragged_gemm_kernel(RaggedGemmArgs g) {
    __shared__ __align__(16) float As[RG_TK][RG_TM + 4];     // [k][m]
    __shared__ __align__(16) float Bs[RG_TK][RG_TN + 4];     // [k][n]
    const int img = blockIdx.y, head = blockIdx.z;
    const int a0 = g.a_off[img], la = g.a_off[img + 1] - a0;
    const int b0 = g.b_off[img], lb = g.b_off[img + 1] - b0;
    const int M = g.ta ? g.a_cols : la;
    const int Ka = g.ta ? la : g.a_cols;
    const int Kb = g.tb ? g.b_cols : lb;
    const int K = min(Ka, Kb);
    const int N = min(g.tb ? lb : g.b_cols, g.out_cols);
    const int m0 = (blockIdx.x / g.tiles_n) * RG_TM, n0 = (blockIdx.x % g.tiles_n) * RG_TN;
    if (m0 >= M || n0 >= N) return;

    const T* A = static_cast<const T*>(g.a) + ((size_t)head * g.a_rows + a0) * g.a_cols;   // [la][a_cols]
    const T* Bm = static_cast<const T*>(g.b) + ((size_t)head * g.b_rows + b0) * g.b_cols;  // [lb][b_cols]
    const long long out_row0 = g.ta ? (long long)img * g.a_cols : (long long)a0;
    T* O = static_cast<T*>(g.out) + ((size_t)head * g.out_rows + out_row0) * g.out_cols;

    const int t = threadIdx.x;
    const int tm = (t / 16) * 4, tn = (t % 16) * 4;          // this thread's 4 x 4 block of the tile
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += RG_TK) {
        // ---- A slice: op(a)(m, k)
        if (!g.ta) {                                          // a_i(m, k): k contiguous
            const int m = t / 4, kk = (t % 4) * 4;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int gm = m0 + m, gk = k0 + kk + j;
                As[kk + j][m] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * g.a_cols + gk]) : 0.f;
            }
        } else {                                              // a_i(k, m): m contiguous
            const int kk = t / 16, m = (t % 16) * 4;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int gm = m0 + m + j, gk = k0 + kk;
                As[kk][m + j] = (gm < M && gk < K) ? to_f32(A[(size_t)gk * g.a_cols + gm]) : 0.f;
            }
        }
        // ---- B slice: op(b)(k, n)
        if (!g.tb) {                                          // b_i(k, n): n contiguous
            const int kk = t / 16, n = (t % 16) * 4;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int gn = n0 + n + j, gk = k0 + kk;
                Bs[kk][n + j] = (gn < N && gk < K) ? to_f32(Bm[(size_t)gk * g.b_cols + gn]) : 0.f;
            }
        } else {                                              // b_i(n, k): k contiguous
            const int n = t / 4, kk = (t % 4) * 4;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int gn = n0 + n, gk = k0 + kk + j;
                Bs[kk + j][n] = (gn < N && gk < K) ? to_f32(Bm[(size_t)gn * g.b_cols + gk]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < RG_TK; ++kk) {
            const float4 av = *reinterpret_cast<const float4*>(&As[kk][tm]);
            const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tn]);
            const float ar[4] = {av.x, av.y, av.z, av.w};
            const float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + tm + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tn + j;
            if (gn < N) O[(size_t)gm * g.out_cols + gn] = from_f32<T>(acc[i][j]);
        }
    }
}

}  // namespace vtp

using namespace vtp;

extern "C" int vtp_batched_sparse_gemm(const void* a, const void* b, void* out, int dtype, int heads,
                                       int n_images, long long a_rows, int a_cols, long long b_rows,
                                       int b_cols, const int32_t* a_offsets, const int32_t* b_offsets,
                                       int max_a_len, int max_b_len, int a_transposed, int b_transposed,
                                       long long out_rows, int out_cols, void* stream) {
    VTP_REQUIRE(a && b && out && a_offsets && b_offsets, VTP_ERR_NULL, "batched_sparse_gemm: null pointer");
    VTP_REQUIRE(dtype == VTP_F32 || dtype == VTP_BF16, VTP_ERR_DTYPE, "batched_sparse_gemm: dtype %d", dtype);
    VTP_REQUIRE(heads > 0 && heads <= 65535 && n_images > 0 && n_images <= 65535 && a_rows >= 0 && b_rows >= 0 &&
                    a_cols > 0 && b_cols > 0 && out_rows >= 0 && out_cols > 0 && max_a_len >= 0 && max_b_len >= 0,
                VTP_ERR_SHAPE, "batched_sparse_gemm: bad shape");
    const int max_m = a_transposed ? a_cols : max_a_len;
    const int max_n = b_transposed ? max_b_len : b_cols;
    VTP_REQUIRE(max_n <= out_cols, VTP_ERR_SHAPE, "batched_sparse_gemm: %d output columns, buffer has %d", max_n,
                out_cols);
    if (max_m == 0 || max_n == 0 || out_rows == 0) return VTP_OK;
    // bf16 on tensor cores (operand arrays that start on a 16-byte boundary: the kernel fetches with aligned
    // 16-byte loads); fp32 keeps full-precision products on CUDA cores
    if (dtype == VTP_BF16 && aligned16(a) && aligned16(b))
        return ragged_gemm_tcgen05(a, b, out, heads, n_images, a_rows, a_cols, b_rows, b_cols, a_offsets, b_offsets,
                                   max_m, max_n, a_transposed ? 1 : 0, b_transposed ? 1 : 0, out_rows, out_cols,
                                   static_cast<cudaStream_t>(stream));
    RaggedGemmArgs g;
    g.a = a; g.b = b; g.out = out;
    g.a_rows = a_rows; g.b_rows = b_rows; g.out_rows = out_rows;
    g.a_cols = a_cols; g.b_cols = b_cols; g.out_cols = out_cols;
    g.a_off = a_offsets; g.b_off = b_offsets;
    g.ta = a_transposed ? 1 : 0; g.tb = b_transposed ? 1 : 0;
    g.tiles_n = ceil_div(max_n, RG_TN);
    const dim3 grid((unsigned)(ceil_div(max_m, RG_TM) * g.tiles_n), (unsigned)n_images, (unsigned)heads);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == VTP_F32) ragged_gemm_kernel<float><<<grid, RG_THREADS, 0, st>>>(g);
    else ragged_gemm_kernel<bf16><<<grid, RG_THREADS, 0, st>>>(g);
    return check_launch("batched_sparse_gemm");
}
