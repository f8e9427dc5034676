// Ragged batched matrix product on tcgen05 tensor cores (bf16 operands, fp32 accumulate).
//
// For every image i and head h:  out_i = op(a_i) * op(b_i)  (see ragged_gemm.cu for the operand
// conventions).  One CTA owns a 128-row x (up to 256-column) tile of one (image, head) product.
// The operands of the training path cannot be fetched by TMA: the score matrices have 257 columns
// (rows of 514 bytes, not 16-byte aligned), the reduction axis is the ragged one in half of the
// products, and half of the operands are needed transposed.  So all 256 threads of the CTA stage a
// 128 x 64 slice of op(a) and an N x 64 slice of op(b) into shared memory with plain loads, writing
// the K-major, 128-byte-swizzled image the tensor core expects (transposing on the way where op is a
// transpose, zero-filling beyond the ragged edges), two slices deep, while one thread issues
// tcgen05.mma on the slice before.  The accumulator (TMEM, up to 256 columns) leaves through shared
// memory so that every output row is written with consecutive lanes on consecutive elements, whatever
// the alignment of its 257-element rows.
//
// Replaces batched_sparse_gemm_forward (vtpack/layers/csrc/batched_sparse_gemm/batched_sparse_gemm.cu:
// 150-196: one library bmm per image and a concatenation) and serves its backward products
// (vtpack/layers/sparse_ops.py:30-55).
#include "common.cuh"
#include "runtime.h"
#include "sm100.cuh"

namespace vtp {

using namespace sm100;

constexpr int RT_M = 128;          // tile rows = TMEM lanes
constexpr int RT_N = 256;          // tile columns, upper bound
constexpr int RT_K = 64;           // reduction slice: one 128-byte swizzle row of bf16
constexpr int RT_THREADS = 256;
constexpr int RT_A_BYTES = RT_M * RT_K * 2;            // 16 KB
constexpr int RT_B_BYTES = RT_N * RT_K * 2;            // 32 KB
constexpr int RT_SMEM = 2 * (RT_A_BYTES + RT_B_BYTES) + 1024 + 256;

struct RaggedTcArgs {
    const bf16* a; const bf16* b; bf16* out;
    long long a_rows, b_rows, out_rows;
    int a_cols, b_cols, out_cols;
    const int32_t* a_off; const int32_t* b_off;
    int ta, tb, tiles_n;
};

// byte offset of element (r, k) of a K-major tile in the 128-byte-swizzled layout: rows of 64 bf16,
// eight-row groups of 1024 bytes, 16-byte chunks XORed with the row index
__device__ __forceinline__ uint32_t sw128_chunk(int r, int kchunk) {
    return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((kchunk ^ (r & 7)) << 4));
}

// Stages the slice op(src)(r0 .. r0 + R, k0 .. k0 + 64) into `dst`.  `trans` = 0: element (r, k) is
// src[r * ld + k] (k contiguous); 1: src[k * ld + r] (r contiguous).  Rows >= r_end and k >= k_end are zero.
// A thread owns up to MAXU units of (row, 16-byte chunk of 8 k); all its global loads are issued before the
// first shared-memory store, so a slice costs one memory latency, not one per unit.
template <int MAXU>
__device__ __forceinline__ void stage_slice(uint8_t* dst, const bf16* __restrict__ src, int ld, int trans, int R,
                                            int r0, int r_end, int k0, int k_end) {
    const int units = R * 8;
    const bool vec_ok = !trans && (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0) && (k0 % 8 == 0);
    uint4 v[MAXU];
#pragma unroll
    for (int i = 0; i < MAXU; ++i) {
        const int u = threadIdx.x + i * RT_THREADS;
        v[i] = make_uint4(0u, 0u, 0u, 0u);
        if (u >= units) continue;
        int r, kc;
        if (!trans) { kc = u & 7; r = u >> 3; }    // eight threads cover a 128-byte row piece
        else { r = u % R; kc = u / R; }            // consecutive threads read consecutive r
        const int gr = r0 + r, gk = k0 + kc * 8;
        if (gr < r_end && gk < k_end) {
            if (vec_ok && gk + 8 <= k_end) {
                v[i] = *reinterpret_cast<const uint4*>(src + (size_t)gr * ld + gk);
            } else {
                unsigned short e[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int k = gk + j;
                    const bf16* p = trans ? src + (size_t)k * ld + gr : src + (size_t)gr * ld + k;
                    e[j] = k < k_end ? *reinterpret_cast<const unsigned short*>(p) : (unsigned short)0;
                }
                v[i] = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
            }
        }
    }
#pragma unroll
    for (int i = 0; i < MAXU; ++i) {
        const int u = threadIdx.x + i * RT_THREADS;
        if (u >= units) continue;
        int r, kc;
        if (!trans) { kc = u & 7; r = u >> 3; }
        else { r = u % R; kc = u / R; }
        *reinterpret_cast<uint4*>(dst + sw128_chunk(r, kc)) = v[i];
    }
}

__global__ void __launch_bounds__(RT_THREADS, 2)
ragged_gemm_tc_kernel(RaggedTcArgs g, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sa = base;                                   // two A slices
    uint8_t* sb = base + 2 * RT_A_BYTES;                  // two B slices
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + 2 * (RT_A_BYTES + RT_B_BYTES));
    uint64_t* slice_done = bars;                          // [2] the MMAs that read a slice buffer have completed
    uint64_t* acc_full = bars + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int img = blockIdx.y, head = blockIdx.z;
    const int a0 = g.a_off[img], la = g.a_off[img + 1] - a0;
    const int b0 = g.b_off[img], lb = g.b_off[img + 1] - b0;
    const int M = g.ta ? g.a_cols : la;
    const int Ka = g.ta ? la : g.a_cols;
    const int Kb = g.tb ? g.b_cols : lb;
    const int K = min(Ka, Kb);
    const int N = min(g.tb ? lb : g.b_cols, g.out_cols);
    const int m0 = (blockIdx.x / g.tiles_n) * RT_M, n0 = (blockIdx.x % g.tiles_n) * RT_N;
    if (m0 >= M || n0 >= N) return;                       // uniform for the CTA: nothing allocated yet
    const int nt = min(RT_N, N - n0);                     // valid columns of this tile
    const int n_mma = (nt + 15) & ~15;                    // MMA width: a multiple of 16
    if (K <= 0) {
        // an empty reduction (an image without rows on the reduced axis): the product is zero
        const long long out_row0 = g.ta ? (long long)img * g.a_cols : (long long)a0;
        bf16* O = g.out + ((size_t)head * g.out_rows + out_row0) * g.out_cols;
        const int rows = min(RT_M, M - m0);
        for (int e = threadIdx.x; e < rows * nt; e += RT_THREADS)
            O[(size_t)(m0 + e / nt) * g.out_cols + n0 + e % nt] = __float2bfloat16_rn(0.f);
        return;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(&slice_done[0], 1); mbar_init(&slice_done[1], 1); mbar_init(acc_full, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, RT_N);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const bf16* A = g.a + ((size_t)head * g.a_rows + a0) * g.a_cols;     // [la][a_cols]
    const bf16* Bm = g.b + ((size_t)head * g.b_rows + b0) * g.b_cols;    // [lb][b_cols]
    const int n_slices = (K + RT_K - 1) / RT_K;
    const uint32_t idesc = idesc_bf16_f32(RT_M, n_mma, 0, 0);
    bool ok = true;
    for (int c = 0; c < n_slices && ok; ++c) {
        const int buf = c & 1, k0 = c * RT_K;
        // the MMAs of slice c - 2 have finished reading this buffer
        ok = mbar_wait(&slice_done[buf], ((c >> 1) & 1) ^ 1, abort_flag, status, STATUS_GEMM_PRODUCER);
        ok = __syncthreads_and(ok) != 0;                   // one verdict for the CTA: nobody is left at a barrier
        if (!ok) break;
        // op(a)(m, k): a not transposed -> a_i[m][k]; transposed -> a_i[k][m]
        stage_slice<RT_M * 8 / RT_THREADS>(sa + buf * RT_A_BYTES, A, g.a_cols, g.ta, RT_M, m0, M, k0, K);
        // op(b)(k, n) as rows n of a K-major tile: b transposed -> b_i[n][k]; not transposed -> b_i[k][n]
        stage_slice<RT_N * 8 / RT_THREADS>(sb + buf * RT_B_BYTES, Bm, g.b_cols, g.tb ? 0 : 1, n_mma, n0, N, k0, K);
        fence_proxy_async_smem();
        __syncthreads();
        if (threadIdx.x == 0) {
            tc_fence_after_sync();
            const uint64_t adesc = smem_desc_sw128(smem_u32(sa + buf * RT_A_BYTES));
            const uint64_t bdesc = smem_desc_sw128(smem_u32(sb + buf * RT_B_BYTES));
            const int ksteps = (min(RT_K, K - k0) + 15) / 16;
            for (int k = 0; k < ksteps; ++k)
                umma_ss(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (c | k) != 0 ? 1u : 0u);
            umma_commit(&slice_done[buf]);
            if (c == n_slices - 1) umma_commit(acc_full);
        }
    }
    ok = ok && mbar_wait(acc_full, 0, abort_flag, status, STATUS_GEMM_EPILOGUE);
    tc_fence_after_sync();
    ok = __syncthreads_and(ok) != 0;                       // every thread sees the same verdict below
    if (ok) {
        // ---- accumulator -> bf16 rows in shared memory (the slice buffers are free now), row pitch nt + 2
        bf16* stage = reinterpret_cast<bf16*>(base);
        const int pitch = RT_N + 2;
        const int row = (warp & 3) * 32 + lane;            // TMEM lane
        const int half = warp >> 2;                        // warps 0-3: columns [0, 128), warps 4-7: [128, 256)
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        for (int c0 = half * 128; c0 < min(n_mma, half * 128 + 128); c0 += 32) {
            uint32_t r[32];
            __syncwarp();
            tmem_ld_32x32(lane_base + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                *reinterpret_cast<__nv_bfloat162*>(stage + (size_t)row * pitch + c0 + i) = h2;
            }
        }
        tc_fence_before_sync();
        __syncthreads();
        // ---- rows out: consecutive lanes on consecutive elements of a row
        const long long out_row0 = g.ta ? (long long)img * g.a_cols : (long long)a0;
        bf16* O = g.out + ((size_t)head * g.out_rows + out_row0) * g.out_cols;
        const int rows = min(RT_M, M - m0);
        for (int rr = warp; rr < rows; rr += RT_THREADS / 32) {
            bf16* dst = O + (size_t)(m0 + rr) * g.out_cols + n0;
            const bf16* src = stage + (size_t)rr * pitch;
            for (int cc = lane; cc < nt; cc += 32) dst[cc] = src[cc];
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, RT_N);
}

int ragged_gemm_tcgen05(const void* a, const void* b, void* out, int heads, int n_images, long long a_rows,
                        int a_cols, long long b_rows, int b_cols, const int32_t* a_off, const int32_t* b_off,
                        int max_m, int max_n, int ta, int tb, long long out_rows, int out_cols, cudaStream_t st) {
    RaggedTcArgs g;
    g.a = static_cast<const bf16*>(a); g.b = static_cast<const bf16*>(b); g.out = static_cast<bf16*>(out);
    g.a_rows = a_rows; g.b_rows = b_rows; g.out_rows = out_rows;
    g.a_cols = a_cols; g.b_cols = b_cols; g.out_cols = out_cols;
    g.a_off = a_off; g.b_off = b_off; g.ta = ta; g.tb = tb;
    g.tiles_n = ceil_div(max_n, RT_N);
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(ragged_gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, RT_SMEM);
        if (e != cudaSuccess) return fail((int)e, "batched_sparse_gemm (tcgen05): shared memory: %s", cudaGetErrorString(e));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    const dim3 grid((unsigned)(ceil_div(max_m, RT_M) * g.tiles_n), (unsigned)n_images, (unsigned)heads);
    ragged_gemm_tc_kernel<<<grid, RT_THREADS, RT_SMEM, st>>>(g, device_status_ptr());
    return check_launch("batched_sparse_gemm (tcgen05)");
}

}  // namespace vtp
