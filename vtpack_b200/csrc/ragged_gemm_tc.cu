// Ragged batched matrix product on tcgen05 tensor cores (bf16 operands, fp32 accumulate).
//
// For every image i and head h:  out_i = op(a_i) * op(b_i)  (see ragged_gemm.cu for the operand
// conventions).  One CTA owns a 128-row x (up to 256-column) tile of one (image, head) product.
// The operands of the training path cannot be fetched by TMA: the score matrices have 257 columns
// (rows of 514 bytes, not 16-byte aligned) and the reduction axis is the ragged one in half of the
// products.  So the CTA's 256 threads stage the operands themselves, always as ROW TILES: R rows of 64
// consecutive elements of the operand as it lies in memory, written as the 128-byte-swizzled image the
// tensor core reads.  Nothing is transposed in software: an operand whose rows run along the reduction
// axis is a K-major tile, one whose rows run along M or N is an MN-major tile, and the instruction
// descriptor says which.  A row that does not start on a 16-byte boundary is fetched with aligned
// 16-byte loads and shifted into place in registers.  Two slices are staged per buffer pair, so the
// loads of slice c+1 run while the MMAs of slice c do.
//
// 257 = 256 + 1: a score product (K-major b) whose width exceeds the tile by at most RT_TAIL columns
// keeps those columns in the same CTA, as dot products on CUDA cores from the staged slices, so the tile
// owns whole output rows.  A tile of whole rows is one contiguous range of the output whatever the
// alignment of its rows: it leaves through a flat image in shared memory as aligned 16-byte stores.
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
constexpr int RT_N = 256;          // tile columns on the tensor core, upper bound
constexpr int RT_TAIL = 8;         // further columns a tile may take on CUDA cores (K-major b only)
constexpr int RT_K = 64;           // reduction slice: one 128-byte swizzle row of bf16
constexpr int RT_THREADS = 256;
constexpr int RT_A_BYTES = RT_M * RT_K * 2;                    // 16 KB
constexpr int RT_B_BYTES = (RT_N + RT_TAIL + 8) * RT_K * 2;    // 34 KB (a multiple of 1024)
// Resident a: where the tile's rows of a (rows of 257 elements, say) fit into shared memory as they lie in
// memory, they are fetched ONCE, as one contiguous range with 16-byte asynchronous copies, and every slice is
// cut out of that image; reading 128-byte pieces of 514-byte rows slice by slice costs a memory round trip per
// slice and uses DRAM badly.  The image lies behind the two a slices and ONE b slice of 64 rows (with two, and
// the shared memory that leaves two CTAs per SM used to the last KB, the products measured 12 % slower).
constexpr int RT_RAW_OFF = 2 * RT_A_BYTES + 64 * 128;
constexpr int RT_RAW_BYTES = RT_M * 257 * 2 + 32;              // 128 rows of 257 elements, shifted by up to 7
constexpr int RT_BAR_OFF = (2 * (RT_A_BYTES + RT_B_BYTES) > RT_RAW_OFF + RT_RAW_BYTES) ? 2 * (RT_A_BYTES + RT_B_BYTES)
                                                                                        : RT_RAW_OFF + RT_RAW_BYTES;
constexpr int RT_USED = RT_BAR_OFF + 256;
// Dynamic shared memory is only promised 16-byte alignment and the buffers want 1024; in practice the base is
// aligned already.  What two CTAs per SM leave is requested, and the kernel checks that its layout fits.
constexpr int RT_SMEM = (RT_USED + 1024 <= 233472 / 2 - 1024) ? RT_USED + 1024 : 233472 / 2 - 1024;
static_assert(RT_RAW_BYTES % 16 == 0 && RT_USED <= RT_SMEM, "two CTAs per SM");
constexpr int RT_ATOM_BYTES = RT_K * 128;                      // one MN-major atom column: 64 k rows of 128 bytes
constexpr int RT_BSUB_MAX = (RT_N + RT_TAIL + 63) / 64;        // 64-row sub-tiles of a b slice, at most
static_assert(RT_B_BYTES % 1024 == 0, "slice buffers stay 1024-byte aligned");

struct RaggedTcArgs {
    const bf16* a; const bf16* b; bf16* out;
    long long a_rows, b_rows, out_rows;
    int a_cols, b_cols, out_cols;
    const int32_t* a_off; const int32_t* b_off;
    int ta, tb, tiles_n, absorb_tail;
    int heads;
};

// byte offset of the 16-byte chunk (row r, chunk c) of a tile of 128-byte rows in the 128-byte-swizzled
// layout: eight-row groups of 1024 bytes, chunks XORed with the row index
__device__ __forceinline__ uint32_t sw128_chunk(int r, int c) {
    return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}

// Shifts the 32 bytes (lo, hi) right by `sh` bf16 elements (0..7) and returns the low 16 bytes.
__device__ __forceinline__ uint4 shift_elems(uint4 lo, uint4 hi, int sh) {
    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    const uint32_t bs = (sh & 1) * 16;                 // half a word or not, after ...
    uint32_t o[4];
    switch (sh >> 1) {                                 // ... the whole 32-bit words
        case 0:
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = __funnelshift_r(w[j], w[j + 1], bs);
            break;
        case 1:
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = __funnelshift_r(w[j + 1], w[j + 2], bs);
            break;
        case 2:
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = __funnelshift_r(w[j + 2], w[j + 3], bs);
            break;
        default:
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = __funnelshift_r(w[j + 3], w[j + 4 < 8 ? j + 4 : 7], bs);
            break;
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// keeps the first `n` (0..8) bf16 of the vector, zeroes the rest
__device__ __forceinline__ uint4 keep_first(uint4 v, int n) {
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (n <= 2 * j) w[j] = 0u;
        else if (n == 2 * j + 1) w[j] &= 0xFFFFu;
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// 16 bytes through L2 only (with two 104 KB CTAs on the SM the L1 is a few KB), or zeros: a predicated
// load, no branch, so that a run of them is issued back to back
__device__ __forceinline__ uint4 ldcg_if(const bf16* p, bool on) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];\n\t}"
        : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
        : "l"(p), "r"((int)on));
    return v;
}

// A sub-tile: 64 rows of 64 consecutive elements of an operand as it lies in memory, element (r, c) =
// src[base + (r0 + r) * ld + c0 + c]; rows at or beyond r_end and columns at or beyond c_end read as zero.
// It becomes 64 swizzled 128-byte rows (8 KB) of a slice buffer: half of a K-major A tile, one 64-column
// atom of an MN-major operand, 64 rows of a K-major B tile.
struct SubTile { long long base; int r0, r_end, c0, c_end; int rows; };   // rows: how many of the 64 the buffer has room for
constexpr int RT_SUB_BYTES = 64 * 128;

// A thread owns two (row, 16-byte chunk) units of a sub-tile.  issue: the global loads, predicated, nothing
// that looks at what they return, so the loads of every sub-tile of a slice are in flight together and a
// slice costs one memory latency.  Rows that start on 16-byte boundaries (a property of the sub-tile) take one
// load per unit; others (WITH_HI) the two aligned vectors around the unit, shifted into place by commit.  The
// last vectors of the array, where an aligned load would read beyond its end, are fetched element by element.
__device__ __forceinline__ bool subtile_aligned(const SubTile& t, int ld) {
    return (ld % 8 == 0) && ((t.base + (long long)t.r0 * ld + t.c0) % 8 == 0);
}
template <bool WITH_HI>
__device__ __forceinline__ void issue_subtile(uint4 (&lo)[2], uint4 (&hi)[2], const bf16* __restrict__ src,
                                              long long total, int ld, const SubTile& t, bool on) {
    const bool al = subtile_aligned(t, ld);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int u = threadIdx.x + i * RT_THREADS;
        const int gr = t.r0 + (u >> 3), gc = t.c0 + (u & 7) * 8;   // eight threads cover a 128-byte row piece
        const long long e0 = (t.base + (long long)gr * ld + gc) & ~7LL;
        const bool fast = on && (u >> 3) < t.rows && gr < t.r_end && gc < t.c_end && e0 + (al ? 8 : 16) <= total;
        lo[i] = ldcg_if(src + e0, fast);
        if (WITH_HI) hi[i] = ldcg_if(src + e0 + 8, fast && !al);
    }
}
template <bool WITH_HI>
__device__ __forceinline__ void commit_subtile(const uint4 (&lo)[2], const uint4 (&hi)[2], uint8_t* dst,
                                               const bf16* __restrict__ src, long long total, int ld,
                                               const SubTile& t, bool on) {
    if (!on) return;
    const bool al = subtile_aligned(t, ld);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int u = threadIdx.x + i * RT_THREADS;
        if ((u >> 3) >= t.rows) continue;
        const int gr = t.r0 + (u >> 3), gc = t.c0 + (u & 7) * 8;
        const long long e = t.base + (long long)gr * ld + gc;
        const bool in_tile = gr < t.r_end && gc < t.c_end;
        uint4 v = (al || !WITH_HI) ? lo[i] : shift_elems(lo[i], hi[i], (int)(e & 7));
        if (in_tile && (e & ~7LL) + (al ? 8 : 16) > total) {       // the end of the array: nothing read beyond it
            unsigned short h[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                h[j] = (e + j < total) ? *reinterpret_cast<const unsigned short*>(src + e + j) : (unsigned short)0;
            v = make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
        }
        if (in_tile && gc + 8 > t.c_end) v = keep_first(v, t.c_end - gc);
        *reinterpret_cast<uint4*>(dst + sw128_chunk(u >> 3, u & 7)) = v;
    }
}

// shared-memory descriptor of a swizzled tile of 128-byte rows whose 64-element atoms along M / N (MN-major
// operands wider than 64) lie RT_ATOM_BYTES apart
__device__ __forceinline__ uint64_t ragged_desc(uint32_t saddr) {
    uint64_t d = smem_desc_sw128(saddr);
    d &= ~(static_cast<uint64_t>(0x3FFF) << 16);
    d |= static_cast<uint64_t>(RT_ATOM_BYTES >> 4) << 16;      // leading byte offset: atom to atom along M / N
    return d;
}

// A_HI: rows of a may start off 16-byte boundaries (two loads per unit, shifted in registers); RT_BSUB: how
// many 64-row sub-tiles a slice of b can have.  Template parameters because they size the register arrays
// that hold a slice's loads in flight: the common products need far fewer than the general case.
template <bool A_HI, int RT_BSUB>
__global__ void __launch_bounds__(RT_THREADS, 2)
ragged_gemm_tc_kernel(RaggedTcArgs g, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sa = base;                                   // two A slices
    uint8_t* sb = base + 2 * RT_A_BYTES;                  // two B slices
    if (static_cast<int>(base - smem_raw) + RT_USED > RT_SMEM) {
        if (threadIdx.x == 0 && status) atomicOr(status, STATUS_GEMM_PRODUCER);
        return;
    }
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + RT_BAR_OFF);
    uint64_t* slice_done = bars;                          // [2] the MMAs that read a slice buffer have completed
    uint64_t* acc_full = bars + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // [128][RT_TAIL] partial tail dots of the upper thread half, exchanged after the last MMA (in the end of the
    // second B slice buffer, beyond what the output image needs)
    float* tail_part = reinterpret_cast<float*>(base + 2 * (RT_A_BYTES + RT_B_BYTES) - RT_M * RT_TAIL * 4);

    const int img = blockIdx.y, head = blockIdx.z;
    const int a0 = g.a_off[img], la = g.a_off[img + 1] - a0;
    const int b0 = g.b_off[img], lb = g.b_off[img + 1] - b0;
    const int M = g.ta ? g.a_cols : la;
    const int Ka = g.ta ? la : g.a_cols;
    const int Kb = g.tb ? g.b_cols : lb;
    const int K = min(Ka, Kb);
    const int N = min(g.tb ? lb : g.b_cols, g.out_cols);
    const int nti = blockIdx.x % g.tiles_n;
    const int m0 = (blockIdx.x / g.tiles_n) * RT_M, n0 = nti * RT_N;
    if (m0 >= M || n0 >= N) return;                       // uniform for the CTA: nothing allocated yet
    const int nt = min(RT_N, N - n0);                     // columns of this tile on the tensor core
    const int n_mma = (nt + 15) & ~15;                    // MMA width: a multiple of 16
    // columns beyond the tensor-core tile that this CTA also takes (the last tile of a K-major b)
    const int ntail = (g.absorb_tail && nti == g.tiles_n - 1) ? max(0, min(RT_TAIL, N - n0 - RT_N)) : 0;
    const int rows = min(RT_M, M - m0);
    const long long out_row0 = g.ta ? (long long)img * g.a_cols : (long long)a0;
    bf16* O = g.out + ((size_t)head * g.out_rows + out_row0) * g.out_cols;
    if (K <= 0) {
        // an empty reduction (an image without rows on the reduced axis): the product is zero
        const int wdt = nt + ntail;
        for (int e = threadIdx.x; e < rows * wdt; e += RT_THREADS)
            O[(size_t)(m0 + e / wdt) * g.out_cols + n0 + e % wdt] = __float2bfloat16_rn(0.f);
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

    // the operand arrays as a whole (for the bounds of the aligned loads) and this image's first row in them
    const long long a_total = (long long)g.heads * g.a_rows * g.a_cols, b_total = (long long)g.heads * g.b_rows * g.b_cols;
    const long long a_base = ((long long)head * g.a_rows + a0) * g.a_cols;
    const long long b_base = ((long long)head * g.b_rows + b0) * g.b_cols;
    const int n_slices = (K + RT_K - 1) / RT_K;
    // a transposed: rows of a run along M (MN-major A); b not transposed: rows of b run along N (MN-major B)
    const uint32_t idesc = idesc_bf16_f32(RT_M, n_mma, g.ta ? 1 : 0, g.tb ? 0 : 1);
    const int b_rows_staged = ntail ? RT_N + RT_TAIL : n_mma;      // K-major b: the tile's rows, then the tail's
    // every row of b starts on a 16-byte boundary (true of the model's products: b is K, V, dO or Q)
    const bool b_all_aligned = g.b_cols % 8 == 0;
    float tail_acc[RT_TAIL];
#pragma unroll
    for (int j = 0; j < RT_TAIL; ++j) tail_acc[j] = 0.f;
    // ---- resident a (see RT_RAW_OFF): the tile's rows of a as one contiguous range, copied asynchronously
    const bool resident = A_HI && RT_BSUB == 1 && !g.ta && (long long)rows * g.a_cols * 2 + 32 <= RT_RAW_BYTES;
    uint8_t* raw = base + RT_RAW_OFF;
    int rshift = 0;                                        // elements between the image's start and the tile's first
    if (resident) {
        const long long e_first = a_base + (long long)m0 * g.a_cols;
        const long long e0 = e_first & ~7LL;
        rshift = (int)(e_first - e0);
        const int nvec = (rshift + rows * g.a_cols + 7) >> 3;
        for (int v = threadIdx.x; v < nvec; v += RT_THREADS) {
            const long long e = e0 + 8LL * v;
            if (e + 8 <= a_total) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(raw + 16 * v)), "l"(g.a + e) : "memory");
            } else {                                       // the end of the array: nothing read beyond it
                unsigned short h[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    h[j] = (e + j < a_total) ? *reinterpret_cast<const unsigned short*>(g.a + e + j) : (unsigned short)0;
                *reinterpret_cast<uint4*>(raw + 16 * v) =
                    make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // resident a: the (single, 64-row) b sub-tile of slice c + 1 is requested while slice c is being put together,
    // so that no slice waits for global memory
    auto b_sub0 = [&](int k0) {
        return g.tb ? SubTile{b_base, n0, N, k0, K, 64} : SubTile{b_base, k0, K, n0, N, 64};
    };
    uint4 bnext[2], bnext_hi[2];
    if (resident && b_all_aligned) issue_subtile<false>(bnext, bnext_hi, g.b, b_total, g.b_cols, b_sub0(0), true);
    bool ok = true;
    for (int c = 0; c < n_slices && ok; ++c) {
        const int buf = c & 1, k0 = c * RT_K;
        // the MMAs of slice c - 2 have finished reading this buffer (resident a: those of slice c - 1, whose b
        // slice lies in the one b buffer there is)
        if (resident) {
            if (c > 0) ok = mbar_wait(&slice_done[(c - 1) & 1], ((c - 1) >> 1) & 1, abort_flag, status, STATUS_GEMM_PRODUCER);
        } else {
            ok = mbar_wait(&slice_done[buf], ((c >> 1) & 1) ^ 1, abort_flag, status, STATUS_GEMM_PRODUCER);
        }
        ok = __syncthreads_and(ok) != 0;                   // one verdict for the CTA: nobody is left at a barrier
        if (!ok) break;
        uint8_t* sa_c = sa + buf * RT_A_BYTES;
        uint8_t* sb_c = resident ? sb : sb + buf * RT_B_BYTES;
        // the slice as sub-tiles of 64 rows x 64 elements (8 KB each): two of a, up to RT_BSUB of b
        SubTile at[2], bt[RT_BSUB];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            if (!g.ta) at[j] = SubTile{a_base, m0 + 64 * j, M, k0, K, 64};        // a_i[m][k]: rows m, columns k
            else at[j] = SubTile{a_base, k0, K, m0 + 64 * j, M, 64};              // a_i[k][m]: rows k, one 64-column atom each
        }
        const int nb = g.tb ? (b_rows_staged + 63) >> 6 : (n_mma + 63) >> 6;
#pragma unroll
        for (int j = 0; j < RT_BSUB; ++j) {
            if (g.tb) bt[j] = SubTile{b_base, n0 + 64 * j, N, k0, K, min(64, RT_N + RT_TAIL + 8 - 64 * j)};         // b_i[n][k]: rows n (the tile's, then the tail's)
            else bt[j] = SubTile{b_base, k0, K, n0 + 64 * j, N, 64};              // b_i[k][n]: rows k, one 64-column atom each
        }
        {
            uint4 alo[2][2], ahi[A_HI ? 2 : 1][2], blo[RT_BSUB][2], bhi[1][2];
#pragma unroll
            for (int j = 0; j < 2; ++j) issue_subtile<A_HI>(alo[j], ahi[A_HI ? j : 0], g.a, a_total, g.a_cols, at[j], !resident);
            const bool b_ahead = resident && b_all_aligned;       // this slice's b is in registers already
            if (b_ahead) {
                commit_subtile<false>(bnext, bnext_hi, sb_c, g.b, b_total, g.b_cols, bt[0], true);
                issue_subtile<false>(bnext, bnext_hi, g.b, b_total, g.b_cols, b_sub0(k0 + RT_K), c + 1 < n_slices);
            } else if (b_all_aligned) {
#pragma unroll
                for (int j = 0; j < RT_BSUB; ++j) issue_subtile<false>(blo[j], bhi[0], g.b, b_total, g.b_cols, bt[j], j < nb);
            }
#pragma unroll
            for (int j = 0; j < 2; ++j)
                commit_subtile<A_HI>(alo[j], ahi[A_HI ? j : 0], sa_c + j * RT_SUB_BYTES, g.a, a_total, g.a_cols, at[j], !resident);
            if (resident) {
                if (c == 0) {                              // the image has landed, for every thread
                    asm volatile("cp.async.wait_group 0;" ::: "memory");
                    __syncthreads();
                }
                // the slice of a out of the image: the two aligned vectors around each unit, shifted into place
#pragma unroll
                for (int i = 0; i < RT_M * 8 / RT_THREADS; ++i) {
                    const int u = threadIdx.x + i * RT_THREADS;
                    const int r = u >> 3, gk = k0 + (u & 7) * 8;
                    uint4 v = make_uint4(0u, 0u, 0u, 0u);
                    if (r < rows && gk < K) {
                        const int eoff = rshift + r * g.a_cols + gk;
                        const uint4* rv = reinterpret_cast<const uint4*>(raw) + (eoff >> 3);
                        v = shift_elems(rv[0], rv[1], eoff & 7);
                        if (gk + 8 > K) v = keep_first(v, K - gk);
                    }
                    *reinterpret_cast<uint4*>(sa_c + sw128_chunk(r, u & 7)) = v;
                }
            }
            if (b_ahead) {
                // committed above
            } else if (b_all_aligned) {
#pragma unroll
                for (int j = 0; j < RT_BSUB; ++j)
                    commit_subtile<false>(blo[j], bhi[0], sb_c + j * RT_SUB_BYTES, g.b, b_total, g.b_cols, bt[j], j < nb);
            } else {
                // rows of b that do not start on 16-byte boundaries: one sub-tile after the other
#pragma unroll
                for (int j = 0; j < RT_BSUB; ++j) {
                    uint4 lo[2], hi[2];
                    issue_subtile<true>(lo, hi, g.b, b_total, g.b_cols, bt[j], j < nb);
                    commit_subtile<true>(lo, hi, sb_c + j * RT_SUB_BYTES, g.b, b_total, g.b_cols, bt[j], j < nb);
                }
            }
        }
        fence_proxy_async_smem();
        __syncthreads();
        if (threadIdx.x == 0) {
            tc_fence_after_sync();
            const uint64_t adesc = ragged_desc(smem_u32(sa_c));
            const uint64_t bdesc = ragged_desc(smem_u32(sb_c));
            const int ksteps = (min(RT_K, K - k0) + 15) / 16;
            // 16 reduction steps further on: 32 bytes inside the row of a K-major tile, 16 rows of an MN-major one
            const uint64_t a_step = g.ta ? (16 * 128) >> 4 : 2, b_step = g.tb ? 2 : (16 * 128) >> 4;
            for (int k = 0; k < ksteps; ++k)
                umma_ss(tmem_base, adesc + a_step * k, bdesc + b_step * k, idesc, (c | k) != 0 ? 1u : 0u);
            umma_commit(&slice_done[buf]);
            if (c == n_slices - 1) umma_commit(acc_full);
        }
        if (ntail) {
            // tail columns: row r = thread % 128 of a (K-major here), k half = thread / 128
            const int r = threadIdx.x & 127, kh = threadIdx.x >> 7;
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                const int kc = kh * 4 + cc;
                const uint4 av = *reinterpret_cast<const uint4*>(sa_c + sw128_chunk(r, kc));
                float af[8];
                Vec<bf16> avv; avv.raw = av; avv.to_float(af);
#pragma unroll
                for (int j = 0; j < RT_TAIL; ++j) {
                    if (j < ntail) {
                        const uint4 bv = *reinterpret_cast<const uint4*>(sb_c + sw128_chunk(RT_N + j, kc));
                        float bf[8];
                        Vec<bf16> bvv; bvv.raw = bv; bvv.to_float(bf);
#pragma unroll
                        for (int i = 0; i < 8; ++i) tail_acc[j] = fmaf(af[i], bf[i], tail_acc[j]);
                    }
                }
            }
        }
    }
    ok = ok && mbar_wait(acc_full, 0, abort_flag, status, STATUS_GEMM_EPILOGUE);
    tc_fence_after_sync();
    ok = __syncthreads_and(ok) != 0;                       // every thread sees the same verdict below
    if (ok) {
        if (ntail) {                                       // the two k halves of the tail dots meet
            const int r = threadIdx.x & 127;
            if (threadIdx.x >= 128) {
#pragma unroll
                for (int j = 0; j < RT_TAIL; ++j) tail_part[r * RT_TAIL + j] = tail_acc[j];
            }
            __syncthreads();
            if (threadIdx.x < 128) {
#pragma unroll
                for (int j = 0; j < RT_TAIL; ++j) tail_acc[j] += tail_part[r * RT_TAIL + j];
            }
        }
        // ---- accumulator -> bf16 image of the tile's output in shared memory (the slice buffers are free now),
        // then out.  Three forms: rows that start on 16-byte boundaries (image rows padded to an odd number of
        // 16-byte chunks, 16-byte accesses throughout); whole rows of any pitch (the tile is one contiguous range
        // of the output: a flat image, shifted so that 16-byte vectors of the image are 16-byte vectors of the
        // output); anything else row by row, two bytes per lane.
        const int wdt = nt + ntail;                        // columns this CTA writes
        const bool out_aligned = (reinterpret_cast<uintptr_t>(g.out) & 15) == 0;
        const bool rows_aligned = out_aligned && g.out_cols % 8 == 0 && ntail == 0;
        const bool whole_rows = !rows_aligned && out_aligned && n0 == 0 && wdt == g.out_cols;
        // element offset of the tile's first element in `out`, and how far it sits into a 16-byte vector
        const long long g0 = ((long long)head * g.out_rows + out_row0 + m0) * g.out_cols + n0;
        const int shift = whole_rows ? (int)(g0 & 7) : 0;
        const int pitch = rows_aligned ? (((n_mma + 7) & ~7) + 8) | 8      // an odd number of 8-element chunks
                          : whole_rows ? wdt : RT_N + RT_TAIL + 2;
        bf16* stage = reinterpret_cast<bf16*>(base);
        const int row = (warp & 3) * 32 + lane;            // TMEM lane
        const int half = warp >> 2;                        // warps 0-3: columns [0, 128), warps 4-7: [128, 256)
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        unsigned short* srow = reinterpret_cast<unsigned short*>(stage) + shift + (size_t)row * pitch;
        for (int c0 = half * 128; c0 < min(n_mma, half * 128 + 128); c0 += 32) {
            uint32_t r[32];
            __syncwarp();
            tmem_ld_32x32(lane_base + c0, r);
            tmem_ld_wait();
            if (row >= rows) continue;
            unsigned short* p = srow + c0;
            const int nvalid = min(32, nt - c0);           // columns of this chunk that exist
            if (rows_aligned) {
                // whole 16-byte chunks; what lies beyond the row's last column stays in the padding
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    if (8 * v < nvalid) {
                        float f[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[8 * v + i]);
                        Vec<bf16> ov;
                        ov.from_float(f);
                        *reinterpret_cast<uint4*>(p + 8 * v) = ov.raw;
                    }
                }
            } else {
                // pairs of columns as 32-bit stores; a row that starts on an odd element of the image stores one
                // element first and pairs one column further on.  Whole chunks take the unguarded form.
                const bool odd = (reinterpret_cast<uintptr_t>(p) & 3) != 0;
                auto bf = [&](int i) { return __bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(r[i]))); };
                if (nvalid >= 32) {
                    if (!odd) {
#pragma unroll
                        for (int i = 0; i < 32; i += 2)
                            *reinterpret_cast<__nv_bfloat162*>(p + i) =
                                __floats2bfloat162_rn(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                    } else {
                        p[0] = bf(0);
#pragma unroll
                        for (int i = 1; i < 31; i += 2)
                            *reinterpret_cast<__nv_bfloat162*>(p + i) =
                                __floats2bfloat162_rn(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                        p[31] = bf(31);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (i < nvalid) p[i] = bf(i);
                }
            }
        }
        if (ntail && threadIdx.x < 128 && threadIdx.x < rows) {
            unsigned short* p = reinterpret_cast<unsigned short*>(stage) + shift + (size_t)threadIdx.x * pitch + RT_N;
#pragma unroll
            for (int j = 0; j < RT_TAIL; ++j)
                if (j < ntail) p[j] = __bfloat16_as_ushort(__float2bfloat16_rn(tail_acc[j]));
        }
        tc_fence_before_sync();
        __syncthreads();
        const unsigned short* simg = reinterpret_cast<const unsigned short*>(stage);
        if (rows_aligned) {
            const int vpr = (nt + 7) >> 3;                                 // vectors per row
            for (int idx = threadIdx.x; idx < rows * vpr; idx += RT_THREADS) {
                const int rr = idx / vpr, v = idx % vpr;
                unsigned short* dst = reinterpret_cast<unsigned short*>(O + (size_t)(m0 + rr) * g.out_cols + n0) + 8 * v;
                const unsigned short* src = simg + (size_t)rr * pitch + 8 * v;
                if (8 * v + 8 <= nt) {
                    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
                } else {
                    for (int j = 0; 8 * v + j < nt; ++j) dst[j] = src[j];
                }
            }
        } else if (whole_rows) {
            // flat copy: vector v of the image <-> elements g0 - shift + 8 v .. + 8 of the output
            const long long total = (long long)rows * wdt;                 // elements of the tile
            const int nvec = (int)((shift + total + 7) >> 3);
            bf16* gvec = g.out + (g0 - shift);
            for (int v = threadIdx.x; v < nvec; v += RT_THREADS) {
                const long long e_lo = (long long)v * 8 - shift;           // tile element of the vector's first lane
                if (e_lo >= 0 && e_lo + 8 <= total) {
                    *reinterpret_cast<uint4*>(gvec + (size_t)v * 8) = *reinterpret_cast<const uint4*>(simg + (size_t)v * 8);
                } else {
                    for (int j = 0; j < 8; ++j)
                        if (e_lo + j >= 0 && e_lo + j < total)
                            reinterpret_cast<unsigned short*>(gvec)[(size_t)v * 8 + j] = simg[(size_t)v * 8 + j];
                }
            }
        } else {
            // rows out one by one: consecutive lanes on consecutive elements of a row
            for (int rr = warp; rr < rows; rr += RT_THREADS / 32) {
                bf16* dst = O + (size_t)(m0 + rr) * g.out_cols + n0;
                const bf16* src = stage + (size_t)rr * pitch;
                for (int cc = lane; cc < wdt; cc += 32) dst[cc] = src[cc];
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, RT_N);
}

int ragged_gemm_tcgen05(const void* a, const void* b, void* out, int heads, int n_images, long long a_rows,
                        int a_cols, long long b_rows, int b_cols, const int32_t* a_off, const int32_t* b_off,
                        int max_m, int max_n, int ta, int tb, long long out_rows, int out_cols, cudaStream_t st) {
    VTP_REQUIRE(aligned16(a) && aligned16(b), VTP_ERR_ALIGN,
                "batched_sparse_gemm (tcgen05): the operand arrays must start on a 16-byte boundary");
    RaggedTcArgs g;
    g.a = static_cast<const bf16*>(a); g.b = static_cast<const bf16*>(b); g.out = static_cast<bf16*>(out);
    g.a_rows = a_rows; g.b_rows = b_rows; g.out_rows = out_rows;
    g.a_cols = a_cols; g.b_cols = b_cols; g.out_cols = out_cols;
    g.a_off = a_off; g.b_off = b_off; g.ta = ta; g.tb = tb; g.heads = heads;
    g.tiles_n = ceil_div(max_n, RT_N);
    // a few columns beyond the last full tile stay with that tile (CUDA-core dot products from the staged
    // slices; needs both operands' rows along the reduction axis)
    const int over = max_n - (g.tiles_n - 1) * RT_N;
    g.absorb_tail = (!ta && tb && g.tiles_n > 1 && over <= RT_TAIL) ? 1 : 0;
    if (g.absorb_tail) g.tiles_n -= 1;
    const dim3 grid((unsigned)(ceil_div(max_m, RT_M) * g.tiles_n), (unsigned)n_images, (unsigned)heads);
    const bool a_hi = a_cols % 8 != 0;                     // rows of a off 16-byte boundaries
    // sub-tiles of a b slice: rows n of the widest tile (plus the tail's) for a K-major b, 64-column atoms otherwise
    const int widest = max_n < RT_N ? max_n : RT_N;
    const bool one_sub = (tb ? (g.absorb_tail ? RT_N + RT_TAIL : ((widest + 15) & ~15)) : ((widest + 15) & ~15)) <= 64;
    auto launch = [&](auto kern) -> int {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, RT_SMEM);
        if (e != cudaSuccess) return fail((int)e, "batched_sparse_gemm (tcgen05): shared memory: %s", cudaGetErrorString(e));
        kern<<<grid, RT_THREADS, RT_SMEM, st>>>(g, device_status_ptr());
        return VTP_OK;
    };
    int rc;
    if (a_hi) rc = one_sub ? launch(ragged_gemm_tc_kernel<true, 1>) : launch(ragged_gemm_tc_kernel<true, RT_BSUB_MAX>);
    else rc = one_sub ? launch(ragged_gemm_tc_kernel<false, 1>) : launch(ragged_gemm_tc_kernel<false, RT_BSUB_MAX>);
    if (rc) return rc;
    return check_launch("batched_sparse_gemm (tcgen05)");
}

}  // namespace vtp
