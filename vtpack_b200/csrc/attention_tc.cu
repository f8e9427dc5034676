// Variable-length-query attention on tcgen05 tensor cores (bf16 in, fp32 accumulate).
//
// Work item = 128 packed queries of one (image, head).  Persistent CTAs (two per SM) walk
// the items with a fixed stride; the item list is derived on the device from the per-image
// offsets, so images with few queries cost nothing and nothing is read back to the host.
// Keys are split into a tensor-core part (the largest multiple of 16, walked in chunks of
// up to 256 keys) and a tail of at most 15 keys done on CUDA cores: token grids with one
// cls token have 16k+1 keys, so 257 keys are ONE 256-key chunk plus one tail key.
//   S = Q K_c^T        tcgen05.mma, A = Q tile, B = K chunk, both K-major from TMA (128B
//                      swizzle); accumulator S in TMEM columns [0, KC)
//   P = exp2(scale*log2e*(S - rowmax))   four softmax warps, one thread per query row: read S
//                      with tcgen05.ld, write bf16 P back into TMEM over the S columns
//                      already consumed (columns [0, KC/2))
//   O_c = P V_c        tcgen05.mma with A = P from TMEM and B = V chunk as an MN-major operand
//                      straight from the TMA image of the [keys, d] rows; accumulator in TMEM
//                      columns [128, 192)
//   O  = O*alpha + O_c in registers of the softmax threads (online-softmax rescale), then the
//                      tail keys, the 1/rowsum and the bf16 store.
// Warp 0 lane 0 issues TMA (Q is double-buffered so the next item's Q and K stream in during
// the current softmax), warp 1 lane 0 issues MMA, warps 2-5 do softmax and output.
// q, k, v are read in place from the Linear outputs through strided tensor maps.
// Every mbarrier wait is bounded (sm100.cuh).
//
// Replaces batched_sparse_attention_forward
// (vtpack/layers/csrc/batched_sparse_gemm/batched_sparse_gemm.cu:219-305: per image two
// cuBLAS strided-batched GEMMs around a cuDNN softmax, scores round-tripping through HBM).
#include "attention.h"
#include "runtime.h"
#include "sm100.cuh"

namespace vtp {

using namespace sm100;

constexpr int QT = 128;            // queries per item = TMEM lanes
constexpr int HD = 64;             // head dim
constexpr int KC_MAX = 256;        // keys per tensor-core chunk, upper bound
constexpr int O_COL = 128;         // TMEM column of the P*V accumulator
constexpr int ATT_TMEM_COLS = 256;

constexpr int SM_Q = 0;                               // two Q buffers
constexpr int SM_K = SM_Q + 2 * QT * HD * 2;          // 32768
constexpr int SM_V = SM_K + KC_MAX * HD * 2;          // 65536
constexpr int SM_BAR = SM_V + KC_MAX * HD * 2;        // 98304
constexpr int SM_ITEM = SM_BAR + 256;                 // two work items (one per Q buffer), written by the producer
constexpr int SM_TAIL = SM_ITEM + 256;                // per Q buffer: up to 15 tail K rows, then 15 tail V rows
constexpr int TAIL_ROWS = 15;
constexpr int SM_PREFIX = SM_TAIL + 2 * 2 * TAIL_ROWS * HD * 2;   // int32 [B + 1] tile prefix

// 2^x on the special-function unit; arguments here are <= 0 (or -inf, giving 0).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct AttnItem { int b, h, row0, nq; };

// Plain bulk copy global -> shared of `bytes` (a multiple of 16, both ends 16-byte aligned), counted on `bar`.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// item w -> (image, head, first packed row, valid rows); tile_prefix is in shared memory
__device__ __forceinline__ AttnItem attn_item(int w, int heads, int B, const int* tile_prefix,
                                              const int32_t* __restrict__ offsets) {
    const int tg = w / heads;
    int lo = 0, hi = B;                        // largest b with tile_prefix[b] <= tg
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (tile_prefix[mid] <= tg) lo = mid; else hi = mid;
    }
    AttnItem it;
    it.b = lo;
    it.h = w - tg * heads;
    const int t = tg - tile_prefix[lo];
    it.row0 = offsets[lo] + t * QT;
    it.nq = min(QT, offsets[lo + 1] - it.row0);
    return it;
}

__global__ void __launch_bounds__(192, 2)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const __grid_constant__ CUtensorMap tmap_v, const bf16* __restrict__ kptr,
               const bf16* __restrict__ vptr, long long q_hs, long long kv_bs, long long kv_rs, long long kv_hs,
               bf16* __restrict__ out, long long o_rs, long long o_hs, int B, int heads, int n_keys, int KC,
               int n_chunks, const int32_t* __restrict__ offsets, int l_max, int max_q, float scale_log2e,
               int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + SM_BAR);
    uint64_t* q_full = bars + 0;    // [2]
    uint64_t* q_free = bars + 2;    // [2]
    uint64_t* k_full = bars + 4;
    uint64_t* k_free = bars + 5;
    uint64_t* v_full = bars + 6;
    uint64_t* v_free = bars + 7;
    uint64_t* s_full = bars + 8;
    uint64_t* p_full = bars + 9;
    uint64_t* o_full = bars + 10;
    uint64_t* o_free = bars + 11;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* tile_prefix = reinterpret_cast<int*>(base + SM_PREFIX);
    AttnItem* items = reinterpret_cast<AttnItem*>(base + SM_ITEM);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 32) {
        for (int i = 0; i < 2; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_free[i], QT); }
        mbar_init(k_full, 1); mbar_init(k_free, 1);
        mbar_init(v_full, 1); mbar_init(v_free, 1);
        mbar_init(s_full, 1); mbar_init(p_full, QT);
        mbar_init(o_full, 1); mbar_init(o_free, QT);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, ATT_TMEM_COLS);
        tmem_relinquish();
    }
    // Nothing above depends on the kernel in front of this one on the stream; the packed-row
    // offsets, q, k and v below do.
    griddep_launch();
    griddep_wait();
    // tile_prefix[b] = number of 128-query tiles of the images in front of b.  All threads fetch the
    // per-image tile counts at once (one global-load latency), then warp 0 scans them in shared memory.
    // (the offsets come from the caller: a count outside [0, max_q] is clamped, so the item list
    // always fits the grid's bound, and rows at or beyond l_max are never stored below)
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        int cnt = offsets[b + 1] - offsets[b];
#if VTP_INDEX_GUARDS
        if (cnt < 0 || cnt > max_q || offsets[b] < 0 || offsets[b + 1] > l_max) {
            if (status && blockIdx.x == 0) atomicOr(status, STATUS_BAD_INDEX);
            cnt = (offsets[b] < 0) ? 0 : min(max(cnt, 0), max_q);
        }
#endif
        tile_prefix[b] = (cnt + QT - 1) / QT;
    }
    __syncthreads();
    if (warp == 0) {
        int run = 0;
        for (int b0 = 0; b0 < B; b0 += 32) {
            const int b = b0 + lane;
            const int tiles = b < B ? tile_prefix[b] : 0;
            int incl = tiles;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int nb = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += nb;
            }
            __syncwarp();
            if (b < B) tile_prefix[b] = run + incl - tiles;
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) tile_prefix[B] = run;
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const bool void_launch = status && (*reinterpret_cast<volatile int*>(status) & STATUS_WAIT_MASK) != 0;
    const int n_work = void_launch ? 0 : tile_prefix[B] * heads;
    const int n_main = (n_keys / 16) * 16;          // keys handled by the tensor cores
    const int tail = n_keys - n_main;               // 0..15 keys handled on CUDA cores

    if (warp == 0) {
        if (lane == 0) {
            // ------------------------------------------------------------ TMA producer
            prefetch_tmap(&tmap_q);
            prefetch_tmap(&tmap_k);
            prefetch_tmap(&tmap_v);
            const uint32_t kv_bytes = (uint32_t)KC * HD * 2;
            int li = 0, g = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++li) {
                const AttnItem it = attn_item(w, heads, B, tile_prefix, offsets);
                const int qb = li & 1;
                ok = mbar_wait(&q_free[qb], ((li >> 1) & 1) ^ 1, abort_flag, status, STATUS_ATTN_LOAD);
                if (!ok) break;
                // the item, its Q tile and the K and V rows of the tail keys all arrive on q_full
                items[qb] = it;
                mbar_arrive_expect_tx(&q_full[qb], QT * HD * 2 + 2 * tail * HD * 2);
                tma_load_2d(base + SM_Q + qb * (QT * HD * 2), &tmap_q, &q_full[qb], (int)(it.h * q_hs), it.row0);
                for (int t = 0; t < tail; ++t) {
                    const size_t koff = (size_t)it.b * kv_bs + (size_t)(n_main + t) * kv_rs + (size_t)it.h * kv_hs;
                    uint8_t* tb = base + SM_TAIL + qb * (2 * TAIL_ROWS * HD * 2) + t * (HD * 2);
                    bulk_load(tb, kptr + koff, HD * 2, &q_full[qb]);
                    bulk_load(tb + TAIL_ROWS * HD * 2, vptr + koff, HD * 2, &q_full[qb]);
                }
                for (int c = 0; c < n_chunks; ++c, ++g) {
                    const uint32_t ph = g & 1;
                    ok = mbar_wait(k_free, ph ^ 1, abort_flag, status, STATUS_ATTN_LOAD);
                    if (!ok) break;
                    mbar_arrive_expect_tx(k_full, kv_bytes);
                    tma_load_3d(base + SM_K, &tmap_k, k_full, (int)(it.h * kv_hs), c * KC, it.b);
                    ok = mbar_wait(v_free, ph ^ 1, abort_flag, status, STATUS_ATTN_LOAD);
                    if (!ok) break;
                    mbar_arrive_expect_tx(v_full, kv_bytes);
                    tma_load_3d(base + SM_V, &tmap_v, v_full, (int)(it.h * kv_hs), c * KC, it.b);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // -------------------------------------------------------------- MMA issuer
            const uint32_t idesc_s = idesc_bf16_f32(QT, KC, 0, 0);
            const uint32_t idesc_o = idesc_bf16_f32(QT, HD, 0, 1);     // B = V, MN-major
            const uint64_t kdesc = smem_desc_sw128(smem_u32(base + SM_K));
            const uint64_t vdesc = smem_desc_sw128(smem_u32(base + SM_V));
            int li = 0, g = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++li) {
                const int qb = li & 1;
                const uint64_t qdesc = smem_desc_sw128(smem_u32(base + SM_Q + qb * (QT * HD * 2)));
                ok = mbar_wait(&q_full[qb], (li >> 1) & 1, abort_flag, status, STATUS_ATTN_MMA);
                for (int c = 0; c < n_chunks && ok; ++c, ++g) {
                    const uint32_t ph = g & 1;
                    // S columns double as the P and O columns of the previous chunk: wait until
                    // the softmax threads have taken O out
                    ok = mbar_wait(k_full, ph, abort_flag, status, STATUS_ATTN_MMA) &&
                         mbar_wait(o_free, ph ^ 1, abort_flag, status, STATUS_ATTN_MMA);
                    if (!ok) break;
                    tc_fence_after_sync();
#pragma unroll
                    for (int k = 0; k < HD / 16; ++k)
                        umma_ss(tmem_base, qdesc + 2 * k, kdesc + 2 * k, idesc_s, k != 0 ? 1u : 0u);
                    umma_commit(s_full);
                    umma_commit(k_free);
                    ok = mbar_wait(p_full, ph, abort_flag, status, STATUS_ATTN_MMA) &&
                         mbar_wait(v_full, ph, abort_flag, status, STATUS_ATTN_MMA);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const int ksteps = KC / 16;
                    for (int t = 0; t < ksteps; ++t) {
                        // P: 16 keys = 8 TMEM columns of bf16 pairs.  V: 16 keys = 16 rows of 128 bytes.
                        umma_ts(tmem_base + O_COL, tmem_base + 8 * t, vdesc + (uint64_t)(t * (16 * 128 >> 4)),
                                idesc_o, t != 0 ? 1u : 0u);
                    }
                    umma_commit(o_full);
                    umma_commit(v_free);
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------- softmax + output warps
        const int r = (warp & 3) * 32 + lane;                     // query row = TMEM lane
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        int li = 0, g = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++li) {
            const int qb = li & 1;
            // the producer worked out which (image, head, rows) this item is; it arrives with the Q tile
            ok = mbar_wait(&q_full[qb], (li >> 1) & 1, abort_flag, status, STATUS_ATTN_SOFTMAX);
            if (!ok) break;
            const AttnItem it = items[qb];
            // a warp whose 32 rows all lie beyond the item's queries only keeps the barriers moving: its rows
            // of P and O are never stored, so what the tensor core computes for them does not matter, and
            // the special-function unit and the issue slots go to the warps that have rows to compute
            const bool live = (warp & 3) * 32 < it.nq;
            float m = -INFINITY, l = 0.f;
            float o[HD];
#pragma unroll
            for (int i = 0; i < HD; ++i) o[i] = 0.f;
            for (int c = 0; c < n_chunks && ok; ++c, ++g) {
                const uint32_t ph = g & 1;
                ok = mbar_wait(s_full, ph, abort_flag, status, STATUS_ATTN_SOFTMAX);
                if (!ok) break;
                tc_fence_after_sync();
                if (!live) {
                    mbar_arrive(p_full);
                    ok = mbar_wait(o_full, ph, abort_flag, status, STATUS_ATTN_SOFTMAX);
                    if (!ok) break;
                    mbar_arrive(o_free);
                    continue;
                }
                const int n_valid = min(KC, n_main - c * KC);
                const bool full = n_valid == KC && (KC & 31) == 0;     // no column needs masking
                // Two sweeps over the S columns, 32 at a time: row maximum, then exp2 + P.  The
                // TMEM load of the next block is always in flight while the current one is used.
                const int nblk = (KC + 31) >> 5;
                uint32_t s[32];
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                __syncwarp();
                tmem_ld_32x32(lane_base, s);
                for (int blk = 0; blk < nblk; ++blk) {
                    tmem_ld_wait();
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(s[i]);
                    __syncwarp();
                    tmem_ld_32x32(lane_base + (blk + 1 < nblk ? (blk + 1) * 32 : 0), s);   // wraps to sweep 2
                    const int c0 = blk * 32;
                    if (full) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], f[i]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (c0 + i < n_valid) mx4[i & 3] = fmaxf(mx4[i & 3], f[i]);
                    }
                }
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                const float m_new = fmaxf(m, mx);
                const float alpha = fast_exp2((m - m_new) * scale_log2e);       // 0 on the first chunk
                const float mb = m_new * scale_log2e;
                float ls4[4] = {0.f, 0.f, 0.f, 0.f};
                for (int blk = 0; blk < nblk; ++blk) {
                    tmem_ld_wait();
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(s[i]);
                    if (blk + 1 < nblk) {
                        __syncwarp();
                        tmem_ld_32x32(lane_base + (blk + 1) * 32, s);
                    }
                    const int c0 = blk * 32;
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        float p0 = fast_exp2(fmaf(f[2 * i], scale_log2e, -mb));
                        float p1 = fast_exp2(fmaf(f[2 * i + 1], scale_log2e, -mb));
                        if (!full) {
                            p0 = (c0 + 2 * i < n_valid) ? p0 : 0.f;
                            p1 = (c0 + 2 * i + 1 < n_valid) ? p1 : 0.f;
                        }
                        ls4[i & 3] += p0 + p1;
                        const __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);   // low half = even key
                        pk[i] = *reinterpret_cast<const uint32_t*>(&h2);
                    }
                    __syncwarp();
                    tmem_st_32x16(lane_base + (c0 >> 1), pk);      // over S columns already consumed
                }
                const float lsum = (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
                tmem_st_wait();
                tc_fence_before_sync();
                mbar_arrive(p_full);
                l = l * alpha + lsum;
                m = m_new;
                ok = mbar_wait(o_full, ph, abort_flag, status, STATUS_ATTN_SOFTMAX);
                if (!ok) break;
                tc_fence_after_sync();
#pragma unroll
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    uint32_t t[32];
                    __syncwarp();
                    tmem_ld_32x32(lane_base + O_COL + c0, t);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[c0 + i] = fmaf(o[c0 + i], alpha, __uint_as_float(t[i]));
                }
                tc_fence_before_sync();
                mbar_arrive(o_free);
            }
            if (!ok) break;
            if (!live) {
                mbar_arrive(&q_free[qb]);
                continue;
            }
            const uint8_t* qrow = base + SM_Q + qb * (QT * HD * 2) + r * 128;
            if (tail > 0) {
                // ---- the last n_keys % 16 keys on CUDA cores, one online-softmax step per key
                const uint8_t* tb = base + SM_TAIL + qb * (2 * TAIL_ROWS * HD * 2);
                for (int t = 0; t < tail; ++t) {
                    const uint4* krow = reinterpret_cast<const uint4*>(tb + t * (HD * 2));
                    const uint4* vrow = reinterpret_cast<const uint4*>(tb + (TAIL_ROWS + t) * (HD * 2));
                    float sdot = 0.f;
#pragma unroll
                    for (int ch = 0; ch < HD / 8; ++ch) {
                        Vec<bf16> qv, kv;
                        float qf[8], kf[8];
                        qv.raw = *reinterpret_cast<const uint4*>(qrow + ((ch ^ (r & 7)) << 4));
                        kv.raw = krow[ch];
                        qv.to_float(qf);
                        kv.to_float(kf);
#pragma unroll
                        for (int i = 0; i < 8; ++i) sdot = fmaf(qf[i], kf[i], sdot);
                    }
                    const float m_new = fmaxf(m, sdot);
                    const float alpha = fast_exp2((m - m_new) * scale_log2e);
                    const float p = fast_exp2((sdot - m_new) * scale_log2e);
                    l = l * alpha + p;
                    m = m_new;
#pragma unroll
                    for (int ch = 0; ch < HD / 8; ++ch) {
                        Vec<bf16> vv;
                        float vf[8];
                        vv.raw = vrow[ch];
                        vv.to_float(vf);
#pragma unroll
                        for (int i = 0; i < 8; ++i) o[8 * ch + i] = fmaf(o[8 * ch + i], alpha, p * vf[i]);
                    }
                }
            }
            // ---- normalise, then out through the warp's own 32 rows of the Q tile (no longer needed) so that
            // eight lanes write one full 128-byte line of a row instead of every lane a piece of its own row
            {
                const float inv = 1.0f / l;
                __syncwarp();                                   // every lane has read its Q row (tail scores)
                uint8_t* my = const_cast<uint8_t*>(qrow);
#pragma unroll
                for (int ch = 0; ch < HD / 8; ++ch) {
                    float v8[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) v8[i] = o[8 * ch + i] * inv;
                    Vec<bf16> ov;
                    ov.from_float(v8);
                    *reinterpret_cast<uint4*>(my + ((ch ^ (r & 7)) << 4)) = ov.raw;
                }
                __syncwarp();
                const uint8_t* wq = base + SM_Q + qb * (QT * HD * 2) + (warp & 3) * 32 * 128;
                const int ch = lane & 7;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int rr = i * 4 + (lane >> 3);          // row within the warp's 32
                    const int row = (warp & 3) * 32 + rr;
                    const uint4 v = *reinterpret_cast<const uint4*>(wq + rr * 128 + ((ch ^ (rr & 7)) << 4));
                    if (row < it.nq && it.row0 + row < l_max)
                        *reinterpret_cast<uint4*>(out + (size_t)(it.row0 + row) * o_rs + it.h * o_hs + ch * 8) = v;
                }
                __syncwarp();
                fence_proxy_async_smem();                       // the next Q tile is written by TMA
            }
            mbar_arrive(&q_free[qb]);
        }
    }
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) { }     // let copies in flight land before releasing memory
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, ATT_TMEM_COLS);
}

int attention_tcgen05_max_images() { return 16384; }

int attention_tcgen05(const AttnArgs& p, cudaStream_t st) {
    VTP_REQUIRE(p.dtype == VTP_BF16, VTP_ERR_DTYPE, "attention (tcgen05): bf16 only");
    VTP_REQUIRE(p.head_dim == HD, VTP_ERR_UNSUPPORTED, "attention (tcgen05): head_dim %d (only %d)", p.head_dim, HD);
    VTP_REQUIRE(p.n_keys >= 16, VTP_ERR_UNSUPPORTED, "attention (tcgen05): needs at least 16 keys, got %d", p.n_keys);
    VTP_REQUIRE(p.B <= 16384, VTP_ERR_SHAPE, "attention (tcgen05): %d images (at most 16384)", p.B);
    VTP_REQUIRE(p.q_rs % 8 == 0 && p.q_hs % 8 == 0 && p.kv_rs % 8 == 0 && p.kv_hs % 8 == 0 && p.kv_bs % 8 == 0 &&
                    p.o_rs % 8 == 0 && p.o_hs % 8 == 0,
                VTP_ERR_ALIGN, "attention (tcgen05): strides must be multiples of 16 bytes");
    VTP_REQUIRE(aligned16(p.q) && aligned16(p.k) && aligned16(p.v) && aligned16(p.out), VTP_ERR_ALIGN,
                "attention (tcgen05): pointers must be 16-byte aligned");
    const int n_main = (p.n_keys / 16) * 16;
    const int n_chunks = ceil_div(n_main, KC_MAX);
    const int KC = (int)round_up(ceil_div(n_main, n_chunks), 16);
    CUtensorMap tq, tk, tv;
    {
        const unsigned long long dims[2] = {(unsigned long long)((p.heads - 1) * p.q_hs + HD),
                                            (unsigned long long)p.l_max};
        const unsigned long long strides[1] = {(unsigned long long)p.q_rs * 2ull};
        const unsigned box[2] = {HD, QT};
        if (int rc = make_tmap_bf16(&tq, p.q, 2, dims, strides, box)) return rc;
    }
    {
        const unsigned long long dims[3] = {(unsigned long long)((p.heads - 1) * p.kv_hs + HD),
                                            (unsigned long long)p.n_keys, (unsigned long long)p.B};
        const unsigned long long strides[2] = {(unsigned long long)p.kv_rs * 2ull, (unsigned long long)p.kv_bs * 2ull};
        const unsigned box[3] = {HD, (unsigned)KC, 1};
        if (int rc = make_tmap_bf16(&tk, p.k, 3, dims, strides, box)) return rc;
        if (int rc = make_tmap_bf16(&tv, p.v, 3, dims, strides, box)) return rc;
    }
    const int smem = SM_PREFIX + (p.B + 1) * 4 + 1024;
    static int attr_smem[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || attr_smem[dev] < smem) {
        const cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) {
            set_error("attention (tcgen05): cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return (int)e;
        }
        if (dev >= 0 && dev < 64) attr_smem[dev] = smem;
    }
    const long long worst = (long long)p.B * ceil_div(p.max_q, QT) * p.heads;
    const int grid = (int)(worst < 2ll * sm_count() ? worst : 2ll * sm_count());
    const cudaError_t le = launch_pdl(attn_tc_kernel, dim3(grid), dim3(192), (size_t)smem, st, tq, tk, tv,
                                      (const bf16*)p.k, (const bf16*)p.v, p.q_hs, p.kv_bs, p.kv_rs, p.kv_hs, (bf16*)p.out,
                                      p.o_rs, p.o_hs, p.B, p.heads, p.n_keys, KC, n_chunks, p.offsets, p.l_max, p.max_q,
                                      p.scale * 1.4426950408889634f, device_status_ptr());
    if (le != cudaSuccess) {
        cudaGetLastError();
        set_error("attention (tcgen05): %s", cudaGetErrorString(le));
        return (int)le;
    }
    return check_launch("attention (tcgen05)");
}

}  // namespace vtp
