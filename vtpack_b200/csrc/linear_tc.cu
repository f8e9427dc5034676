// Linear layer on 5th-generation tensor cores (tcgen05), bf16 operands, fp32 accumulate in
// tensor memory, operands staged by TMA with a 128-byte swizzle.
//
//   y[m, n] = act(sum_k a[m,k] w[n,k] + bias[n]) + res[m, n]
//
// Persistent, warp-specialised: one CTA per SM walks 128 x BN output tiles (n fastest, so the
// CTAs running at the same time share an A row tile in L2).
//   warp 0   (one lane)  TMA producer: fills a STAGES-deep ring of {A 128x64, W BNx64} tiles;
//                        the ring runs across tile boundaries, so the next tile's operands
//                        stream in during the current tile's epilogue
//   warp 1   (one lane)  issues tcgen05.mma (M=128, N=BN, K=16) into one of two TMEM
//                        accumulators and commits each stage back to the producer
//   warps 2-17           epilogue: read the finished accumulator with tcgen05.ld (warp w may
//                        touch TMEM lanes 32*(w%4)..+31 = tile rows; four warps share a lane
//                        quarter and split the columns), apply bias / GELU / residual, then
//                        write the tile 64 columns at a time into one of two swizzled staging
//                        slabs (full 128-byte lines, no partial sectors) and signal it full
//                        on an mbarrier: the warps never wait for each other inside a tile.  The accumulator goes back to the MMA warp as soon as its
//                        last columns are in registers.  Tiles that touch the last valid row,
//                        row-remapped outputs and fp32 outputs store straight from registers.
//   warp 18  (one lane)  store thread: waits for a full slab, hands it to a TMA store, waits until
//                        the store has read it, then marks it free again or, when there is a
//                        residual, has the TMA load the residual of the slab after next into it.
// The two accumulators let the MMA of tile i+1 overlap the epilogue of tile i.
// The tiles left for the last, partial round of the grid are cut into two to four column strips
// (their own W boxes, a narrower MMA), one per CTA, so that round costs a fraction of a tile.
// The number of valid rows is read from device memory: tiles beyond it do not exist, rows
// beyond it are never stored.
//
// Every mbarrier wait is bounded (see sm100.cuh); a wait that gives up ORs a code into the
// device status word and the CTA unwinds.
//
// Replaces nn.Linear q/kv/proj/fc1/fc2/head, nn.GELU and the residual adds of
// vtpack/models/dge/deit_dge.py:38-44,72-74,96,127-128 (cuBLAS + ATen kernels there).
#include <cuda_fp16.h>
#include <stdlib.h>

#include "linear.h"
#include "runtime.h"
#include "sm100.cuh"

namespace vtp {

using namespace sm100;

constexpr int TBM = 128;   // tile rows of one CTA = TMEM lanes
// CTAs per MMA tile.  2: the CTAs of a cluster of two share 256-row tiles (tcgen05 cta_group::2): each stages
// its own 128 rows of A and half of the tile's W rows, the rank-0 CTA issues the MMAs, each CTA runs the
// epilogue of its own 128 rows.  A CTA then stages and the tensor core reads 8 KB per 128 x 256 x 16 MMA step
// instead of 12 KB; with one CTA per tile the shared-memory operand reads, not the tensor core, set the pace.
#ifndef VTP_LINEAR_CTA_GROUP
#define VTP_LINEAR_CTA_GROUP 1
#endif
constexpr int CG = VTP_LINEAR_CTA_GROUP;
static_assert(CG == 1 || CG == 2, "one CTA or a pair per tile");
constexpr int TM = TBM * CG;   // tile rows of the CTA group
// Staging slabs of the epilogue (128 rows x 64 columns each); half as many TMA stores may be reading them at
// a time.  A store's shared-memory read takes longer than the epilogue needs to fill the next slab, so with
// two slabs the epilogue waits on the store; the pair kernel's smaller operand stages leave room for four.
// A narrow Linear (N <= 128) with one k-block per tile, or two and a residual to fetch, spends its time in the
// epilogue's hand-offs: it runs with a ring of SHALLOW_RING stages, gives the shared memory to four staging
// slabs and keeps its bias slice across tiles (measured at 1 M rows, K = N = 64: 80 -> 71 us, with a residual
// 117 -> 85 us; wide tiles with GELU and K = 128 without a residual were faster on the deep ring).
constexpr int SHALLOW_RING = 3;
constexpr int staging_slabs(int stages) { return CG == 2 ? 4 : (stages <= SHALLOW_RING ? 4 : 2); }
// depth of the operand ring for a tile width: what fits beside the staging slabs
constexpr int ring_stages(int bn) { return CG == 2 ? (bn == 128 ? 6 : 5) : (bn == 128 ? 5 : 4); }
constexpr int TBK = 64;    // 64 bf16 = one 128-byte swizzle row
constexpr int EPI_THREADS = 512;  // 16 epilogue warps, four per TMEM lane quarter
constexpr int TC_THREADS = 64 + EPI_THREADS + 32;   // + the store warp

template <int BN, int STAGES>
struct TcSmem {
    static constexpr int A_BYTES = TBM * TBK * 2;
    static constexpr int B_BYTES = (BN / CG) * TBK * 2;   // this CTA's share of the W rows
    static constexpr int RING = STAGES * (A_BYTES + B_BYTES);
    static constexpr int NSTG = staging_slabs(STAGES);
    static constexpr int STORES_IN_FLIGHT = NSTG / 2;
    static constexpr int STAGE_OUT = NSTG * TBM * 128;   // 128-row x 64-column bf16 slabs
    static constexpr int BIAS = 2 * BN * 4;           // the bias and LayerNorm-fold slices of the tile in the epilogue
    static constexpr int USED = RING + STAGE_OUT + BIAS + 512 /* barriers */;
    // Dynamic shared memory is only promised 16-byte alignment; the ring wants 1024.  In
    // practice the base is already aligned; the kernel checks that what is left fits.
    static constexpr int TOTAL = (USED + 1024 <= 232448) ? USED + 1024 : 232448;
    static_assert(USED <= 232448, "shared memory budget");
    static constexpr int TMEM_COLS = (2 * BN <= 256) ? 256 : 512;
};

template <typename OutT> struct OutVec;
template <> struct OutVec<bf16> {
    // 8 values -> one 16-byte store
    static __device__ __forceinline__ void store8(bf16* p, const float* v) {
        Vec<bf16> o;
        o.from_float(v);
        o.store(p);
    }
};
template <> struct OutVec<float> {
    static __device__ __forceinline__ void store8(float* p, const float* v) {
        reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
};

// erf-GELU of eight values, packed two per register in fp16, as 0.5 x (1 + tanh(x (k0 + k1 x^2))) with
// k0, k1 fitted to 0.5 x (1 + erf(x / sqrt 2)) (max abs error 2.7e-4); fp16 arithmetic adds an rms
// error of 5e-4, a fifth of the rounding of the bf16 result.  Six packed instructions and one
// tanh.approx per pair: the form with ex2 + rcp per value kept the special-function unit
// (16 results per clock per SM) busier than the tensor core.  Inputs beyond the fp16 range
// saturate; there x^2 overflows to +inf, tanh gives +-1 and the result is x or 0 as it should.
__device__ __forceinline__ uint32_t gelu_pair_f16(float lo, float hi) {
    uint32_t x, t;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(x) : "f"(hi), "f"(lo));
    const __half2 xh = *reinterpret_cast<__half2*>(&x);
    const __half2 u = __hmul2(xh, xh);
    const __half2 p = __hfma2(u, __float2half2_rn(0.03470089f), __float2half2_rn(0.80015708f));
    const __half2 a = __hmul2(xh, p);
    asm("tanh.approx.f16x2 %0, %1;" : "=r"(t) : "r"(*reinterpret_cast<const uint32_t*>(&a)));
    const __half2 hx = __hmul2(xh, __float2half2_rn(0.5f));
    const __half2 g = __hfma2(hx, *reinterpret_cast<__half2*>(&t), hx);
    return *reinterpret_cast<const uint32_t*>(&g);
}
__device__ __forceinline__ void gelu8(float* v) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t g = gelu_pair_f16(v[2 * i], v[2 * i + 1]);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&g));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

// EPI: what the epilogue does besides the bias, fixed at compile time so that a kernel only
// issues the instructions of the variant it is (a runtime flag would be if-converted and the
// GELU / LayerNorm arithmetic issued, predicated off, by every GEMM).
constexpr int EPI_GELU = 1, EPI_LN = 2, EPI_EMIT = 4;

// One GEMM problem of a launch: its tensor maps and epilogue operands.
struct TcProblem {
    CUtensorMap ta, tw, tw2, tw3, ty, tr;    // A, W (tile / half / quarter height boxes), output, residual
    const float* bias; const bf16* res; long long ldr;
    void* y; long long ldy;
    int m_max; const int32_t* m_dev; int N;
    int use_tma_store;
    RowMap rm; LnFold ln;
};
// A launch works through one problem or two independent ones (same K, tile shape and epilogue kind): the
// tiles of the second fill the last, partial round of the first, and one launch's ramp and tail is saved.
struct TcLaunch { TcProblem p[2]; int n; };

template <int BN, int STAGES, typename OutT, int EPI, int NPROB>
__global__ void __launch_bounds__(TC_THREADS, 1)
linear_tc_kernel(const __grid_constant__ TcLaunch L, int K, int* status) {
    using S = TcSmem<BN, STAGES>;
    constexpr int NSTG = S::NSTG, STORES_IN_FLIGHT = S::STORES_IN_FLIGHT;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = base;
    uint8_t* smem_b = base + STAGES * S::A_BYTES;
    if (static_cast<int>(base - smem_raw) + S::USED > S::TOTAL) {
        if (threadIdx.x == 0 && status) atomicOr(status, STATUS_GEMM_PRODUCER);
        return;
    }
    uint8_t* smem_out = base + S::RING;
    float* bias_s = reinterpret_cast<float*>(base + S::RING + S::STAGE_OUT);
    uint64_t* full = reinterpret_cast<uint64_t*>(base + S::RING + S::STAGE_OUT + S::BIAS);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;       // [2]
    uint64_t* acc_empty = acc_full + 2;        // [2]
    uint64_t* res_full = acc_empty + 2;        // [NSTG] residual slab landed in the staging buffer
    uint64_t* slab_full = res_full + NSTG;     // [NSTG] every epilogue warp has written its part of the staging slab
    uint64_t* slab_free = slab_full + NSTG;    // [NSTG] the TMA store has read the staging slab
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(slab_free + NSTG);
    static_assert((2 * STAGES + 4 + 3 * NSTG) * 8 + 8 <= 512, "barrier area");
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_kb = K / TBK;
    const int rank = CG == 2 ? (int)cluster_ctarank() : 0;             // this CTA within its group
    const int n_groups = (int)gridDim.x / CG, group = (int)blockIdx.x / CG;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], CG * (EPI_THREADS / 32));   // rank 0's: the epilogue warps of the whole group
        }
        for (int b = 0; b < NSTG; ++b) {
            mbar_init(&res_full[b], 1);
            mbar_init(&slab_full[b], EPI_THREADS / 32);
            mbar_init(&slab_free[b], 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        if (CG == 2) { tmem_alloc_pair(tmem_slot, S::TMEM_COLS); tmem_relinquish_pair(); }
        else { tmem_alloc(tmem_slot, S::TMEM_COLS); tmem_relinquish(); }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (CG == 2) cluster_sync_all();     // the partner's barriers exist before anything arrives on them
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // Everything above is independent of the kernel in front of this one on the stream; from
    // here on its results (row count, operands, residual, statistics) are read.
    griddep_launch();
    griddep_wait();
    // valid rows, column tiles and tile count of each problem
    int Mp[2], ntp[2], totp[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        Mp[i] = ntp[i] = totp[i] = 0;
        if (i < NPROB) {
            Mp[i] = L.p[i].m_max;
            if (L.p[i].m_dev) Mp[i] = min(*reinterpret_cast<const volatile int32_t*>(L.p[i].m_dev), L.p[i].m_max);
            ntp[i] = (L.p[i].N + BN - 1) / BN;
            totp[i] = ((Mp[i] + TM - 1) / TM) * ntp[i];
        }
    }
    // no tiles for this CTA, or an earlier CTA gave up on a wait (the launch is void): skip the work
    const bool void_launch = status && (*reinterpret_cast<volatile int*>(status) & STATUS_WAIT_MASK) != 0;
    const int total = void_launch ? 0 : totp[0] + totp[1];
    // Tail splitting.  A CTA group takes tiles group, + n_groups, ...; the R tiles left for the last,
    // partial round are cut into `parts` column strips of BN / parts columns, one strip per group, so that
    // the round costs a fraction of a tile instead of a whole one with most SMs idle.  Strips use their
    // own W boxes (tw2 / tw3) and a narrower MMA; kernels that keep per-tile row statistics
    // (EPI_EMIT) do not split.
    const int full_items = (total / n_groups) * n_groups;
    int parts = 1;
    {
        const int R = total - full_items, G = n_groups;
        if (!(EPI & EPI_EMIT) && R > 0) {
            if (BN == 256) parts = (R * 4 <= G) ? 4 : (R * 2 <= G ? 2 : 1);
            else if (BN == 192) parts = (R * 3 <= G) ? 3 : 1;
            else parts = (R * 2 <= G) ? 2 : 1;
        }
    }
    // j-th work item of this CTA: problem p, this CTA's rows m0.., columns ct0 .. ct0 + width of its output.  The last
    // column tile of a problem whose N is not a multiple of BN is as wide as the columns left, in 64s.
    struct Item { int p, m0, nt, ct0, width; };
    auto item_at = [&](int j, Item& it) -> bool {
        const int idx = group + j * n_groups;
        int tile, sub = 0, pr = 1;
        if (idx < full_items) {
            tile = idx;
        } else {
            const int u = idx - full_items;
            if (u >= (total - full_items) * parts) return false;
            tile = full_items + u / parts;
            sub = u % parts;
            pr = parts;
        }
        it.p = (NPROB == 2 && tile >= totp[0]) ? 1 : 0;       // one-problem launches index their problem statically
        const int lt = tile - (it.p ? totp[0] : 0);
        const int n_tiles = ntp[it.p];
        it.m0 = (lt / n_tiles) * TM + rank * TBM;
        it.nt = lt % n_tiles;
        int tile_w = BN;
        if (NPROB == 2) {
            // narrow last column tile where a W box of that height exists (128 or 64 columns at BN = 256)
            const int cols_left = ((L.p[it.p].N - it.nt * BN + 63) / 64) * 64;
            if (BN == 256 && (cols_left == 64 || cols_left == 128)) tile_w = cols_left;
        }
        it.width = pr == 1 ? tile_w : BN / pr;
        it.ct0 = it.nt * BN + sub * it.width;
        return sub * it.width < tile_w;        // a strip beyond a narrow tile's columns does not exist
    };

    if (warp == 0) {
        if (lane == 0) {
            // ------------------------------------------------------------ TMA producer
            for (int i = 0; i < NPROB; ++i) { prefetch_tmap(&L.p[i].ta); prefetch_tmap(&L.p[i].tw); }
            int it = 0;
            bool ok = true;
            Item wi;
            for (int j = 0; ok && item_at(j, wi); ++j) {
                // the W box that holds this CTA's share of the item's columns
                const TcProblem& P = L.p[wi.p];
                const CUtensorMap* wm = wi.width == BN ? &P.tw : ((BN == 256 && wi.width == 64) ? &P.tw3 : &P.tw2);
                const int wshare = wi.width / CG;
                const uint32_t bytes = CG * (S::A_BYTES + (uint32_t)wshare * TBK * 2);     // of the whole group
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    ok = mbar_wait(&empty[s], ph ^ 1, abort_flag, status, STATUS_GEMM_PRODUCER);
                    if (!ok) break;
#if defined(VTP_LINEAR_EXPERIMENT) && (VTP_LINEAR_EXPERIMENT & 1)
                    // measurement build: no operand traffic, the MMAs run on whatever the ring holds
                    (void)bytes; (void)wm;
                    mbar_arrive(&full[s]);
#else
                    if (CG == 1) {
                        mbar_arrive_expect_tx(&full[s], bytes);
                        tma_load_2d(smem_a + s * S::A_BYTES, &P.ta, &full[s], kb * TBK, wi.m0);
                        tma_load_2d(smem_b + s * S::B_BYTES, wm, &full[s], kb * TBK, wi.ct0);
                    } else {
                        // both CTAs' bytes are counted on rank 0's barrier, which its MMA thread waits on
                        if (rank == 0) mbar_arrive_expect_tx(&full[s], bytes);
                        const uint32_t fb = mapa_u32(smem_u32(&full[s]), 0);
                        tma_load_2d_pair(smem_a + s * S::A_BYTES, &P.ta, fb, kb * TBK, wi.m0);
                        tma_load_2d_pair(smem_b + s * S::B_BYTES, wm, fb, kb * TBK, wi.ct0 + rank * wshare);
                    }
#endif
                }
            }
            if (CG == 2 && ok) {
                // The MMA thread's last commits arrive on this CTA's `empty` barriers, from the partner for
                // rank 1: wait for them, so that nothing is signalled into a CTA that has retired.
                for (int s = 0; s < STAGES && ok; ++s) {
                    if (it <= s) break;
                    const int uses = (it - s + STAGES - 1) / STAGES;
                    ok = mbar_wait(&empty[s], (uses - 1) & 1, abort_flag, status, STATUS_GEMM_PRODUCER);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // -------------------------------------------------------------- MMA issuer (of the group)
            int it = 0, lt = 0;
            bool ok = true;
            Item wi;
            for (int j = 0; ok && item_at(j, wi); ++j, ++lt) {
                const uint32_t idesc = idesc_bf16_f32(TM, wi.width, 0, 0);
                const int buf = lt & 1;
                const uint32_t aph = (lt >> 1) & 1;
                ok = mbar_wait(&acc_empty[buf], aph ^ 1, abort_flag, status, STATUS_GEMM_MMA);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    ok = mbar_wait(&full[s], ph, abort_flag, status, STATUS_GEMM_MMA);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint64_t adesc = smem_desc_sw128(smem_u32(smem_a + s * S::A_BYTES));
                    const uint64_t bdesc = smem_desc_sw128(smem_u32(smem_b + s * S::B_BYTES));
#pragma unroll
                    for (int k = 0; k < TBK / 16; ++k) {
                        // 16 bf16 of K = 32 bytes = 2 descriptor address units inside the swizzle row
                        if (CG == 2) umma_ss_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                        else umma_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    if (CG == 2) umma_commit_pair(&empty[s]); else umma_commit(&empty[s]);
                }
                if (ok) { if (CG == 2) umma_commit_pair(&acc_full[buf]); else umma_commit(&acc_full[buf]); }
            }
        }
        __syncwarp();
    } else if (warp == 2 + EPI_THREADS / 32) {
        if (lane == 0 && L.p[0].use_tma_store) {
            // -------------------------------------------------------------- store thread
            // Walks the staged slabs in the epilogue's order: (item j, slab sl) of every item whose 128 rows
            // are all valid (the items with the last, partial rows come last and store from registers).
            struct Cursor { int j, sl; Item it; bool ok; };
            // the staged items: all 128 rows valid.  (Items with the last, partial rows of a problem store from
            // registers; they are skipped here exactly as the epilogue warps skip the staging for them.)
            auto staged = [&](const Item& it) { return it.m0 + TBM <= Mp[it.p]; };
            auto seek = [&](Cursor& c) {                  // first staged item at or after c.j
                for (;;) {
                    if (!item_at(c.j, c.it)) { c.ok = false; return; }
                    if (staged(c.it)) { c.ok = true; return; }
                    ++c.j;
                }
            };
            auto first = [&]() { Cursor c; c.j = 0; c.sl = 0; seek(c); return c; };
            auto advance = [&](Cursor& c) {
                if (++c.sl == c.it.width / 64) { c.sl = 0; ++c.j; seek(c); }
            };
            auto load_residual = [&](const Cursor& c, int b) {
                mbar_arrive_expect_tx(&res_full[b], TBM * 128);
                tma_load_2d(smem_out + b * (TBM * 128), &L.p[c.it.p].tr, &res_full[b], c.it.ct0 + c.sl * 64, c.it.m0);
            };
            Cursor cur = first(), ahead = cur;        // `ahead` runs NSTG slabs in front (residual prefetch)
            const bool res = L.p[0].res != nullptr;
            if (res) {
                for (int b = 0; b < NSTG && ahead.ok; ++b) { load_residual(ahead, b); advance(ahead); }
            }
            bool ok = true;
            for (int slab_no = 0; cur.ok && ok; ++slab_no, advance(cur)) {
                const int b = slab_no % NSTG;
                ok = mbar_wait(&slab_full[b], (slab_no / NSTG) & 1, abort_flag, status, STATUS_GEMM_EPILOGUE);
                if (!ok) break;
#if !(defined(VTP_LINEAR_EXPERIMENT) && (VTP_LINEAR_EXPERIMENT & 2))     // measurement build: no output traffic
                tma_store_2d(&L.p[cur.it.p].ty, smem_out + b * (TBM * 128), cur.it.ct0 + cur.sl * 64, cur.it.m0);
#endif
                bulk_commit_group();
                // every store but the newest STORES_IN_FLIGHT - 1 has read its slab: the slab of the last of those
                // can be written again (with a residual: it receives the residual of the slab NSTG further on)
                bulk_wait_group_read<STORES_IN_FLIGHT - 1>();
                if (slab_no >= STORES_IN_FLIGHT - 1) {
                    const int fb = (slab_no - (STORES_IN_FLIGHT - 1)) % NSTG;
                    if (res) {
                        if (ahead.ok) { load_residual(ahead, fb); advance(ahead); }
                    } else {
                        mbar_arrive(&slab_free[fb]);
                    }
                }
            }
            bulk_wait_group0();                       // every TMA store has landed before the CTA retires
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------- epilogue
        // the accumulator goes back to the MMA thread, which runs in the group's rank-0 CTA
        auto release_acc = [&](int b) {
            if (CG == 2) mbar_arrive_cluster(mapa_u32(smem_u32(&acc_empty[b]), 0));
            else mbar_arrive(&acc_empty[b]);
        };
        const int quarter = warp & 3;                 // TMEM lane quarter this warp may read
        const int qsub = (warp - 2) >> 2;             // which of the four warps of that quarter
        const int row = quarter * 32 + lane;          // tile row = TMEM lane
        int lt = 0, slab_no = 0;
        int held_p = -1, held_ct0 = -1, held_width = -1;   // the bias slice that is in shared memory
        bool ok = true;
        Item wi;
        for (int j = 0; ok && item_at(j, wi); ++j, ++lt) {
            const TcProblem& P = L.p[wi.p];
            const int M = Mp[wi.p], N = P.N;
            const float* __restrict__ bias = P.bias;
            const bf16* __restrict__ res = P.res;
            const LnFold& ln = P.ln;
            const int m0 = wi.m0;
            const int nt0 = wi.ct0;                   // first output column of the item
            const int NSLAB = wi.width / 64;          // 64-column slabs in it
            const int buf = lt & 1;
            const uint32_t aph = (lt >> 1) & 1;
            const bool tma_path = P.use_tma_store && m0 + TBM <= M;
            // A CTA whose tiles keep to one column range (a Linear no wider than a tile, or a column-tile count
            // that divides the grid) loads the slice once: a short-K tile is too brief to hide a global load and
            // two barriers of the sixteen warps in.
            const bool new_slice = tma_path && !(STAGES <= SHALLOW_RING && wi.p == held_p && nt0 == held_ct0 &&
                                                 wi.width == held_width);
            if (new_slice) {
                // this tile's bias slice -> shared memory (one value per thread), so the column
                // loop reads it as a broadcast instead of through the global-load path
                named_barrier(1, EPI_THREADS);                       // nobody reads the previous slice any more
                held_p = wi.p; held_ct0 = nt0; held_width = wi.width;
                const int te = threadIdx.x - 64;
                if (te < wi.width) {
                    bias_s[te] = (bias && nt0 + te < N) ? __ldg(bias + nt0 + te) : 0.f;
                    if (EPI & EPI_LN) bias_s[BN + te] = (nt0 + te < N) ? __ldg(ln.s + nt0 + te) : 0.f;
                }
            }
            ok = mbar_wait(&acc_full[buf], aph, abort_flag, status, STATUS_GEMM_EPILOGUE);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t tacc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            // folded LayerNorm: out = ln_a * acc + ln_b * s[n] + bias[n]
            float ln_a = 1.f, ln_b = 0.f;
            if ((EPI & EPI_LN) && m0 + row < M) {
                float2 st;
                if (ln.mode == 2) {
                    // partial (sum, sum of squares) left by the GEMM that produced the rows, one slot
                    // per (column tile, epilogue warp of the lane quarter); added in a fixed order
                    st = make_float2(0.f, 0.f);
                    const float4* sp = reinterpret_cast<const float4*>(ln.stats + (size_t)(m0 + row) * STAT_SLOTS);
                    float4 v4[STAT_SLOTS / 2];
#pragma unroll
                    for (int i = 0; i < STAT_SLOTS / 2; ++i)           // independent 16-byte loads, one latency
                        v4[i] = (2 * i < ln.slots) ? sp[i] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int i = 0; i < STAT_SLOTS / 2; ++i) { st.x += v4[i].x; st.y += v4[i].y; st.x += v4[i].z; st.y += v4[i].w; }
                } else {
                    st = ln.stats[m0 + row];
                }
                float mean = st.x, rstd = st.y;
                if (ln.mode == 2) {
                    mean = st.x / (float)ln.dim;
                    rstd = rsqrtf(fmaxf(st.y / (float)ln.dim - mean * mean, 0.f) + ln.eps);
                }
                ln_a = rstd;
                ln_b = -rstd * mean;
            }
            if (EPI & EPI_LN) {
                // warm L1 with the row statistics the next tile of this CTA will start with
                Item nxt;
                const int mn = (item_at(j + 1, nxt) && nxt.p == wi.p) ? nxt.m0 + row : M;
                if (mn < M) {
                    const float2* nxt = ln.stats + (size_t)mn * (ln.mode == 2 ? STAT_SLOTS : 1);
                    asm volatile("prefetch.global.L1 [%0];" ::"l"(nxt));
                }
            }
            float e1 = 0.f, e2 = 0.f;     // sum and sum of squares of this thread's outputs
            if (tma_path) {
                // ---- full tile: registers -> swizzled staging slab -> TMA store
                // The slab loop is unrolled (two register sets take the tensor-memory loads in turn, so nothing is
                // copied) and every shared-memory access goes through a 32-bit shared-space address worked out once
                // per tile: the tensor core pays for each instruction these sixteen warps issue.
                if (new_slice) named_barrier(1, EPI_THREADS);        // bias slice complete
                const uint32_t cell0 = (uint32_t)row * 128u + ((uint32_t)((qsub * 2) ^ (row & 7)) << 4);
                const uint32_t cell1 = (uint32_t)row * 128u + ((uint32_t)((qsub * 2 + 1) ^ (row & 7)) << 4);
                const uint32_t stage_a = smem_u32(smem_out);
                const uint32_t vec_a = smem_u32(bias_s) + (uint32_t)qsub * 64u;     // this thread's 16 columns of slab 0
                uint32_t rbuf[2][16];
                __syncwarp();
                tmem_ld_32x16(tacc + qsub * 16, rbuf[0]);
#pragma unroll
                for (int sl = 0; sl < BN / 64; ++sl) {
                    if (sl >= NSLAB || !ok) continue;
                    uint32_t (&r)[16] = rbuf[sl & 1];
                    // the additive part of this slab's 16 columns (bias, or bias + ln_b * s for a folded
                    // LayerNorm), fetched from shared memory while the accumulator columns are on their way
                    float cadd[16];
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const float4 b = lds_f4(vec_a + (uint32_t)sl * 256u + q4 * 16u);
                        cadd[4 * q4] = b.x; cadd[4 * q4 + 1] = b.y; cadd[4 * q4 + 2] = b.z; cadd[4 * q4 + 3] = b.w;
                        if (EPI & EPI_LN) {
                            const float4 sv = lds_f4(vec_a + (uint32_t)BN * 4u + (uint32_t)sl * 256u + q4 * 16u);
                            cadd[4 * q4] = fmaf(ln_b, sv.x, b.x); cadd[4 * q4 + 1] = fmaf(ln_b, sv.y, b.y);
                            cadd[4 * q4 + 2] = fmaf(ln_b, sv.z, b.z); cadd[4 * q4 + 3] = fmaf(ln_b, sv.w, b.w);
                        }
                    }
                    tmem_ld_wait();
                    if (sl + 1 < NSLAB) {
                        __syncwarp();
                        tmem_ld_32x16(tacc + (sl + 1) * 64 + qsub * 16, rbuf[(sl + 1) & 1]);     // next slab in flight
                    } else {
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) release_acc(buf);                        // accumulator is free
                    }
                    const int sb = slab_no % NSTG;                                // staging slab of this one
                    const uint32_t srow_a = stage_a + (uint32_t)sb * (TBM * 128);
                    if (res) {
                        // the residual of this slab is in the staging slab (so the slab is free, too)
                        ok = mbar_wait(&res_full[sb], (slab_no / NSTG) & 1, abort_flag, status,
                                       STATUS_GEMM_EPILOGUE);
                    } else if (slab_no >= NSTG) {
                        // the store of the slab that used this staging slab last has read it
                        ok = mbar_wait(&slab_free[sb], ((slab_no / NSTG) - 1) & 1, abort_flag, status,
                                       STATUS_GEMM_EPILOGUE);
                    }
                    if (!ok) continue;
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const uint32_t cell = srow_a + (j ? cell1 : cell0);
                        float vj[8];
                        if (EPI & EPI_LN) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) vj[i] = fmaf(ln_a, __uint_as_float(r[8 * j + i]), cadd[8 * j + i]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 8; ++i) vj[i] = __uint_as_float(r[8 * j + i]) + cadd[8 * j + i];
                        }
                        if (EPI & EPI_GELU) gelu8(vj);
                        if (res) {
                            Vec<bf16> rv;
                            float rf[8];
                            rv.raw = lds_u4(cell);                               // residual slab, same layout
                            rv.to_float(rf);
#pragma unroll
                            for (int i = 0; i < 8; ++i) vj[i] += rf[i];
                        }
                        if ((EPI & EPI_EMIT) && nt0 + sl * 64 + (qsub * 2 + j) * 8 < N) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) { e1 += vj[i]; e2 = fmaf(vj[i], vj[i], e2); }
                        }
                        Vec<bf16> ov;
                        ov.from_float(vj);
                        sts_u4(cell, ov.raw);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&slab_full[sb]);                // this warp's part of the slab is in place
                    ++slab_no;
                }
                if (!ok) break;
                if (EPI & EPI_EMIT) ln.emit[(size_t)(m0 + row) * STAT_SLOTS + wi.nt * 4 + qsub] = make_float2(e1, e2);
                continue;
            }
            // ---- boundary tile / row-remapped / fp32 output: store straight from registers
            const int m = m0 + row;
            const bool row_ok = m < M;
            const long long orow = map_out_row(P.rm, row_ok ? m : m0);
            const long long rrow = map_res_row(P.rm, row_ok ? m : m0);
            OutT* __restrict__ y = static_cast<OutT*>(P.y);
            const long long ldy = P.ldy, ldr = P.ldr;
            // same column split as the staged path (16 columns of each 64-column slab per warp), so a
            // row's statistics do not depend on which kind of tile it falls in
#pragma unroll 1
            for (int sl = 0; sl < NSLAB; ++sl) {
                const int n0 = nt0 + sl * 64 + qsub * 16;
                uint32_t r[16];
                __syncwarp();                 // tcgen05.ld is warp-collective
                tmem_ld_32x16(tacc + sl * 64 + qsub * 16, r);
                tmem_ld_wait();
                if (sl + 1 == NSLAB) {
                    // every column of this warp's slice is in registers: release the accumulator
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) release_acc(buf);
                }
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int n = n0 + 8 * j;
                    if (n >= N || !row_ok) continue;
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[8 * j + i]);
                    float bb[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    if (bias) {
                        const float4 b0 = __ldg(reinterpret_cast<const float4*>(bias + n));
                        const float4 b1 = __ldg(reinterpret_cast<const float4*>(bias + n) + 1);
                        bb[0] = b0.x; bb[1] = b0.y; bb[2] = b0.z; bb[3] = b0.w;
                        bb[4] = b1.x; bb[5] = b1.y; bb[6] = b1.z; bb[7] = b1.w;
                    }
                    if (EPI & EPI_LN) {
                        const float4 s0 = __ldg(reinterpret_cast<const float4*>(ln.s + n));
                        const float4 s1 = __ldg(reinterpret_cast<const float4*>(ln.s + n) + 1);
                        const float ss[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[i] = fmaf(ln_a, v[i], fmaf(ln_b, ss[i], bb[i]));
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[i] += bb[i];
                    }
                    if (EPI & EPI_GELU) gelu8(v);
                    if (res) {
                        Vec<bf16> rv;
                        float rf[8];
                        rv.load(res + rrow * ldr + n);
                        rv.to_float(rf);
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[i] += rf[i];
                    }
                    if (EPI & EPI_EMIT) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) { e1 += v[i]; e2 = fmaf(v[i], v[i], e2); }
                    }
                    OutVec<OutT>::store8(y + orow * ldy + n, v);
                }
            }
            if ((EPI & EPI_EMIT) && row_ok) ln.emit[(size_t)m * STAT_SLOTS + wi.nt * 4 + qsub] = make_float2(e1, e2);
        }
    }
    if (*abort_flag) {
        // Unwinding after a wait gave up: give copies still in flight time to land before
        // shared memory and TMEM are released.
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) { }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (CG == 2) cluster_sync_all();     // the partner no longer reads this CTA's operands or signals its barriers
    if (warp == 1) {
        if (CG == 2) tmem_dealloc_pair(tmem_base, S::TMEM_COLS);
        else tmem_dealloc(tmem_base, S::TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------ host

static EncodeTiledFn g_encode = nullptr;

EncodeTiledFn encode_tiled_fn() {
    if (g_encode) return g_encode;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || !fn) {
        cudaGetLastError();
        return nullptr;
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    return g_encode;
}

int make_tmap_bf16(CUtensorMap* map, const void* base, int rank, const unsigned long long* dims,
                   const unsigned long long* strides_bytes, const unsigned* box) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(VTP_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t gdim[5];
    cuuint64_t gstride[5];
    cuuint32_t bdim[5];
    cuuint32_t estride[5];
    for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; bdim[i] = box[i]; estride[i] = 1; }
    for (int i = 0; i + 1 < rank; ++i) gstride[i] = strides_bytes[i];
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdim,
                           gstride, bdim, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return (int)r;
    }
    return VTP_OK;
}

template <int BN, typename OutT>
static int fill_problem(TcProblem& q, const LinearArgs& p) {
    {
        const unsigned long long dims[2] = {(unsigned long long)p.K, (unsigned long long)p.m_max};
        const unsigned long long strides[1] = {(unsigned long long)p.lda * 2ull};
        const unsigned box[2] = {TBK, TBM};
        if (int rc = make_tmap_bf16(&q.ta, p.a, 2, dims, strides, box)) return rc;
    }
    {
        // W boxes: a whole tile, and the column strips of split tail tiles / narrow last tiles (half, or a
        // third for BN = 192, and a quarter)
        const unsigned long long dims[2] = {(unsigned long long)p.K, (unsigned long long)p.N};
        const unsigned long long strides[1] = {(unsigned long long)p.K * 2ull};
        // (each CTA of a group loads its share of the rows: box heights divide by CG)
        const unsigned box[2] = {TBK, BN / CG};
        if (int rc = make_tmap_bf16(&q.tw, p.w, 2, dims, strides, box)) return rc;
        const unsigned box2[2] = {TBK, (BN == 256 ? 128u : 64u) / CG};
        if (int rc = make_tmap_bf16(&q.tw2, p.w, 2, dims, strides, box2)) return rc;
        const unsigned box3[2] = {TBK, 64u / CG};
        if (int rc = make_tmap_bf16(&q.tw3, p.w, 2, dims, strides, box3)) return rc;
    }
    // Output map for the TMA-store epilogue (bf16 output, rows not remapped).
    q.use_tma_store = (sizeof(OutT) == 2 && p.out_grp == 0) ? 1 : 0;
    q.ty = q.tw;
    q.tr = q.tw;
    if (q.use_tma_store) {
        const unsigned long long dims[2] = {(unsigned long long)p.N, (unsigned long long)p.m_max};
        const unsigned long long strides[1] = {(unsigned long long)p.ldy * 2ull};
        const unsigned box[2] = {64, TBM};
        if (int rc = make_tmap_bf16(&q.ty, p.y, 2, dims, strides, box)) return rc;
        if (p.res) {
            const unsigned long long rstrides[1] = {(unsigned long long)p.ldr * 2ull};
            if (int rc = make_tmap_bf16(&q.tr, p.res, 2, dims, rstrides, box)) return rc;
        }
    }
    q.bias = p.bias; q.res = (const bf16*)p.res; q.ldr = p.ldr; q.y = p.y; q.ldy = p.ldy;
    q.m_max = p.m_max; q.m_dev = p.m_dev; q.N = p.N;
    q.rm = RowMap{p.out_grp, p.out_skip, p.res_mod, p.res_off};
    VTP_REQUIRE(!p.emit_stats || ceil_div(p.N, BN) * 4 <= STAT_SLOTS, VTP_ERR_SHAPE,
                "linear (tcgen05): N=%d has too many column tiles for the row-statistics slots", p.N);
    q.ln = LnFold{p.ln_stats, p.ln_s, p.ln_mode, p.ln_dim, p.ln_eps, p.emit_stats, p.ln_slots};
    return VTP_OK;
}

// p1 = null: one problem.  Otherwise two problems of the same K and epilogue kind in one launch.
template <int BN, int STAGES, typename OutT, int EPI>
static int launch_tc(const LinearArgs& p, const LinearArgs* p1, cudaStream_t st) {
    using S = TcSmem<BN, STAGES>;
    TcLaunch L;
    L.n = p1 ? 2 : 1;
    if (int rc = fill_problem<BN, OutT>(L.p[0], p)) return rc;
    if (p1) {
        if (int rc = fill_problem<BN, OutT>(L.p[1], *p1)) return rc;
    } else {
        L.p[1] = L.p[0];
    }
    if (p1 && !(BN == 256 && EPI == EPI_LN && sizeof(OutT) == 2))
        return fail(VTP_ERR_UNSUPPORTED, "linear (tcgen05): two-problem launches are built for 256-wide LayerNorm-fold tiles");
    auto kern = (p1 && BN == 256 && EPI == EPI_LN && sizeof(OutT) == 2) ? linear_tc_kernel<BN, STAGES, OutT, EPI, (BN == 256 && EPI == EPI_LN && sizeof(OutT) == 2) ? 2 : 1>
                                                                       : linear_tc_kernel<BN, STAGES, OutT, EPI, 1>;
    static bool attr_set[64][2] = {};   // per instantiation, device and problem count
    int dev = 0;
    cudaGetDevice(&dev);
    const int np = p1 ? 1 : 0;
    if (dev < 0 || dev >= 64 || !attr_set[dev][np]) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        if (e != cudaSuccess) {
            set_error("linear (tcgen05): cannot reserve %d bytes of shared memory: %s", S::TOTAL,
                      cudaGetErrorString(e));
            return (int)e;
        }
        if (dev >= 0 && dev < 64) attr_set[dev][np] = true;
    }
    long long tiles = (long long)ceil_div(p.N, BN) * ceil_div(p.m_max, TM);
    if (p1) tiles += (long long)ceil_div(p1->N, BN) * ceil_div(p1->m_max, TM);
    const int groups = sm_count() / CG;
    const int grid = CG * (int)(tiles < groups ? tiles : groups);
    const cudaError_t le = launch_pdl_cluster(kern, CG, dim3(grid), dim3(TC_THREADS), (size_t)S::TOTAL, st, L, p.K, device_status_ptr());
    if (le != cudaSuccess) {
        cudaGetLastError();
        set_error("linear (tcgen05): %s", cudaGetErrorString(le));
        return (int)le;
    }
    return check_launch("linear (tcgen05)");
}

static int pick_bn(int N) {
    // widest tile that does not pad N more than a narrower one would
    auto padded = [&](int bn) { return ceil_div(N, bn) * bn; };
    int bn = 256;
    if (padded(192) < padded(bn)) bn = 192;
    if (padded(128) < padded(bn)) bn = 128;
    return bn;
}

int linear_stat_slots(int N) { return ceil_div(N, pick_bn(N)) * 4; }

static int check_tc_args(const LinearArgs& p) {
    VTP_REQUIRE(p.dtype == VTP_BF16, VTP_ERR_DTYPE, "linear (tcgen05): bf16 operands only");
    VTP_REQUIRE(p.K % TBK == 0, VTP_ERR_SHAPE, "linear (tcgen05): K=%d must be a multiple of %d", p.K, TBK);
    VTP_REQUIRE(p.N % 8 == 0, VTP_ERR_SHAPE, "linear (tcgen05): N=%d must be a multiple of 8", p.N);
    VTP_REQUIRE(p.ln_mode == 0 || (p.ln_stats && p.ln_s && p.out_grp == 0 &&
                                   (p.ln_mode == 1 || (p.ln_dim > 0 && p.ln_slots > 0 && p.ln_slots <= STAT_SLOTS))),
                VTP_ERR_NULL, "linear (tcgen05): folded LayerNorm needs row statistics and the column sums");
    VTP_REQUIRE(p.lda % 8 == 0 && p.ldy % 8 == 0 && (!p.res || p.ldr % 8 == 0), VTP_ERR_ALIGN,
                "linear (tcgen05): row strides must be multiples of 16 bytes");
    return VTP_OK;
}

// Two independent Linears that follow the same kind of LayerNorm fold (the q and kv projections of a block)
// in ONE launch of 128 x 256 tiles: the tiles of the second problem fill the last, partial round of the first,
// and one launch's ramp and tail is saved.  Both: bf16 output, bias + folded LayerNorm (ln_mode 1), no
// residual, no row remap; N a multiple of 64.
bool linear_pair_supported(const LinearArgs& a, const LinearArgs& b) {
    auto ok = [](const LinearArgs& p) {
        // whole 64-column slabs: a last tile of 64 or 128 columns is a narrow tile, one of 192 a full tile whose
        // W rows beyond N the TMA load fills with zeros and whose last slab the TMA store drops
        return p.dtype == VTP_BF16 && p.ln_mode == 1 && !p.res && !p.emit_stats && p.out_grp == 0 && p.flags == 0 &&
               p.m_max > 0 && p.N >= 64 && p.N % 64 == 0;
    };
    return ok(a) && ok(b) && a.K == b.K;
}

int linear_tcgen05_pair(const LinearArgs& a, const LinearArgs& b, cudaStream_t st) {
    if (int rc = linear_validate(a)) return rc;
    if (int rc = linear_validate(b)) return rc;
    if (int rc = check_tc_args(a)) return rc;
    if (int rc = check_tc_args(b)) return rc;
    VTP_REQUIRE(linear_pair_supported(a, b), VTP_ERR_UNSUPPORTED, "linear (tcgen05): these two problems cannot share a launch");
    return launch_tc<256, ring_stages(256), bf16, EPI_LN>(a, &b, st);
}

int linear_tcgen05(const LinearArgs& p, cudaStream_t st) {
    if (p.m_max == 0) return VTP_OK;
    VTP_REQUIRE(p.dtype == VTP_BF16, VTP_ERR_DTYPE, "linear (tcgen05): bf16 operands only");
    VTP_REQUIRE(p.K % TBK == 0, VTP_ERR_SHAPE, "linear (tcgen05): K=%d must be a multiple of %d", p.K, TBK);
    VTP_REQUIRE(p.N % 8 == 0, VTP_ERR_SHAPE, "linear (tcgen05): N=%d must be a multiple of 8", p.N);
    VTP_REQUIRE(p.ln_mode == 0 || (p.ln_stats && p.ln_s && p.out_grp == 0 &&
                                   (p.ln_mode == 1 || (p.ln_dim > 0 && p.ln_slots > 0 && p.ln_slots <= STAT_SLOTS))),
                VTP_ERR_NULL, "linear (tcgen05): folded LayerNorm needs row statistics and the column sums");
    VTP_REQUIRE(p.lda % 8 == 0 && p.ldy % 8 == 0 && (!p.res || p.ldr % 8 == 0), VTP_ERR_ALIGN,
                "linear (tcgen05): row strides must be multiples of 16 bytes");
    const int bn = pick_bn(p.N);
    const bool f32 = (p.flags & VTP_FLAG_OUT_F32) != 0;
    const int epi = ((p.flags & VTP_FLAG_GELU) ? EPI_GELU : 0) | (p.ln_mode ? EPI_LN : 0) | (p.emit_stats ? EPI_EMIT : 0);
    if (f32) {
        VTP_REQUIRE(epi == 0, VTP_ERR_UNSUPPORTED, "linear (tcgen05): fp32 output supports bias and residual only");
        if (bn == 256) return launch_tc<256, ring_stages(256), float, 0>(p, nullptr, st);
        if (bn == 192) return launch_tc<192, ring_stages(192), float, 0>(p, nullptr, st);
        return launch_tc<128, ring_stages(128), float, 0>(p, nullptr, st);
    }
    const bool shallow = CG == 1 && bn == 128 && (p.K <= TBK || (p.K <= 2 * TBK && p.res));
#define VTP_TC_CASE(E)                                                  \
    if (epi == (E)) {                                                   \
        if (shallow) return launch_tc<128, SHALLOW_RING, bf16, (E)>(p, nullptr, st);            \
        if (bn == 256) return launch_tc<256, ring_stages(256), bf16, (E)>(p, nullptr, st);      \
        if (bn == 192) return launch_tc<192, ring_stages(192), bf16, (E)>(p, nullptr, st);      \
        return launch_tc<128, ring_stages(128), bf16, (E)>(p, nullptr, st);                     \
    }
    VTP_TC_CASE(0)
    VTP_TC_CASE(EPI_GELU)
    VTP_TC_CASE(EPI_LN)
    VTP_TC_CASE(EPI_LN | EPI_GELU)
    VTP_TC_CASE(EPI_EMIT)
#undef VTP_TC_CASE
    return fail(VTP_ERR_UNSUPPORTED, "linear (tcgen05): epilogue combination %d is not instantiated", epi);
}

}  // namespace vtp
