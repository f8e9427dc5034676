// Variable-length-query attention on tcgen05 tensor cores (bf16 in, fp32 accumulate).
//
// One CTA owns 128 packed queries of one (image, head).  Keys/values are walked in chunks
// of KC keys (KC a multiple of 16, at most 160; 257 keys -> 2 chunks of 144):
//   S = Q K_c^T        tcgen05.mma, A = Q tile, B = K chunk (both K-major, TMA, 128B swizzle),
//                      accumulator S in TMEM columns [0, KC)
//   P = exp2(scale*log2e*(S - rowmax))   4 softmax warps, one thread per query row, read S
//                      with tcgen05.ld, write bf16 P to shared memory in the swizzled K-major
//                      layout an A operand needs
//   O_c = P V_c        tcgen05.mma, B = V chunk as an MN-major operand straight from the TMA
//                      image of the [keys, d] rows; accumulator in TMEM columns [192, 256)
//   O  = O*alpha + O_c in registers of the softmax threads (online softmax rescale)
// Warp 0 lane 0 issues TMA, warp 1 lane 0 issues MMA, warps 2-5 do softmax and the output.
// K and V have separate single buffers, so the next K chunk streams in while softmax runs;
// two CTAs share an SM so one CTA's softmax overlaps the other's MMA.
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

constexpr int QT = 128;            // queries per CTA = TMEM lanes
constexpr int HD = 64;             // head dim
constexpr int KC_MAX = 160;        // keys per chunk, upper bound
constexpr int O_COL = 192;         // TMEM column of the P*V accumulator
constexpr int TMEM_COLS = 256;

constexpr int SM_Q = 0;
constexpr int SM_K = SM_Q + QT * HD * 2;              // 16384
constexpr int SM_V = SM_K + KC_MAX * HD * 2;          // 36864
constexpr int SM_P = SM_V + KC_MAX * HD * 2;          // 57344
constexpr int SM_BAR = SM_P + 3 * QT * 128;           // 106496
constexpr int ATT_SMEM = SM_BAR + 256 + 1024;

__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, int n, uint32_t (&r)[32]) {
    // n is 32 or 16 (warp-uniform)
    if (n == 32) {
        tmem_ld_32x32(taddr, r);
    } else {
        uint32_t h[16];
        tmem_ld_32x16(taddr, h);
#pragma unroll
        for (int i = 0; i < 16; ++i) r[i] = h[i];
    }
    tmem_ld_wait();
}

__global__ void __launch_bounds__(192)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const __grid_constant__ CUtensorMap tmap_v, long long q_hs, long long kv_hs,
               bf16* __restrict__ out, long long o_rs, long long o_hs, int n_keys, int KC, int n_chunks,
               const int32_t* __restrict__ offsets, float scale_log2e, int* status) {
    const int b = blockIdx.z, h = blockIdx.y;
    const int row0 = __ldg(offsets + b) + blockIdx.x * QT;
    const int row_end = __ldg(offsets + b + 1);
    if (row0 >= row_end) return;
    if (status && *reinterpret_cast<volatile int*>(status) != 0) return;
    const int nq = min(QT, row_end - row0);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + SM_BAR);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;
    uint64_t* k_free = bars + 2;
    uint64_t* v_full = bars + 3;
    uint64_t* v_free = bars + 4;
    uint64_t* s_full = bars + 5;
    uint64_t* p_full = bars + 6;
    uint64_t* o_full = bars + 7;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(k_full, 1); mbar_init(k_free, 1);
        mbar_init(v_full, 1); mbar_init(v_free, 1);
        mbar_init(s_full, 1); mbar_init(p_full, QT); mbar_init(o_full, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ------------------------------------------------------------ TMA producer
            prefetch_tmap(&tmap_q);
            prefetch_tmap(&tmap_k);
            prefetch_tmap(&tmap_v);
            mbar_arrive_expect_tx(q_full, QT * HD * 2);
            tma_load_2d(base + SM_Q, &tmap_q, q_full, (int)(h * q_hs), row0);
            const uint32_t kv_bytes = (uint32_t)KC * HD * 2;
            for (int j = 0; j < n_chunks; ++j) {
                const uint32_t ph = j & 1;
                if (!mbar_wait(k_free, ph ^ 1, abort_flag, status, STATUS_ATTN_LOAD)) break;
                mbar_arrive_expect_tx(k_full, kv_bytes);
                tma_load_3d(base + SM_K, &tmap_k, k_full, (int)(h * kv_hs), j * KC, b);
                if (!mbar_wait(v_free, ph ^ 1, abort_flag, status, STATUS_ATTN_LOAD)) break;
                mbar_arrive_expect_tx(v_full, kv_bytes);
                tma_load_3d(base + SM_V, &tmap_v, v_full, (int)(h * kv_hs), j * KC, b);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // -------------------------------------------------------------- MMA issuer
            const uint32_t idesc_s = idesc_bf16_f32(QT, KC, 0, 0);
            const uint32_t idesc_o = idesc_bf16_f32(QT, HD, 0, 1);     // B = V, MN-major
            const uint64_t qdesc = smem_desc_sw128(smem_u32(base + SM_Q));
            const uint64_t kdesc = smem_desc_sw128(smem_u32(base + SM_K));
            const uint64_t vdesc = smem_desc_sw128(smem_u32(base + SM_V));
            const uint64_t pdesc = smem_desc_sw128(smem_u32(base + SM_P));
            bool ok = mbar_wait(q_full, 0, abort_flag, status, STATUS_ATTN_MMA);
            for (int j = 0; j < n_chunks && ok; ++j) {
                const uint32_t ph = j & 1;
                ok = mbar_wait(k_full, ph, abort_flag, status, STATUS_ATTN_MMA);
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
                    // P: 64-key sub-tiles of 16 KB, 32 bytes per 16 keys inside the swizzle row.
                    // V: 16 keys = 16 rows of 128 bytes.
                    const uint64_t a = pdesc + (uint64_t)((t >> 2) * (QT * 128 >> 4)) + 2 * (t & 3);
                    const uint64_t bb = vdesc + (uint64_t)(t * (16 * 128 >> 4));
                    umma_ss(tmem_base + O_COL, a, bb, idesc_o, t != 0 ? 1u : 0u);
                }
                umma_commit(o_full);
                umma_commit(v_free);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------- softmax + output warps
        const int r = (warp & 3) * 32 + lane;                     // query row = TMEM lane
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        uint8_t* prow = base + SM_P + r * 128;
        float m = -INFINITY, l = 0.f;
        float o[HD];
#pragma unroll
        for (int i = 0; i < HD; ++i) o[i] = 0.f;
        bool ok = true;
        for (int j = 0; j < n_chunks && ok; ++j) {
            const uint32_t ph = j & 1;
            ok = mbar_wait(s_full, ph, abort_flag, status, STATUS_ATTN_SOFTMAX);
            if (!ok) break;
            tc_fence_after_sync();
            const int n_valid = min(KC, n_keys - j * KC);
            float mx = -INFINITY;
            for (int c0 = 0; c0 < KC; c0 += 32) {
                uint32_t s[32];
                const int n = min(32, KC - c0);
                __syncwarp();
                tmem_ld_cols(lane_base + c0, n, s);
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (i < n && c0 + i < n_valid) mx = fmaxf(mx, __uint_as_float(s[i]));
            }
            const float m_new = fmaxf(m, mx);
            const float alpha = exp2f((m - m_new) * scale_log2e);       // 0 on the first chunk
            const float mb = m_new * scale_log2e;
            float lsum = 0.f;
            for (int c0 = 0; c0 < KC; c0 += 32) {
                uint32_t s[32];
                const int n = min(32, KC - c0);
                __syncwarp();
                tmem_ld_cols(lane_base + c0, n, s);
                float p[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const bool valid = i < n && c0 + i < n_valid;
                    p[i] = valid ? exp2f(fmaf(__uint_as_float(s[i]), scale_log2e, -mb)) : 0.f;
                    lsum += p[i];
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if (8 * c < n) {
                        const int key = c0 + 8 * c;
                        Vec<bf16> pv;
                        pv.from_float(p + 8 * c);
                        uint8_t* dst = prow + (key >> 6) * (QT * 128) + ((((key & 63) >> 3) ^ (r & 7)) << 4);
                        *reinterpret_cast<uint4*>(dst) = pv.raw;
                    }
                }
            }
            fence_proxy_async_smem();          // P visible to the tensor core's async proxy
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
        }
        if (ok && r < nq) {
            const float inv = 1.0f / l;
            bf16* dst = out + (size_t)(row0 + r) * o_rs + h * o_hs;
#pragma unroll
            for (int c = 0; c < HD / 8; ++c) {
                float v8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v8[i] = o[8 * c + i] * inv;
                Vec<bf16> ov;
                ov.from_float(v8);
                ov.store(dst + 8 * c);
            }
        }
    }
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) { }     // let copies in flight land before releasing memory
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

int attention_tcgen05(const AttnArgs& p, cudaStream_t st) {
    VTP_REQUIRE(p.dtype == VTP_BF16, VTP_ERR_DTYPE, "attention (tcgen05): bf16 only");
    VTP_REQUIRE(p.head_dim == HD, VTP_ERR_UNSUPPORTED, "attention (tcgen05): head_dim %d (only %d)", p.head_dim, HD);
    VTP_REQUIRE(p.q_rs % 8 == 0 && p.q_hs % 8 == 0 && p.kv_rs % 8 == 0 && p.kv_hs % 8 == 0 && p.kv_bs % 8 == 0 &&
                    p.o_rs % 8 == 0 && p.o_hs % 8 == 0,
                VTP_ERR_ALIGN, "attention (tcgen05): strides must be multiples of 16 bytes");
    VTP_REQUIRE(aligned16(p.q) && aligned16(p.k) && aligned16(p.v) && aligned16(p.out), VTP_ERR_ALIGN,
                "attention (tcgen05): pointers must be 16-byte aligned");
    const int n_chunks = ceil_div(p.n_keys, KC_MAX);
    const int KC = (int)round_up(ceil_div(p.n_keys, n_chunks), 16);
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
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM);
        if (e != cudaSuccess) {
            set_error("attention (tcgen05): cannot reserve %d bytes of shared memory: %s", ATT_SMEM, cudaGetErrorString(e));
            return (int)e;
        }
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    const dim3 grid(ceil_div(p.max_q, QT), p.heads, p.B);
    attn_tc_kernel<<<grid, 192, ATT_SMEM, st>>>(tq, tk, tv, p.q_hs, p.kv_hs, (bf16*)p.out, p.o_rs, p.o_hs, p.n_keys, KC,
                                                n_chunks, p.offsets, p.scale * 1.4426950408889634f,
                                                device_status_ptr());
    return check_launch("attention (tcgen05)");
}

}  // namespace vtp
