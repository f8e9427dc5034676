// Linear layer on 5th-generation tensor cores (tcgen05), bf16 operands, fp32 accumulate in
// tensor memory, operands staged by TMA with a 128-byte swizzle.
//
//   y[m, n] = act(sum_k a[m,k] w[n,k] + bias[n]) + res[m, n]
//
// One CTA computes a 128 x BN tile.  Warp 0 (one lane) issues the TMA loads through a
// STAGES-deep ring of shared-memory buffers, warp 1 (one lane) issues tcgen05.mma and
// commits each stage back to the producer, then all four warps read the accumulator out of
// TMEM (warp w owns lanes 32w..32w+31 = tile rows) and apply bias / GELU / residual.
// Two CTAs fit on an SM (shared memory and TMEM), so one CTA's epilogue overlaps the
// other's main loop.  The number of valid rows is read from device memory: CTAs whose row
// tile starts beyond it exit at once, rows beyond it are never stored.
//
// Every mbarrier wait is bounded (see sm100.cuh); a wait that gives up ORs a code into the
// device status word and the CTA unwinds.
//
// Replaces nn.Linear q/kv/proj/fc1/fc2/head, nn.GELU and the residual adds of
// vtpack/models/dge/deit_dge.py:38-44,72-74,96,127-128 (cuBLAS + ATen kernels there).
#include "linear.h"
#include "runtime.h"
#include "sm100.cuh"

namespace vtp {

using namespace sm100;

constexpr int TBM = 128;   // tile rows = TMEM lanes
constexpr int TBK = 64;    // 64 bf16 = one 128-byte swizzle row

template <int BN, int STAGES>
struct TcSmem {
    static constexpr int A_BYTES = TBM * TBK * 2;
    static constexpr int B_BYTES = BN * TBK * 2;
    static constexpr int RING = STAGES * (A_BYTES + B_BYTES);
    static constexpr int TOTAL = RING + 1024 /* alignment slack */ + 256 /* barriers */;
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

template <int BN, int STAGES, typename OutT>
__global__ void __launch_bounds__(128)
linear_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                 const float* __restrict__ bias, const bf16* __restrict__ res, long long ldr,
                 OutT* __restrict__ y, long long ldy, int m_max, const int32_t* __restrict__ m_dev, int N,
                 int K, unsigned flags, RowMap rm, int* status) {
    using S = TcSmem<BN, STAGES>;
    int M = m_max;
    if (m_dev) M = min(__ldg(m_dev), m_max);
    const int m0 = blockIdx.y * TBM;
    const int n0 = blockIdx.x * BN;
    if (m0 >= M) return;
    // once any CTA has given up on a wait the launch is void: do not queue up more waits
    if (status && *reinterpret_cast<volatile int*>(status) != 0) return;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = base;
    uint8_t* smem_b = base + STAGES * S::A_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(base + S::RING);
    uint64_t* empty = full + STAGES;
    uint64_t* accum = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_kb = K / TBK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(accum, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, BN);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------------- TMA producer
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_w);
        for (int kb = 0; kb < num_kb; ++kb) {
            const int s = kb % STAGES;
            const uint32_t ph = (kb / STAGES) & 1;
            if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, status, STATUS_GEMM_PRODUCER)) break;
            mbar_arrive_expect_tx(&full[s], S::A_BYTES + S::B_BYTES);
            tma_load_2d(smem_a + s * S::A_BYTES, &tmap_a, &full[s], kb * TBK, m0);
            tma_load_2d(smem_b + s * S::B_BYTES, &tmap_w, &full[s], kb * TBK, n0);
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc = idesc_bf16_f32(TBM, BN, 0, 0);
        bool ok = true;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
            const int s = kb % STAGES;
            const uint32_t ph = (kb / STAGES) & 1;
            ok = mbar_wait(&full[s], ph, abort_flag, status, STATUS_GEMM_MMA);
            if (!ok) break;
            tc_fence_after_sync();
            const uint64_t adesc = smem_desc_sw128(smem_u32(smem_a + s * S::A_BYTES));
            const uint64_t bdesc = smem_desc_sw128(smem_u32(smem_b + s * S::B_BYTES));
#pragma unroll
            for (int k = 0; k < TBK / 16; ++k) {
                // 16 bf16 of K = 32 bytes = 2 descriptor address units inside the swizzle row
                umma_ss(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit(&empty[s]);
        }
        if (ok) umma_commit(accum);
    }
    __syncwarp();

    // ------------------------------------------------------------------------ epilogue
    const bool have_acc = mbar_wait(accum, 0, abort_flag, status, STATUS_GEMM_EPILOGUE);
    tc_fence_after_sync();
    if (have_acc) {
        const int m = m0 + warp * 32 + lane;
        const bool row_ok = m < M;
        const long long orow = map_out_row(rm, row_ok ? m : m0);
        const long long rrow = map_res_row(rm, row_ok ? m : m0);
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t r[32];
            __syncwarp();                 // tcgen05.ld is warp-collective
            tmem_ld_32x32(lane_base + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = n0 + c0 + 8 * j;
                if (n >= N || !row_ok) continue;
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[8 * j + i]);
                if (bias) {
                    const float4 b0 = __ldg(reinterpret_cast<const float4*>(bias + n));
                    const float4 b1 = __ldg(reinterpret_cast<const float4*>(bias + n) + 1);
                    v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
                    v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
                }
                if (flags & VTP_FLAG_GELU) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = gelu_erf(v[i]);
                }
                if (res) {
                    Vec<bf16> rv;
                    float rf[8];
                    rv.load(res + rrow * ldr + n);
                    rv.to_float(rf);
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] += rf[i];
                }
                OutVec<OutT>::store8(y + orow * ldy + n, v);
            }
        }
    } else {
        // Unwinding after a wait gave up: give copies still in flight time to land before
        // shared memory and TMEM are released.
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) { }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, BN);
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

template <int BN, int STAGES, typename OutT>
static int launch_tc(const LinearArgs& p, cudaStream_t st) {
    using S = TcSmem<BN, STAGES>;
    CUtensorMap ta, tw;
    {
        const unsigned long long dims[2] = {(unsigned long long)p.K, (unsigned long long)p.m_max};
        const unsigned long long strides[1] = {(unsigned long long)p.lda * 2ull};
        const unsigned box[2] = {TBK, TBM};
        if (int rc = make_tmap_bf16(&ta, p.a, 2, dims, strides, box)) return rc;
    }
    {
        const unsigned long long dims[2] = {(unsigned long long)p.K, (unsigned long long)p.N};
        const unsigned long long strides[1] = {(unsigned long long)p.K * 2ull};
        const unsigned box[2] = {TBK, BN};
        if (int rc = make_tmap_bf16(&tw, p.w, 2, dims, strides, box)) return rc;
    }
    auto kern = linear_tc_kernel<BN, STAGES, OutT>;
    static bool attr_set[64] = {};   // per instantiation and device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        if (e != cudaSuccess) {
            set_error("linear (tcgen05): cannot reserve %d bytes of shared memory: %s", S::TOTAL,
                      cudaGetErrorString(e));
            return (int)e;
        }
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    const dim3 grid(ceil_div(p.N, BN), ceil_div(p.m_max, TBM));
    const RowMap rm{p.out_grp, p.out_skip, p.res_mod, p.res_off};
    kern<<<grid, 128, S::TOTAL, st>>>(ta, tw, p.bias, (const bf16*)p.res, p.ldr, (OutT*)p.y, p.ldy, p.m_max,
                                      p.m_dev, p.N, p.K, p.flags, rm, device_status_ptr());
    return check_launch("linear (tcgen05)");
}

int linear_tcgen05(const LinearArgs& p, cudaStream_t st) {
    if (p.m_max == 0) return VTP_OK;
    VTP_REQUIRE(p.dtype == VTP_BF16, VTP_ERR_DTYPE, "linear (tcgen05): bf16 operands only");
    VTP_REQUIRE(p.K % TBK == 0, VTP_ERR_SHAPE, "linear (tcgen05): K=%d must be a multiple of %d", p.K, TBK);
    VTP_REQUIRE(p.N % 8 == 0, VTP_ERR_SHAPE, "linear (tcgen05): N=%d must be a multiple of 8", p.N);
    VTP_REQUIRE(p.lda % 8 == 0 && p.ldy % 8 == 0 && (!p.res || p.ldr % 8 == 0), VTP_ERR_ALIGN,
                "linear (tcgen05): row strides must be multiples of 16 bytes");
    if (p.flags & VTP_FLAG_OUT_F32) return launch_tc<128, 3, float>(p, st);
    return launch_tc<128, 3, bf16>(p, st);
}

}  // namespace vtp
