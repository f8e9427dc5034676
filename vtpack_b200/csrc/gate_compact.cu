// Router gate (region mean -> Linear -> argmax) and patch-list compaction.
//
// Replaces DynamicRouter.forward / gate.argmax (vtpack/layers/dge.py:145-150,75) and
// grained_sample_index_to_patch (vtpack/layers/csrc/grained_sample/grained_sample.cu:146-196,
// 302-345).  Unlike the reference nothing is copied to the host: the per-image counts and
// their exclusive prefix stay in device memory for the kernels that follow.
#include "region_ops.h"

namespace vtp {

// One warp per region.  Lanes stride over 16-byte channel chunks, sum the region's
// tokens in (dy, dx) order in fp32, divide by the token count, then take n_splits dot
// products with the fp32 gate weights.  HBM-bound: reads B*H*W*C elements once.
template <typename T, int MAXCH>
__global__ void __launch_bounds__(128)
router_gate_kernel(const T* __restrict__ x, int n_regions, int Hr, int Wr, int W, int N, int C,
                   int num_extra, int region, const float* __restrict__ gw,
                   const float* __restrict__ gb, int S, float* __restrict__ logits_out,
                   int32_t* __restrict__ idx_out) {
    constexpr int VN = Vec<T>::N;
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= n_regions) return;
    const int b = r / (Hr * Wr);
    const int ry = (r / Wr) % Hr;
    const int rx = r % Wr;
    const int nchunks = C / VN;

    float acc[MAXCH][VN];
#pragma unroll
    for (int ch = 0; ch < MAXCH; ++ch)
#pragma unroll
        for (int i = 0; i < VN; ++i) acc[ch][i] = 0.f;

    const T* img = x + (size_t)b * N * C;
    for (int dy = 0; dy < region; ++dy) {
        const T* row0 = img + (size_t)(num_extra + (ry * region + dy) * W + rx * region) * C;
#pragma unroll 4
        for (int dx = 0; dx < region; ++dx) {
#pragma unroll
            for (int ch = 0; ch < MAXCH; ++ch) {
                const int chunk = lane + 32 * ch;
                if (chunk < nchunks) {
                    Vec<T> v;
                    v.load(row0 + (size_t)dx * C + chunk * VN);
                    float f[VN];
                    v.to_float(f);
#pragma unroll
                    for (int i = 0; i < VN; ++i) acc[ch][i] += f[i];
                }
            }
        }
    }
    const float denom = (float)(region * region);
    float best = 0.f;
    int best_i = 0;
    for (int s = 0; s < S; ++s) {
        float p = 0.f;
#pragma unroll
        for (int ch = 0; ch < MAXCH; ++ch) {
            const int chunk = lane + 32 * ch;
            if (chunk < nchunks) {
                const float4* wp = reinterpret_cast<const float4*>(gw + (size_t)s * C + chunk * VN);
#pragma unroll
                for (int i4 = 0; i4 < VN / 4; ++i4) {
                    const float4 w4 = __ldg(wp + i4);
                    p = fmaf(acc[ch][4 * i4 + 0] / denom, w4.x, p);
                    p = fmaf(acc[ch][4 * i4 + 1] / denom, w4.y, p);
                    p = fmaf(acc[ch][4 * i4 + 2] / denom, w4.z, p);
                    p = fmaf(acc[ch][4 * i4 + 3] / denom, w4.w, p);
                }
            }
        }
        p = warp_sum(p) + __ldg(gb + s);
        if (lane == 0 && logits_out) logits_out[(size_t)r * S + s] = p;
        if (s == 0 || p > best) { best = p; best_i = s; }   // first maximum wins
    }
    if (lane == 0) idx_out[r] = best_i;
}

__global__ void gate_argmax_kernel(const float* __restrict__ logits, int rows, int S,
                                   int32_t* __restrict__ idx_out) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    float best = logits[(size_t)r * S];
    int best_i = 0;
    for (int s = 1; s < S; ++s) {
        const float p = logits[(size_t)r * S + s];
        if (p > best) { best = p; best_i = s; }
    }
    idx_out[r] = best_i;
}

// One warp per image: counts[b] = num_extra + sum over regions of split^2.
template <typename I>
__global__ void count_kernel(const I* __restrict__ idx, int B, int R, Splits sp, int num_extra,
                             int32_t* __restrict__ counts) {
    const int lane = threadIdx.x & 31;
    const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= B) return;
    int c = 0;
    for (int r = lane; r < R; r += 32) {
        int k = (int)idx[(size_t)b * R + r];
        k = min(max(k, 0), sp.n - 1);
        c += sp.v[k] * sp.v[k];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if (lane == 0) counts[b] = c + num_extra;
}

// One CTA per image.  The image's first row is the sum of the counts in front of it;
// regions are scanned in shared memory; then (region, dy) items write their rows
// [b, y, x, step], sub-patches row-major, extra tokens first.
template <typename I>
__global__ void __launch_bounds__(128)
write_patches_kernel(const I* __restrict__ idx, int B, int Hr, int Wr, Splits sp, int region,
                     int num_extra, const int32_t* __restrict__ counts,
                     int32_t* __restrict__ offsets, int32_t* __restrict__ patches,
                     int64_t* __restrict__ patches64, int32_t* __restrict__ region_first) {
    extern __shared__ int s_start[];   // [R + 1] first row of each region within the image
    __shared__ int s_warp[4];
    __shared__ int s_base;
    const int b = blockIdx.x;
    const int R = Hr * Wr;
    const int tid = threadIdx.x;

    int part = 0;
    for (int j = tid; j < b; j += blockDim.x) part += counts[j];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if ((tid & 31) == 0) s_warp[tid >> 5] = part;
    for (int r = tid; r < R; r += blockDim.x) {
        int k = (int)idx[(size_t)b * R + r];
        k = min(max(k, 0), sp.n - 1);
        s_start[r + 1] = sp.v[k];      // split for now, turned into a prefix below
    }
    __syncthreads();
    if (tid == 0) {
        const int base = s_warp[0] + s_warp[1] + s_warp[2] + s_warp[3];
        s_base = base;
        offsets[b] = base;
        if (b == B - 1) offsets[B] = base + counts[b];
        int run = num_extra;
        s_start[0] = run;
        for (int r = 0; r < R; ++r) {
            const int s = s_start[r + 1];
            run += s * s;
            s_start[r + 1] = run;
        }
    }
    __syncthreads();
    const int base = s_base;
    if (region_first)
        for (int r = tid; r < R; r += blockDim.x) region_first[(size_t)b * R + r] = base + s_start[r];

    for (int e = tid; e < num_extra && patches; e += blockDim.x) {
        const int row = base + e;
        reinterpret_cast<int4*>(patches)[row] = make_int4(b, -e - 1, 0, 1);
        if (patches64) {
            longlong2* p = reinterpret_cast<longlong2*>(patches64 + (size_t)row * 4);
            p[0] = make_longlong2(b, -e - 1);
            p[1] = make_longlong2(0, 1);
        }
    }
    const int items = R * region;           // (region, dy) with dy < split
    if (!patches) return;
    for (int it = tid; it < items; it += blockDim.x) {
        const int r = it / region;
        const int dy = it % region;
        const int first = s_start[r];
        const int rows = s_start[r + 1] - first;      // split^2
        int s = 1;
        while (s * s < rows) ++s;
        if (dy >= s) continue;
        const int step = region / s;
        const int y = (r / Wr) * region + dy * step;
        const int x0 = (r % Wr) * region;
        int row = base + first + dy * s;
        for (int dx = 0; dx < s; ++dx, ++row) {
            reinterpret_cast<int4*>(patches)[row] = make_int4(b, y, x0 + dx * step, step);
            if (patches64) {
                longlong2* p = reinterpret_cast<longlong2*>(patches64 + (size_t)row * 4);
                p[0] = make_longlong2(b, y);
                p[1] = make_longlong2(x0 + dx * step, step);
            }
        }
    }
}

template <typename T>
static int launch_router(const void* x, int B, int H, int W, int C, int num_extra, int region,
                         const float* gw, const float* gb, int S, float* logits, int32_t* idx,
                         cudaStream_t st) {
    const int Hr = H / region, Wr = W / region;
    const int n_regions = B * Hr * Wr;
    const int N = num_extra + H * W;
    const int nchunks = C / Vec<T>::N;
    const int maxch = ceil_div(nchunks, 32);
    const int grid = ceil_div(n_regions, 4);
    const T* xp = static_cast<const T*>(x);
#define VTP_LAUNCH_ROUTER(M)                                                                   \
    router_gate_kernel<T, M><<<grid, 128, 0, st>>>(xp, n_regions, Hr, Wr, W, N, C, num_extra,  \
                                                   region, gw, gb, S, logits, idx)
    if (maxch <= 1) VTP_LAUNCH_ROUTER(1);
    else if (maxch == 2) VTP_LAUNCH_ROUTER(2);
    else if (maxch == 3) VTP_LAUNCH_ROUTER(3);
    else if (maxch == 4) VTP_LAUNCH_ROUTER(4);
    else if (maxch <= 6) VTP_LAUNCH_ROUTER(6);
    else return fail(VTP_ERR_SHAPE, "router gate: C=%d too large", C);
#undef VTP_LAUNCH_ROUTER
    return check_launch("router_gate");
}

}  // namespace vtp

using namespace vtp;

extern "C" int vtp_router_gate(const void* x, int dtype, int B, int H, int W, int C,
                               int num_extra, int region, const float* gate_w,
                               const float* gate_b, int n_splits, float* logits_out,
                               int32_t* grain_idx, void* stream) {
    VTP_REQUIRE(x && gate_w && gate_b && grain_idx, VTP_ERR_NULL, "router gate: null pointer");
    VTP_REQUIRE(dtype == VTP_F32 || dtype == VTP_BF16, VTP_ERR_DTYPE, "router gate: dtype %d", dtype);
    VTP_REQUIRE(B > 0 && H > 0 && W > 0 && region > 0 && H % region == 0 && W % region == 0,
                VTP_ERR_SHAPE, "router gate: grid %dx%d not divisible by region %d", H, W, region);
    VTP_REQUIRE(n_splits >= 1 && n_splits <= 8 && num_extra >= 0, VTP_ERR_SHAPE,
                "router gate: n_splits %d", n_splits);
    VTP_REQUIRE(C > 0 && C % (16 / (int)elem_size(dtype)) == 0 && C % 4 == 0, VTP_ERR_SHAPE,
                "router gate: C=%d must be a multiple of 16 bytes", C);
    VTP_REQUIRE(aligned16(x) && aligned16(gate_w), VTP_ERR_ALIGN, "router gate: unaligned pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == VTP_F32)
        return launch_router<float>(x, B, H, W, C, num_extra, region, gate_w, gate_b, n_splits,
                                    logits_out, grain_idx, st);
    return launch_router<bf16>(x, B, H, W, C, num_extra, region, gate_w, gate_b, n_splits,
                               logits_out, grain_idx, st);
}

extern "C" int vtp_gate_argmax(const float* logits, int rows, int n_splits, int32_t* grain_idx,
                               void* stream) {
    VTP_REQUIRE(logits && grain_idx, VTP_ERR_NULL, "gate argmax: null pointer");
    VTP_REQUIRE(rows >= 0 && n_splits >= 1, VTP_ERR_SHAPE, "gate argmax: bad shape");
    if (rows == 0) return VTP_OK;
    gate_argmax_kernel<<<ceil_div(rows, 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        logits, rows, n_splits, grain_idx);
    return check_launch("gate_argmax");
}

namespace vtp {
int index_to_patch(const void* indices, int idx_is_i64, const Splits& sp, int B, int Hr, int Wr, int region,
                   int num_extra, int32_t* counts, int32_t* offsets, int32_t* patches, int64_t* patches64,
                   int32_t* region_first, cudaStream_t st) {
    const int R = Hr * Wr;
    const size_t smem = (size_t)(R + 1) * sizeof(int);
    if (idx_is_i64) {
        const int64_t* ip = static_cast<const int64_t*>(indices);
        count_kernel<int64_t><<<ceil_div(B, 4), 128, 0, st>>>(ip, B, R, sp, num_extra, counts);
        write_patches_kernel<int64_t><<<B, 128, smem, st>>>(ip, B, Hr, Wr, sp, region, num_extra, counts, offsets,
                                                            patches, patches64, region_first);
    } else {
        const int32_t* ip = static_cast<const int32_t*>(indices);
        count_kernel<int32_t><<<ceil_div(B, 4), 128, 0, st>>>(ip, B, R, sp, num_extra, counts);
        write_patches_kernel<int32_t><<<B, 128, smem, st>>>(ip, B, Hr, Wr, sp, region, num_extra, counts, offsets,
                                                            patches, patches64, region_first);
    }
    return check_launch("index_to_patch");
}

int make_splits(Splits* sp, const int* splits, int n_splits, int region) {
    VTP_REQUIRE(n_splits >= 1 && n_splits <= 8, VTP_ERR_SHAPE, "index_to_patch: n_splits %d", n_splits);
    sp->n = n_splits;
    for (int i = 0; i < 8; ++i) sp->v[i] = 1;
    for (int i = 0; i < n_splits; ++i) {
        VTP_REQUIRE(splits[i] >= 1 && splits[i] <= region && region % splits[i] == 0, VTP_ERR_SHAPE,
                    "index_to_patch: split %d does not divide region %d", splits[i], region);
        sp->v[i] = splits[i];
    }
    return VTP_OK;
}
}  // namespace vtp

extern "C" int vtp_index_to_patch(const void* indices, int idx_is_i64, const int* splits, int n_splits, int B,
                                  int Hr, int Wr, int region, int num_extra, int32_t* counts, int32_t* offsets,
                                  int32_t* patches, int64_t* patches64, void* stream) {
    VTP_REQUIRE(indices && splits && counts && offsets && patches, VTP_ERR_NULL, "index_to_patch: null pointer");
    VTP_REQUIRE(B > 0 && Hr > 0 && Wr > 0 && region > 0 && num_extra >= 0, VTP_ERR_SHAPE,
                "index_to_patch: bad shape");
    VTP_REQUIRE(Hr * Wr <= 8192, VTP_ERR_SHAPE, "index_to_patch: %d regions per image", Hr * Wr);
    Splits sp;
    if (int rc = make_splits(&sp, splits, n_splits, region)) return rc;
    VTP_REQUIRE(aligned16(patches) && (!patches64 || aligned16(patches64)), VTP_ERR_ALIGN,
                "index_to_patch: unaligned patch buffer");
    return index_to_patch(indices, idx_is_i64, sp, B, Hr, Wr, region, num_extra, counts, offsets, patches,
                          patches64, nullptr, static_cast<cudaStream_t>(stream));
}
