// Region-parallel token movers used by the fused block forward: router gate, multi-grain
// pooling (with LayerNorm statistics or explicit LayerNorm rows) and replicate-unpool with
// residual.  One CTA of four warps owns one 4x4 region of the token grid, whatever grain
// the gate picked for it: warp w owns grid row w.  A token row is spread over a GROUP of G
// lanes, each lane holding CPL chunks of 16 bytes (C = G * CPL * 16 bytes exactly, e.g.
// 16 lanes x 3 chunks at C=384 bf16), so no lane idles and no access needs a bounds check;
// a warp holds 32/G groups.  All 16 rows of a region are requested before any arithmetic,
// every region costs the same, and nothing depends on walking the patch list.
// Sums that span tokens go through shared memory: each group sums its own tokens in order,
// then the partial sums of a patch are added top-left to bottom-right (the reference adds
// the same tokens in one sequential chain; results differ by fp32 rounding only).
//
// Replaces DynamicRouter.forward (vtpack/layers/dge.py:145-150), grained_sample_compress /
// grained_sample_decompress (vtpack/layers/csrc/grained_sample/grained_sample.cu:31-69,
// 107-144) and the nn.LayerNorm norm1 calls of Block.forward
// (vtpack/models/dge/deit_dge.py:127) on the fused path.
#include "region_ops.h"
#include "runtime.h"

namespace vtp {

constexpr int RG = 4;              // tokens per region side = warps per CTA

template <typename T, int G, int CPL>
struct Lay {
    static constexpr int VN = Vec<T>::N;
    static constexpr int GROUPS = 32 / G;          // token rows a warp holds at once
    static constexpr int TPG = RG / GROUPS;        // tokens of a grid row per group (4, 2 or 1)
};

// group-wide sum over the G lanes that share a row
template <int G>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename T, int CPL>
__device__ __forceinline__ void load_row(Vec<T> (&r)[CPL], const T* src, int sub, int G) {
#pragma unroll
    for (int ch = 0; ch < CPL; ++ch) r[ch].load(src + (sub + G * ch) * Vec<T>::N);
}
template <typename T, int CPL>
__device__ __forceinline__ void store_row(const Vec<T> (&r)[CPL], T* dst, int sub, int G) {
#pragma unroll
    for (int ch = 0; ch < CPL; ++ch) r[ch].store(dst + (sub + G * ch) * Vec<T>::N);
}
template <typename T, int CPL>
__device__ __forceinline__ void to_f(float (&f)[CPL][Vec<T>::N], const Vec<T> (&r)[CPL]) {
#pragma unroll
    for (int ch = 0; ch < CPL; ++ch) r[ch].to_float(f[ch]);
}
template <typename T, int CPL>
__device__ __forceinline__ void zero_f(float (&f)[CPL][Vec<T>::N]) {
#pragma unroll
    for (int ch = 0; ch < CPL; ++ch)
#pragma unroll
        for (int i = 0; i < Vec<T>::N; ++i) f[ch][i] = 0.f;
}
// shared-memory row of C floats, accessed as float4 (a lane's chunk is VN consecutive floats)
template <typename T, int CPL>
__device__ __forceinline__ void smem_store(float* row, const float (&f)[CPL][Vec<T>::N], int sub, int G) {
    constexpr int VN = Vec<T>::N;
#pragma unroll
    for (int ch = 0; ch < CPL; ++ch)
#pragma unroll
        for (int i = 0; i < VN / 4; ++i)
            reinterpret_cast<float4*>(row + (sub + G * ch) * VN)[i] =
                make_float4(f[ch][4 * i], f[ch][4 * i + 1], f[ch][4 * i + 2], f[ch][4 * i + 3]);
}
template <typename T, int CPL>
__device__ __forceinline__ void smem_add(float (&f)[CPL][Vec<T>::N], const float* row, int sub, int G) {
    constexpr int VN = Vec<T>::N;
#pragma unroll
    for (int ch = 0; ch < CPL; ++ch)
#pragma unroll
        for (int i = 0; i < VN / 4; ++i) {
            const float4 v = reinterpret_cast<const float4*>(row + (sub + G * ch) * VN)[i];
            f[ch][4 * i] += v.x; f[ch][4 * i + 1] += v.y; f[ch][4 * i + 2] += v.z; f[ch][4 * i + 3] += v.w;
        }
}

// (sum, sum of squares) of a row held across a group
template <typename T, int G, int CPL>
__device__ __forceinline__ float2 row_sums(const float (&f)[CPL][Vec<T>::N]) {
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int ch = 0; ch < CPL; ++ch)
#pragma unroll
        for (int i = 0; i < Vec<T>::N; ++i) { s1 += f[ch][i]; s2 = fmaf(f[ch][i], f[ch][i], s2); }
    return make_float2(group_sum<G>(s1), group_sum<G>(s2));
}
// (mean, rstd) from (sum, sum of squares): exact enough for bf16 rows (8 significant bits)
__device__ __forceinline__ float2 mean_rstd(float2 s, int C, float eps) {
    const float mean = s.x / (float)C;
    return make_float2(mean, rsqrtf(fmaxf(s.y / (float)C - mean * mean, 0.f) + eps));
}

// explicit LayerNorm of a row (two-pass) and store
template <typename T, int G, int CPL>
__device__ __forceinline__ void ln_store(const float (&f)[CPL][Vec<T>::N], int sub, int C,
                                         const float* __restrict__ lnw, const float* __restrict__ lnb, float eps,
                                         T* dst) {
    constexpr int VN = Vec<T>::N;
    float s = 0.f;
#pragma unroll
    for (int ch = 0; ch < CPL; ++ch)
#pragma unroll
        for (int i = 0; i < VN; ++i) s += f[ch][i];
    const float mean = group_sum<G>(s) / (float)C;
    float v = 0.f;
#pragma unroll
    for (int ch = 0; ch < CPL; ++ch)
#pragma unroll
        for (int i = 0; i < VN; ++i) { const float d = f[ch][i] - mean; v = fmaf(d, d, v); }
    const float rstd = rsqrtf(group_sum<G>(v) / (float)C + eps);
#pragma unroll
    for (int ch = 0; ch < CPL; ++ch) {
        const int c0 = (sub + G * ch) * VN;
        float o[VN];
#pragma unroll
        for (int i = 0; i < VN; ++i) o[i] = (f[ch][i] - mean) * rstd * __ldg(lnw + c0 + i) + __ldg(lnb + c0 + i);
        Vec<T> ov;
        ov.from_float(o);
        ov.store(dst + c0);
    }
}

// round a row to T (what the consumer GEMM will read), store it, keep the rounded values
template <typename T, int CPL>
__device__ __forceinline__ void round_store(float (&f)[CPL][Vec<T>::N], T* dst, int sub, int G) {
#pragma unroll
    for (int ch = 0; ch < CPL; ++ch) {
        Vec<T> ov;
        ov.from_float(f[ch]);
        ov.store(dst + (sub + G * ch) * Vec<T>::N);
        ov.to_float(f[ch]);
    }
}

// packed row of a region's first query, from the per-image counts and the grain indices of
// the image's earlier regions (executed redundantly by every warp)
__device__ __forceinline__ int derive_first(const int32_t* __restrict__ counts, const int32_t* __restrict__ idx, int b,
                                            int rr, int R, const Splits& sp, int num_extra, int lane, int* img_base) {
    int part_sum = 0, own = 0;
    for (int j = lane; j < b; j += 32) part_sum += counts[j];
    for (int r = lane; r < rr; r += 32) {
        const int kk = min(max(idx[b * R + r], 0), sp.n - 1);
        own += sp.v[kk] * sp.v[kk];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        part_sum += __shfl_xor_sync(0xffffffffu, part_sum, o);
        own += __shfl_xor_sync(0xffffffffu, own, o);
    }
    *img_base = part_sum;
    return part_sum + num_extra + own;
}

// Each group leaves the in-order sum of its tokens of grid row w in shared memory.
// Slot layout: part[(w * 2 + half) * C], half 0 = left two tokens of the row, 1 = right two.
// A group that owns the whole row (TPG == 4) fills slot (w, 0) only, unless it was told to
// split (`left` holds the first two tokens, `acc` the last two).  Groups that own a single
// token (TPG == 1) are paired through shared memory.  Ends with the CTA barrier.
template <typename T, int G, int CPL>
__device__ __forceinline__ void publish_partials(float* part, float (&acc)[CPL][Vec<T>::N], int w, int grp, int sub,
                                                 int C) {
    constexpr int TPG = Lay<T, G, CPL>::TPG;
    if (TPG == 4) {
        smem_store<T, CPL>(part + (size_t)(w * 2) * C, acc, sub, G);
    } else if (TPG == 2) {
        smem_store<T, CPL>(part + (size_t)(w * 2 + grp) * C, acc, sub, G);
    } else {
        float* slot = part + (size_t)(w * 2 + (grp >> 1)) * C;
        if ((grp & 1) == 0) smem_store<T, CPL>(slot, acc, sub, G);
        __syncwarp();
        if ((grp & 1) == 1) {
            float tmp[CPL][Vec<T>::N];
            zero_f<T, CPL>(tmp);
            smem_add<T, CPL>(tmp, slot, sub, G);          // even token first, then the odd one
#pragma unroll
            for (int ch = 0; ch < CPL; ++ch)
#pragma unroll
                for (int i = 0; i < Vec<T>::N; ++i) tmp[ch][i] += acc[ch][i];
            smem_store<T, CPL>(slot, tmp, sub, G);
        }
    }
    __syncthreads();
}

// ------------------------------------------------------------------------------- pool
// POOL_STATS: comp rows + (mean, rstd) of every comp row (and of every token row unless
//             they are already known), for the GEMMs that apply LayerNorm in their
//             epilogue; zeroes the stats_acc rows.
// POOL_LN:    comp rows + explicit LN(x) rows and LN(comp) rows.
// POOL_PLAIN: comp rows only, as means or (sum_only) as sums: the latter is the gradient of the
//             replicate-unpool with respect to its packed rows (vtpack/layers/grained_sample.py:61-72).
// Seven CTAs per SM (at most 73 registers, a few spilled words): the kernel is bound by how many
// regions are in flight, and measured faster over the whole forward than at the 88 registers / five
// CTAs the compiler picks on its own (six: +0.5 %, seven: +0.9 %, eight: +0.8 %).
constexpr int POOL_LN = 0, POOL_STATS = 1, POOL_PLAIN = 2;
// (A thread of a narrow-row layout holds one or two 16-byte vectors of a region: such kernels run with 16 or 12 CTAs per SM
// (a few spilled words in the unpool; measured faster all the same), and the kernel is bound by how many regions are in flight.)
template <typename T, int G, int CPL, int MODE>
__global__ void __launch_bounds__(128, (Lay<T, G, CPL>::TPG * CPL <= 1) ? 16 : ((Lay<T, G, CPL>::TPG * CPL <= 2) ? 12 : 7))
pool_region_kernel(const T* __restrict__ x, RegionGeom g, const int32_t* __restrict__ idx,
                   const int32_t* __restrict__ region_first, const int32_t* __restrict__ offsets,
                   const int32_t* __restrict__ counts, int32_t* __restrict__ offsets_out,
                   int32_t* __restrict__ region_first_out, int32_t* __restrict__ counts_next, Splits sp,
                   T* __restrict__ comp, float2* __restrict__ stats_x, float2* __restrict__ stats_q,
                   float2* __restrict__ stats_acc, int write_stats_x, const float* __restrict__ lnw,
                   const float* __restrict__ lnb, float eps, T* __restrict__ xn, T* __restrict__ qn, int sum_only,
                   int* status) {
    constexpr bool STATS = MODE == POOL_STATS, EXPLICIT_LN = MODE == POOL_LN;
    using L = Lay<T, G, CPL>;
    constexpr int VN = L::VN, GROUPS = L::GROUPS, TPG = L::TPG;
    extern __shared__ float part[];          // [4 grid rows][2 halves][C] partial sums
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int grp = lane / G, sub = lane % G;
    const int R = g.Hr * g.Wr;
    const int rid = blockIdx.x;

    if (rid >= g.B * R) {
        // ---- extra (cls) tokens: one per group, copied
        const int e = ((rid - g.B * R) * RG + w) * GROUPS + grp;
        if (e >= g.B * g.num_extra) return;
        const int b = e / g.num_extra, t = e % g.num_extra;
        const size_t src_row = (size_t)b * g.N + t;
        int dst_row;
        if (region_first) {
            dst_row = offsets[b] + t;
            if (VTP_INDEX_GUARDS && g.l_max > 0 && (dst_row < 0 || dst_row >= g.l_max)) {   // caller's offsets
                if (sub == 0 && status) atomicOr(status, STATUS_BAD_INDEX);
                return;
            }
        } else {
            int base = 0;
            for (int j = sub; j < b; j += G) base += counts[j];
#pragma unroll
            for (int o = G / 2; o > 0; o >>= 1) base += __shfl_xor_sync(0xffffffffu, base, o);
            dst_row = base + t;
            // start the next block's per-image count at the extra tokens; its gate adds the rest
            if (t == 0 && sub == 0 && counts_next) counts_next[b] = g.num_extra;
        }
        Vec<T> row[CPL];
        load_row<T, CPL>(row, x + src_row * g.C, sub, G);
        store_row<T, CPL>(row, comp + (size_t)dst_row * g.C, sub, G);
        float f[CPL][VN];
        to_f<T, CPL>(f, row);
        if (STATS) {
            float2 st;
            if (write_stats_x) {
                st = mean_rstd(row_sums<T, G, CPL>(f), g.C, eps);
                if (sub == 0) stats_x[src_row] = st;
            } else {
                st = stats_x[src_row];
            }
            if (sub == 0) { stats_q[dst_row] = st; if (stats_acc) stats_acc[dst_row] = make_float2(0.f, 0.f); }
        } else if (EXPLICIT_LN) {
            ln_store<T, G, CPL>(f, sub, g.C, lnw, lnb, eps, xn + src_row * g.C);
            ln_store<T, G, CPL>(f, sub, g.C, lnw, lnb, eps, qn + (size_t)dst_row * g.C);
        }
        return;
    }

    const int b = rid / R, rr = rid % R;
    const int ry = rr / g.Wr, rx = rr % g.Wr;
    const int k = min(max(idx[rid], 0), sp.n - 1);
    const int s = sp.v[k];                     // sub-patches per region side: 4, 2 or 1
    const int step = RG / s;
    // this group's tokens: grid row w, columns grp*TPG .. grp*TPG + TPG - 1
    const size_t tok0 = (size_t)b * g.N + g.num_extra + (size_t)(ry * RG + w) * g.W + rx * RG + grp * TPG;

    Vec<T> rows[TPG][CPL];
#pragma unroll
    for (int j = 0; j < TPG; ++j) load_row<T, CPL>(rows[j], x + (tok0 + j) * g.C, sub, G);

    int first;
    if (region_first) {
        first = region_first[rid];
        // a caller-supplied first row whose patches would not fit the packed array: skip the region
        if (VTP_INDEX_GUARDS && g.l_max > 0 && (first < 0 || first + s * s > g.l_max)) {
            if (threadIdx.x == 0 && status) atomicOr(status, STATUS_BAD_INDEX);
            return;
        }
    } else {
        int img_base;
        first = derive_first(counts, idx, b, rr, R, sp, g.num_extra, lane, &img_base);
        if (w == 0 && lane == 0) {
            region_first_out[rid] = first;
            if (rr == 0) {
                offsets_out[b] = img_base;
                if (b == g.B - 1) offsets_out[g.B] = img_base + counts[b];
                // a grid without extra tokens has no extra-token CTA to start the next block's count
                if (counts_next && g.num_extra == 0) counts_next[b] = 0;
            }
        }
    }

    // per token: statistics / explicit LayerNorm, and at the finest grain the token is its own patch
    float acc[CPL][VN];                          // in-order sum of this group's tokens (of the current half)
    zero_f<T, CPL>(acc);
#pragma unroll
    for (int j = 0; j < TPG; ++j) {
        float f[CPL][VN];
        to_f<T, CPL>(f, rows[j]);
        const int col = grp * TPG + j;                        // column inside the grid row
        const int prow = first + w * RG + col;                // packed row if step == 1
        if (STATS) {
            float2 st = make_float2(0.f, 1.f);
            if (write_stats_x) {
                st = mean_rstd(row_sums<T, G, CPL>(f), g.C, eps);
                if (sub == 0) stats_x[tok0 + j] = st;
            } else if (step == 1) {
                st = stats_x[tok0 + j];
            }
            if (step == 1 && sub == 0) { stats_q[prow] = st; if (stats_acc) stats_acc[prow] = make_float2(0.f, 0.f); }
        } else if (EXPLICIT_LN) {
            ln_store<T, G, CPL>(f, sub, g.C, lnw, lnb, eps, xn + (tok0 + j) * g.C);
            if (step == 1) ln_store<T, G, CPL>(f, sub, g.C, lnw, lnb, eps, qn + (size_t)prow * g.C);
        }
        if (step == 1) {
            store_row<T, CPL>(rows[j], comp + (size_t)prow * g.C, sub, G);
        } else {
#pragma unroll
            for (int ch = 0; ch < CPL; ++ch)
#pragma unroll
                for (int i = 0; i < VN; ++i) acc[ch][i] += f[ch][i];
            // a group that owns the whole grid row closes the left half after two tokens (2x2 patches)
            if (TPG == 4 && step == 2 && j == 1) {
                smem_store<T, CPL>(part + (size_t)(w * 2) * g.C, acc, sub, G);
                zero_f<T, CPL>(acc);
            }
        }
    }
    if (step == 1) return;

    if (TPG == 4 && step == 2) {
        smem_store<T, CPL>(part + (size_t)(w * 2 + 1) * g.C, acc, sub, G);
        __syncthreads();
    } else {
        publish_partials<T, G, CPL>(part, acc, w, grp, sub, g.C);
    }
    const bool row_in_one_slot = (TPG == 4) && step == 4;     // slot (w, 0) holds the whole grid row

    // finishing: unit u = w * GROUPS + grp takes patch u.  step 2: four patches (dy, dx); step 4: one.
    const int u = w * GROUPS + grp;
    if (u >= s * s) return;
    const int dy = (step == 2) ? (u >> 1) : 0;
    const int dx = (step == 2) ? (u & 1) : 0;
    zero_f<T, CPL>(acc);
    if (step == 2) {
        smem_add<T, CPL>(acc, part + (size_t)((2 * dy) * 2 + dx) * g.C, sub, G);
        smem_add<T, CPL>(acc, part + (size_t)((2 * dy + 1) * 2 + dx) * g.C, sub, G);
    } else {
        for (int r2 = 0; r2 < RG; ++r2) {
            smem_add<T, CPL>(acc, part + (size_t)(r2 * 2) * g.C, sub, G);
            if (!row_in_one_slot) smem_add<T, CPL>(acc, part + (size_t)(r2 * 2 + 1) * g.C, sub, G);
        }
    }
    // step * step is 4 or 16: multiplying by its reciprocal is the division, bit for bit
    const float inv_denom = sum_only ? 1.0f : 1.0f / (float)(step * step);
#pragma unroll
    for (int ch = 0; ch < CPL; ++ch)
#pragma unroll
        for (int i = 0; i < VN; ++i) acc[ch][i] = acc[ch][i] * inv_denom;
    const int row = first + dy * s + dx;
    if (STATS) {
        round_store<T, CPL>(acc, comp + (size_t)row * g.C, sub, G);
        const float2 st = mean_rstd(row_sums<T, G, CPL>(acc), g.C, eps);
        if (sub == 0) { stats_q[row] = st; if (stats_acc) stats_acc[row] = make_float2(0.f, 0.f); }
    } else {
        if (EXPLICIT_LN) ln_store<T, G, CPL>(acc, sub, g.C, lnw, lnb, eps, qn + (size_t)row * g.C);
        round_store<T, CPL>(acc, comp + (size_t)row * g.C, sub, G);
    }
}

// ------------------------------------------------------------------------ router gate
// Region mean of the raw tokens (/ 16), n_splits fp32 dot products, argmax with the lowest
// index winning ties.  `part` holds the partial row sums published by publish_partials;
// executed by one group of G lanes.
template <typename T, int G, int CPL>
__device__ __forceinline__ void gate_from_partials(const float* part, int C, int sub, const float* __restrict__ gw,
                                                   const float* __restrict__ gb, int S, float* __restrict__ logits_out,
                                                   int32_t* __restrict__ idx_out, int rid, int32_t* counts_img,
                                                   const Splits& sp, const float* __restrict__ img_bias) {
    constexpr int VN = Vec<T>::N;
    constexpr bool both_halves = Lay<T, G, CPL>::TPG != 4;
    float acc[CPL][VN];
    zero_f<T, CPL>(acc);
    for (int r2 = 0; r2 < RG; ++r2) {
        smem_add<T, CPL>(acc, part + (size_t)(r2 * 2) * C, sub, G);
        if (both_halves) smem_add<T, CPL>(acc, part + (size_t)(r2 * 2 + 1) * C, sub, G);
    }
    // the region mean: 1/16 is a power of two, so the product equals the quotient
#pragma unroll
    for (int ch = 0; ch < CPL; ++ch)
#pragma unroll
        for (int i = 0; i < VN; ++i) acc[ch][i] *= 1.0f / (float)(RG * RG);
    float best = 0.f;
    int best_i = 0;
    for (int sI = 0; sI < S; ++sI) {
        float pdot = 0.f;
#pragma unroll
        for (int ch = 0; ch < CPL; ++ch) {
            const float4* wp = reinterpret_cast<const float4*>(gw + (size_t)sI * C + (sub + G * ch) * VN);
#pragma unroll
            for (int i4 = 0; i4 < VN / 4; ++i4) {
                const float4 w4 = __ldg(wp + i4);
                pdot = fmaf(acc[ch][4 * i4 + 0], w4.x, pdot);
                pdot = fmaf(acc[ch][4 * i4 + 1], w4.y, pdot);
                pdot = fmaf(acc[ch][4 * i4 + 2], w4.z, pdot);
                pdot = fmaf(acc[ch][4 * i4 + 3], w4.w, pdot);
            }
        }
        pdot = group_sum<G>(pdot) + __ldg(gb + sI);
        if (img_bias) pdot += __ldg(img_bias + sI);          // per-image offset of the logits (forced grain mixes)
        if (sub == 0 && logits_out) logits_out[(size_t)rid * S + sI] = pdot;
        if (sI == 0 || pdot > best) { best = pdot; best_i = sI; }
    }
    if (sub == 0) {
        idx_out[rid] = best_i;
        // queries this region contributes to its image (the image's slot starts at num_extra)
        if (counts_img) atomicAdd(counts_img, sp.v[min(best_i, sp.n - 1)] * sp.v[min(best_i, sp.n - 1)]);
    }
}

// ----------------------------------------------------------------------------- unpool
// out[b,tok] = ref[b,tok] + (q[p] - comp[p]) for the patch p that covers the token; optionally
// also the next block's token statistics, router gate decisions and per-image counts.
template <typename T, int G, int CPL>
__global__ void __launch_bounds__(128, (Lay<T, G, CPL>::TPG * CPL <= 1) ? 16 : ((Lay<T, G, CPL>::TPG * CPL <= 2) ? 12 : 4))
unpool_region_kernel(const T* __restrict__ q, const T* __restrict__ comp, const T* ref, T* out, RegionGeom g,
                     const int32_t* __restrict__ idx, const int32_t* __restrict__ region_first,
                     const int32_t* __restrict__ offsets, Splits sp, NextBlock nx) {
    using L = Lay<T, G, CPL>;
    constexpr int VN = L::VN, GROUPS = L::GROUPS, TPG = L::TPG;
    extern __shared__ float part[];          // [4 grid rows][2 halves][C] row sums of the output (next gate)
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int grp = lane / G, sub = lane % G;
    const int R = g.Hr * g.Wr;
    const int rid = blockIdx.x;

    if (rid >= g.B * R) {
        const int e = ((rid - g.B * R) * RG + w) * GROUPS + grp;
        if (e >= g.B * g.num_extra) return;
        const int b = e / g.num_extra, t = e % g.num_extra;
        const size_t tok = (size_t)b * g.N + t;
        const size_t p = (size_t)(offsets[b] + t);
        Vec<T> qv[CPL], cv[CPL], rv[CPL];
        load_row<T, CPL>(qv, q + p * g.C, sub, G);
        load_row<T, CPL>(cv, comp + p * g.C, sub, G);
        load_row<T, CPL>(rv, ref + tok * g.C, sub, G);
        float qf[CPL][VN], cf[CPL][VN], rf[CPL][VN];
        to_f<T, CPL>(qf, qv); to_f<T, CPL>(cf, cv); to_f<T, CPL>(rf, rv);
#pragma unroll
        for (int ch = 0; ch < CPL; ++ch)
#pragma unroll
            for (int i = 0; i < VN; ++i) rf[ch][i] = (qf[ch][i] - cf[ch][i]) + rf[ch][i];
        round_store<T, CPL>(rf, out + tok * g.C, sub, G);
        if (nx.stats_x) {
            const float2 st = mean_rstd(row_sums<T, G, CPL>(rf), g.C, nx.eps);
            if (sub == 0) nx.stats_x[tok] = st;
        }
        return;
    }
    const int b = rid / R, rr = rid % R;
    const int ry = rr / g.Wr, rx = rr % g.Wr;
    const int k = min(max(idx[rid], 0), sp.n - 1);
    const int s = sp.v[k];
    const int step = RG / s;
    const int first = region_first[rid];
    const size_t tok0 = (size_t)b * g.N + g.num_extra + (size_t)(ry * RG + w) * g.W + rx * RG + grp * TPG;
    const int prow = first + (w / step) * s;            // packed row of this grid row's first patch

    // every row this group needs, requested up front: TPG reference rows and the patch rows they map to.
    // At the finest grain a token is its own patch and comp[p] is a copy of ref[tok], so
    // ref + (q - comp) is q: neither ref nor comp is read (a third of the regions on average; the
    // grain is the same for the whole CTA, so nothing diverges)
    const bool fine = step == 1;
    Vec<T> rrow[TPG][CPL], qrow[TPG][CPL], crow[TPG][CPL];
#pragma unroll
    for (int j = 0; j < TPG; ++j) {
        const int col = grp * TPG + j;
        if (!fine) load_row<T, CPL>(rrow[j], ref + (tok0 + j) * g.C, sub, G);
        if (j == 0 || (col % step) == 0) {               // a new patch starts at this column
            const int p = prow + col / step;
            load_row<T, CPL>(qrow[j], q + (size_t)p * g.C, sub, G);
            if (!fine) load_row<T, CPL>(crow[j], comp + (size_t)p * g.C, sub, G);
        }
    }
    float acc[CPL][VN];                                  // in-order sum of this group's output tokens
    zero_f<T, CPL>(acc);
    float d[CPL][VN];
    zero_f<T, CPL>(d);
#pragma unroll
    for (int j = 0; j < TPG; ++j) {
        const int col = grp * TPG + j;
        if (j == 0 || (col % step) == 0) {
            to_f<T, CPL>(d, qrow[j]);
            if (!fine) {
                float cf[CPL][VN];
                to_f<T, CPL>(cf, crow[j]);
#pragma unroll
                for (int ch = 0; ch < CPL; ++ch)
#pragma unroll
                    for (int i = 0; i < VN; ++i) d[ch][i] -= cf[ch][i];
            }
        }
        float o[CPL][VN];
        if (fine) {
#pragma unroll
            for (int ch = 0; ch < CPL; ++ch)
#pragma unroll
                for (int i = 0; i < VN; ++i) o[ch][i] = d[ch][i];
        } else {
            to_f<T, CPL>(o, rrow[j]);
#pragma unroll
            for (int ch = 0; ch < CPL; ++ch)
#pragma unroll
                for (int i = 0; i < VN; ++i) o[ch][i] = d[ch][i] + o[ch][i];
        }
        round_store<T, CPL>(o, out + (tok0 + j) * g.C, sub, G);       // o now holds the rounded values
        if (nx.stats_x) {
            const float2 st = mean_rstd(row_sums<T, G, CPL>(o), g.C, nx.eps);
            if (sub == 0) nx.stats_x[tok0 + j] = st;
#pragma unroll
            for (int ch = 0; ch < CPL; ++ch)
#pragma unroll
                for (int i = 0; i < VN; ++i) acc[ch][i] += o[ch][i];
        }
    }
    if (!nx.gw) return;
    // ---- the next block's router gate on the region this CTA has just written
    publish_partials<T, G, CPL>(part, acc, w, grp, sub, g.C);
    if (w != 0 || grp != 0) return;
    gate_from_partials<T, G, CPL>(part, g.C, sub, nx.gw, nx.gb, nx.S, nx.logits, nx.idx, rid,
                                  nx.counts ? nx.counts + b : nullptr, sp,
                                  nx.image_bias ? nx.image_bias + (size_t)b * nx.S : nullptr);
}

// Stand-alone gate (first block of a model, or a block called on its own); optionally also
// writes the LayerNorm statistics of every token row it reads.
template <typename T, int G, int CPL>
__global__ void __launch_bounds__(128)
gate_region_kernel(const T* __restrict__ x, RegionGeom g, const float* __restrict__ gw,
                   const float* __restrict__ gb, int S, float* __restrict__ logits_out,
                   int32_t* __restrict__ idx_out, float2* __restrict__ stats_x, float eps,
                   const float* __restrict__ image_bias) {
    using L = Lay<T, G, CPL>;
    constexpr int VN = L::VN, GROUPS = L::GROUPS, TPG = L::TPG;
    extern __shared__ float part[];          // [4][2][C]
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int grp = lane / G, sub = lane % G;
    const int R = g.Hr * g.Wr;
    const int rid = blockIdx.x;
    if (rid >= g.B * R) {
        // extra (cls) tokens only matter for the statistics
        const int e = ((rid - g.B * R) * RG + w) * GROUPS + grp;
        if (!stats_x || e >= g.B * g.num_extra) return;
        const size_t tok = (size_t)(e / g.num_extra) * g.N + e % g.num_extra;
        Vec<T> row[CPL];
        load_row<T, CPL>(row, x + tok * g.C, sub, G);
        float f[CPL][VN];
        to_f<T, CPL>(f, row);
        const float2 st = mean_rstd(row_sums<T, G, CPL>(f), g.C, eps);
        if (sub == 0) stats_x[tok] = st;
        return;
    }
    const int b = rid / R, rr = rid % R;
    const int ry = rr / g.Wr, rx = rr % g.Wr;
    const size_t tok0 = (size_t)b * g.N + g.num_extra + (size_t)(ry * RG + w) * g.W + rx * RG + grp * TPG;
    Vec<T> rows[TPG][CPL];
#pragma unroll
    for (int j = 0; j < TPG; ++j) load_row<T, CPL>(rows[j], x + (tok0 + j) * g.C, sub, G);
    float acc[CPL][VN];
    zero_f<T, CPL>(acc);
#pragma unroll
    for (int j = 0; j < TPG; ++j) {
        float f[CPL][VN];
        to_f<T, CPL>(f, rows[j]);
        if (stats_x) {
            const float2 st = mean_rstd(row_sums<T, G, CPL>(f), g.C, eps);
            if (sub == 0) stats_x[tok0 + j] = st;
        }
#pragma unroll
        for (int ch = 0; ch < CPL; ++ch)
#pragma unroll
            for (int i = 0; i < VN; ++i) acc[ch][i] += f[ch][i];
    }
    publish_partials<T, G, CPL>(part, acc, w, grp, sub, g.C);
    if (w != 0 || grp != 0) return;
    Splits none;
    none.n = 1; none.v[0] = 0;
    gate_from_partials<T, G, CPL>(part, g.C, sub, gw, gb, S, logits_out, idx_out, rid, nullptr, none,
                                  image_bias ? image_bias + (size_t)b * S : nullptr);
}

// ------------------------------------------------------------------------------- host

// (G, CPL) with G * CPL == number of 16-byte chunks in a row; false if the row does not factor
static bool pick_layout(int nchunks, int* G, int* CPL) {
    static const int cpls[] = {3, 2, 1, 6, 4, 5};      // 5: C = 320 (PVT stage 3) is 8 lanes x 5 chunks in bf16
    for (int c : cpls)
        for (int g = 32; g >= 8; g >>= 1)
            if (g * c == nchunks && (g == 32 || c <= 3 || c == 5)) { *G = g; *CPL = c; return true; }
    return false;
}

template <typename T, int G, int CPL>
static void launch_pool_t(const RegionPoolArgs& a, cudaStream_t st) {
    const int R = a.g.Hr * a.g.Wr;
    const int grid = a.g.B * R + ceil_div(a.g.B * a.g.num_extra, RG * (32 / G));
    const size_t smem = (size_t)8 * a.g.C * sizeof(float);
    if (a.stats_q)
        pool_region_kernel<T, G, CPL, POOL_STATS><<<grid, 128, smem, st>>>(
            (const T*)a.x, a.g, a.idx, a.region_first, a.offsets, a.counts, a.offsets_out, a.region_first_out,
            a.counts_next, a.sp, (T*)a.comp, a.stats_x, a.stats_q, a.stats_acc, a.stats_x_ready ? 0 : 1, nullptr,
            nullptr, a.eps, nullptr, nullptr, 0, nullptr);
    else if (a.xn && a.qn)
        pool_region_kernel<T, G, CPL, POOL_LN><<<grid, 128, smem, st>>>(
            (const T*)a.x, a.g, a.idx, a.region_first, a.offsets, a.counts, a.offsets_out, a.region_first_out,
            a.counts_next, a.sp, (T*)a.comp, nullptr, nullptr, nullptr, 0, a.lnw, a.lnb, a.eps, (T*)a.xn, (T*)a.qn, 0, nullptr);
    else
        pool_region_kernel<T, G, CPL, POOL_PLAIN><<<grid, 128, smem, st>>>(
            (const T*)a.x, a.g, a.idx, a.region_first, a.offsets, a.counts, a.offsets_out, a.region_first_out,
            a.counts_next, a.sp, (T*)a.comp, nullptr, nullptr, nullptr, 0, nullptr, nullptr, a.eps, nullptr, nullptr,
            a.sum_only ? 1 : 0, device_status_ptr());
}

template <typename T, int G, int CPL>
static void launch_unpool_t(const RegionUnpoolArgs& a, cudaStream_t st) {
    const int R = a.g.Hr * a.g.Wr;
    const int grid = a.g.B * R + ceil_div(a.g.B * a.g.num_extra, RG * (32 / G));
    unpool_region_kernel<T, G, CPL><<<grid, 128, (size_t)8 * a.g.C * sizeof(float), st>>>(
        (const T*)a.q, (const T*)a.comp, (const T*)a.ref, (T*)a.out, a.g, a.idx, a.region_first, a.offsets, a.sp, a.next);
}

template <typename T, int G, int CPL>
static void launch_gate_t(const RegionGateArgs& a, cudaStream_t st) {
    const int R = a.g.Hr * a.g.Wr;
    const int grid = a.g.B * R + (a.stats_x ? ceil_div(a.g.B * a.g.num_extra, RG * (32 / G)) : 0);
    gate_region_kernel<T, G, CPL><<<grid, 128, (size_t)8 * a.g.C * sizeof(float), st>>>(
        (const T*)a.x, a.g, a.gw, a.gb, a.S, a.logits_out, a.idx_out, a.stats_x, a.eps, a.image_bias);
}

#define VTP_DISPATCH_LAYOUT(FN, T, ARGS, ST)                                    \
    do {                                                                        \
        int G = 0, CPL = 0;                                                     \
        if (!pick_layout((ARGS).g.C / Vec<T>::N, &G, &CPL))                     \
            return fail(VTP_ERR_SHAPE, "C=%d has no lane layout", (ARGS).g.C);  \
        if (G == 32 && CPL == 3) FN<T, 32, 3>(ARGS, ST);                        \
        else if (G == 16 && CPL == 3) FN<T, 16, 3>(ARGS, ST);                   \
        else if (G == 8 && CPL == 3) FN<T, 8, 3>(ARGS, ST);                     \
        else if (G == 32 && CPL == 2) FN<T, 32, 2>(ARGS, ST);                   \
        else if (G == 16 && CPL == 2) FN<T, 16, 2>(ARGS, ST);                   \
        else if (G == 8 && CPL == 2) FN<T, 8, 2>(ARGS, ST);                     \
        else if (G == 32 && CPL == 1) FN<T, 32, 1>(ARGS, ST);                   \
        else if (G == 16 && CPL == 1) FN<T, 16, 1>(ARGS, ST);                   \
        else if (G == 8 && CPL == 1) FN<T, 8, 1>(ARGS, ST);                     \
        else if (G == 32 && CPL == 6) FN<T, 32, 6>(ARGS, ST);                   \
        else if (G == 32 && CPL == 4) FN<T, 32, 4>(ARGS, ST);                   \
        else if (G == 32 && CPL == 5) FN<T, 32, 5>(ARGS, ST);                   \
        else if (G == 16 && CPL == 5) FN<T, 16, 5>(ARGS, ST);                   \
        else if (G == 8 && CPL == 5) FN<T, 8, 5>(ARGS, ST);                     \
        else return fail(VTP_ERR_SHAPE, "C=%d has no lane layout", (ARGS).g.C); \
    } while (0)

bool region_ops_supported(const RegionGeom& g, int dtype) {
    const int vn = dtype == VTP_BF16 ? 8 : 4;
    int G, CPL;
    if (g.region != RG || g.C % vn != 0 || g.B <= 0 || g.Hr <= 0 || g.Wr <= 0) return false;
    return pick_layout(g.C / vn, &G, &CPL);
}

int region_pool(const RegionPoolArgs& a, int dtype, cudaStream_t st) {
    if (dtype == VTP_F32) VTP_DISPATCH_LAYOUT(launch_pool_t, float, a, st);
    else VTP_DISPATCH_LAYOUT(launch_pool_t, bf16, a, st);
    return check_launch("pool (region)");
}

int region_unpool(const RegionUnpoolArgs& a, int dtype, cudaStream_t st) {
    if (dtype == VTP_F32) VTP_DISPATCH_LAYOUT(launch_unpool_t, float, a, st);
    else VTP_DISPATCH_LAYOUT(launch_unpool_t, bf16, a, st);
    return check_launch("unpool (region)");
}

int region_gate(const RegionGateArgs& a, int dtype, cudaStream_t st) {
    if (dtype == VTP_F32) VTP_DISPATCH_LAYOUT(launch_gate_t, float, a, st);
    else VTP_DISPATCH_LAYOUT(launch_gate_t, bf16, a, st);
    return check_launch("router gate (region)");
}

}  // namespace vtp
