// Region-parallel token movers used by the fused block forward: router gate, multi-grain
// pooling (with LayerNorm statistics or explicit LayerNorm rows) and replicate-unpool with
// residual.  One CTA of four warps owns one 4x4 region of the token grid, whatever grain
// the gate picked for it: warp w loads the four tokens of grid row w (each lane 16-byte
// channel chunks), so all 16 rows of the region (12 KB at C=384 bf16) are in flight at
// once, every region costs the same, and nothing depends on walking the patch list.
// Sums that span grid rows go through shared memory: each grid row is summed in token order,
// then the rows of a patch are added top to bottom (the reference adds the same tokens in one
// sequential chain; the results differ by fp32 rounding only).
//
// Replaces DynamicRouter.forward (vtpack/layers/dge.py:145-150), grained_sample_compress /
// grained_sample_decompress (vtpack/layers/csrc/grained_sample/grained_sample.cu:31-69,
// 107-144) and the nn.LayerNorm norm1 calls of Block.forward
// (vtpack/models/dge/deit_dge.py:127) on the fused path.
#include "region_ops.h"

namespace vtp {

constexpr int RG = 4;              // tokens per region side = warps per CTA

template <typename T, int MAXCH>
struct Rows4 {
    Vec<T> raw[RG][MAXCH];
    __device__ __forceinline__ void load(const T* src, int C, int lane, int nchunks) {
#pragma unroll
        for (int j = 0; j < RG; ++j)
#pragma unroll
            for (int ch = 0; ch < MAXCH; ++ch)
                if (lane + 32 * ch < nchunks) raw[j][ch].load(src + (size_t)j * C + (lane + 32 * ch) * Vec<T>::N);
    }
};

template <typename T, int MAXCH>
__device__ __forceinline__ void add_row(float (&acc)[MAXCH][Vec<T>::N], const Vec<T> (&row)[MAXCH], int lane,
                                        int nchunks) {
#pragma unroll
    for (int ch = 0; ch < MAXCH; ++ch)
        if (lane + 32 * ch < nchunks) {
            float f[Vec<T>::N];
            row[ch].to_float(f);
#pragma unroll
            for (int i = 0; i < Vec<T>::N; ++i) acc[ch][i] += f[i];
        }
}

// (mean, rstd) of one row held as fp32 values across the warp, single pass (sum, sum of
// squares): exact enough for bf16 rows, whose values carry 8 significant bits.
template <int MAXCH, int VN>
__device__ __forceinline__ float2 row_stats_1pass(const float (&f)[MAXCH][VN], int lane, int nchunks, int C,
                                                  float eps) {
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int ch = 0; ch < MAXCH; ++ch)
        if (lane + 32 * ch < nchunks)
#pragma unroll
            for (int i = 0; i < VN; ++i) { s1 += f[ch][i]; s2 = fmaf(f[ch][i], f[ch][i], s2); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    const float mean = s1 / (float)C;
    const float var = fmaxf(s2 / (float)C - mean * mean, 0.f);
    return make_float2(mean, rsqrtf(var + eps));
}

// LayerNorm of one row (two-pass) and store; w/b are read through L1.
template <typename T, int MAXCH>
__device__ __forceinline__ void ln_store(const float (&f)[MAXCH][Vec<T>::N], int lane, int nchunks, int C,
                                         const float* __restrict__ lnw, const float* __restrict__ lnb, float eps,
                                         T* __restrict__ dst) {
    constexpr int VN = Vec<T>::N;
    float s = 0.f;
#pragma unroll
    for (int ch = 0; ch < MAXCH; ++ch)
        if (lane + 32 * ch < nchunks)
#pragma unroll
            for (int i = 0; i < VN; ++i) s += f[ch][i];
    const float mean = warp_sum(s) / (float)C;
    float v = 0.f;
#pragma unroll
    for (int ch = 0; ch < MAXCH; ++ch)
        if (lane + 32 * ch < nchunks)
#pragma unroll
            for (int i = 0; i < VN; ++i) { const float d = f[ch][i] - mean; v = fmaf(d, d, v); }
    const float rstd = rsqrtf(warp_sum(v) / (float)C + eps);
#pragma unroll
    for (int ch = 0; ch < MAXCH; ++ch) {
        const int chunk = lane + 32 * ch;
        if (chunk < nchunks) {
            float o[VN];
#pragma unroll
            for (int i = 0; i < VN; ++i)
                o[i] = (f[ch][i] - mean) * rstd * __ldg(lnw + chunk * VN + i) + __ldg(lnb + chunk * VN + i);
            Vec<T> ov;
            ov.from_float(o);
            ov.store(dst + chunk * VN);
        }
    }
}

template <typename T, int MAXCH>
__device__ __forceinline__ void row_to_float(float (&f)[MAXCH][Vec<T>::N], const Vec<T> (&row)[MAXCH], int lane,
                                             int nchunks) {
#pragma unroll
    for (int ch = 0; ch < MAXCH; ++ch) {
        if (lane + 32 * ch < nchunks) row[ch].to_float(f[ch]);
        else
#pragma unroll
            for (int i = 0; i < Vec<T>::N; ++i) f[ch][i] = 0.f;
    }
}

// The value the consumer GEMM will see: the row after rounding to T.
template <typename T, int MAXCH>
__device__ __forceinline__ void round_store(float (&f)[MAXCH][Vec<T>::N], int lane, int nchunks, T* __restrict__ dst) {
#pragma unroll
    for (int ch = 0; ch < MAXCH; ++ch) {
        const int chunk = lane + 32 * ch;
        if (chunk < nchunks) {
            Vec<T> ov;
            ov.from_float(f[ch]);
            ov.store(dst + chunk * Vec<T>::N);
            ov.to_float(f[ch]);
        }
    }
}

// ------------------------------------------------------------------------------- pool
// STATS = true : comp rows + (mean, rstd) of every token row and every comp row, for the
//                GEMMs that apply LayerNorm in their epilogue; zeroes stats_acc rows.
// STATS = false: comp rows + explicit LN(x) rows and LN(comp) rows.
template <typename T, int MAXCH, bool STATS>
__global__ void __launch_bounds__(128)
pool_region_kernel(const T* __restrict__ x, RegionGeom g, const int32_t* __restrict__ idx,
                   const int32_t* __restrict__ region_first, const int32_t* __restrict__ offsets,
                   const int32_t* __restrict__ counts, int32_t* __restrict__ offsets_out,
                   int32_t* __restrict__ region_first_out, int32_t* __restrict__ counts_next, Splits sp,
                   T* __restrict__ comp, float2* __restrict__ stats_x, float2* __restrict__ stats_q,
                   float2* __restrict__ stats_acc, int write_stats_x, const float* __restrict__ lnw,
                   const float* __restrict__ lnb, float eps, T* __restrict__ xn, T* __restrict__ qn) {
    constexpr int VN = Vec<T>::N;
    extern __shared__ float part[];          // [4 grid rows][2 patch columns][C] row sums
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int nchunks = g.C / VN;
    const int R = g.Hr * g.Wr;
    const int rid = blockIdx.x;

    if (rid >= g.B * R) {
        // ---- extra (cls) tokens: one per warp, copied
        const int e = (rid - g.B * R) * RG + w;
        if (e >= g.B * g.num_extra) return;
        const int b = e / g.num_extra, t = e % g.num_extra;
        const size_t src_row = (size_t)b * g.N + t;
        int dst_row;
        if (region_first) {
            dst_row = __ldg(offsets + b) + t;
        } else {
            int part_sum = 0;
            for (int j = lane; j < b; j += 32) part_sum += __ldg(counts + j);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) part_sum += __shfl_xor_sync(0xffffffffu, part_sum, o);
            dst_row = part_sum + t;
            // start the next block's per-image count at the extra tokens; its gate adds the rest
            if (t == 0 && lane == 0 && counts_next) counts_next[b] = g.num_extra;
        }
        Vec<T> row[MAXCH];
#pragma unroll
        for (int ch = 0; ch < MAXCH; ++ch)
            if (lane + 32 * ch < nchunks) row[ch].load(x + src_row * g.C + (lane + 32 * ch) * VN);
        float f[MAXCH][VN];
        row_to_float<T, MAXCH>(f, row, lane, nchunks);
#pragma unroll
        for (int ch = 0; ch < MAXCH; ++ch)
            if (lane + 32 * ch < nchunks) row[ch].store(comp + (size_t)dst_row * g.C + (lane + 32 * ch) * VN);
        if (STATS) {
            const float2 st = row_stats_1pass<MAXCH, VN>(f, lane, nchunks, g.C, eps);
            if (lane == 0) {
                if (write_stats_x) stats_x[src_row] = st;
                stats_q[dst_row] = st;
                stats_acc[dst_row] = make_float2(0.f, 0.f);
            }
        } else {
            ln_store<T, MAXCH>(f, lane, nchunks, g.C, lnw, lnb, eps, xn + src_row * g.C);
            ln_store<T, MAXCH>(f, lane, nchunks, g.C, lnw, lnb, eps, qn + (size_t)dst_row * g.C);
        }
        return;
    }

    const int b = rid / R, rr = rid % R;
    const int ry = rr / g.Wr, rx = rr % g.Wr;
    int k = __ldg(idx + rid);
    k = min(max(k, 0), sp.n - 1);
    const int s = sp.v[k];                     // sub-patches per region side: 4, 2 or 1
    const int step = RG / s;
    const size_t tok0 = (size_t)b * g.N + g.num_extra + (size_t)(ry * RG + w) * g.W + rx * RG;

    Rows4<T, MAXCH> rows;
    rows.load(x + tok0 * g.C, g.C, lane, nchunks);

    int first;
    if (region_first) {
        first = __ldg(region_first + rid);
    } else {
        // No patch-list kernel ran: this region's first packed row = queries of the images in
        // front (per-image counts, accumulated by whoever computed the gate) + extra tokens +
        // queries of this image's earlier regions.  Every warp computes it redundantly.
        int part_sum = 0;
        for (int j = lane; j < b; j += 32) part_sum += __ldg(counts + j);
        int own = 0;
        for (int r = lane; r < rr; r += 32) {
            int kk = __ldg(idx + b * R + r);
            kk = min(max(kk, 0), sp.n - 1);
            own += sp.v[kk] * sp.v[kk];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            part_sum += __shfl_xor_sync(0xffffffffu, part_sum, o);
            own += __shfl_xor_sync(0xffffffffu, own, o);
        }
        first = part_sum + g.num_extra + own;
        if (w == 0 && lane == 0) region_first_out[rid] = first;
        if (rr == 0 && w == 0 && lane == 0) {
            offsets_out[b] = part_sum;
            if (b == g.B - 1) offsets_out[g.B] = part_sum + __ldg(counts + b);
        }
    }

    // per-token LayerNorm statistics or rows
#pragma unroll
    for (int j = 0; j < RG; ++j) {
        float f[MAXCH][VN];
        row_to_float<T, MAXCH>(f, rows.raw[j], lane, nchunks);
        if (STATS) {
            if (write_stats_x || step == 1) {
                const float2 st = row_stats_1pass<MAXCH, VN>(f, lane, nchunks, g.C, eps);
                if (lane == 0 && write_stats_x) stats_x[tok0 + j] = st;
                if (step == 1 && lane == 0) {                     // the token is its own patch
                    stats_q[first + w * RG + j] = st;
                    stats_acc[first + w * RG + j] = make_float2(0.f, 0.f);
                }
            }
        } else {
            ln_store<T, MAXCH>(f, lane, nchunks, g.C, lnw, lnb, eps, xn + (tok0 + j) * g.C);
            if (step == 1) ln_store<T, MAXCH>(f, lane, nchunks, g.C, lnw, lnb, eps, qn + (size_t)(first + w * RG + j) * g.C);
        }
    }

    if (step == 1) {
        // finest grain: mean of one token = the token
#pragma unroll
        for (int j = 0; j < RG; ++j)
#pragma unroll
            for (int ch = 0; ch < MAXCH; ++ch)
                if (lane + 32 * ch < nchunks)
                    rows.raw[j][ch].store(comp + (size_t)(first + w * RG + j) * g.C + (lane + 32 * ch) * VN);
        return;
    }

    // step 2: two patches per pair of grid rows; step 4: one patch for the region.  Every warp
    // leaves the in-order sum of its grid row's tokens (per patch column) in shared memory;
    // after one barrier the rows of a patch are added top to bottom.
    const int npx = s;                         // patch columns: 2 (step 2) or 1 (step 4)
    for (int dx = 0; dx < npx; ++dx) {
        float acc[MAXCH][VN];
#pragma unroll
        for (int ch = 0; ch < MAXCH; ++ch)
#pragma unroll
            for (int i = 0; i < VN; ++i) acc[ch][i] = 0.f;
        if (step == 2) {
            if (dx == 0) { add_row<T, MAXCH>(acc, rows.raw[0], lane, nchunks); add_row<T, MAXCH>(acc, rows.raw[1], lane, nchunks); }
            else         { add_row<T, MAXCH>(acc, rows.raw[2], lane, nchunks); add_row<T, MAXCH>(acc, rows.raw[3], lane, nchunks); }
        } else {
#pragma unroll
            for (int j = 0; j < RG; ++j) add_row<T, MAXCH>(acc, rows.raw[j], lane, nchunks);
        }
        float* slot = part + (size_t)(w * 2 + dx) * g.C;
#pragma unroll
        for (int ch = 0; ch < MAXCH; ++ch) {
            const int chunk = lane + 32 * ch;
            if (chunk < nchunks)
#pragma unroll
                for (int i = 0; i < VN; ++i) slot[chunk * VN + i] = acc[ch][i];
        }
    }
    __syncthreads();
    // step 2: warp w finishes patch (dy = w / 2, dx = w % 2); step 4: warp 0 finishes the patch
    if (step == 4 && w != 0) return;
    const int dy = (step == 2) ? (w >> 1) : 0;
    const int dx = (step == 2) ? (w & 1) : 0;
    float acc[MAXCH][VN];
#pragma unroll
    for (int ch = 0; ch < MAXCH; ++ch)
#pragma unroll
        for (int i = 0; i < VN; ++i) acc[ch][i] = 0.f;
    for (int p = 0; p < step; ++p) {
        const float* slot = part + (size_t)((dy * step + p) * 2 + dx) * g.C;
#pragma unroll
        for (int ch = 0; ch < MAXCH; ++ch) {
            const int chunk = lane + 32 * ch;
            if (chunk < nchunks)
#pragma unroll
                for (int i = 0; i < VN; ++i) acc[ch][i] += slot[chunk * VN + i];
        }
    }
    const float denom = (float)(step * step);
#pragma unroll
    for (int ch = 0; ch < MAXCH; ++ch)
#pragma unroll
        for (int i = 0; i < VN; ++i) acc[ch][i] = acc[ch][i] / denom;
    const int row = first + dy * s + dx;
    if (STATS) {
        round_store<T, MAXCH>(acc, lane, nchunks, comp + (size_t)row * g.C);
        const float2 st = row_stats_1pass<MAXCH, VN>(acc, lane, nchunks, g.C, eps);
        if (lane == 0) { stats_q[row] = st; stats_acc[row] = make_float2(0.f, 0.f); }
    } else {
        ln_store<T, MAXCH>(acc, lane, nchunks, g.C, lnw, lnb, eps, qn + (size_t)row * g.C);
        round_store<T, MAXCH>(acc, lane, nchunks, comp + (size_t)row * g.C);
    }
}

template <typename T, int MAXCH>
__device__ __forceinline__ void gate_from_row_sums(const float* part, int C, int lane, int nchunks,
                                                   const float* __restrict__ gw, const float* __restrict__ gb, int S,
                                                   float* __restrict__ logits_out, int32_t* __restrict__ idx_out,
                                                   int rid, int32_t* counts_img, const Splits& sp);

// ----------------------------------------------------------------------------- unpool
// out[b,tok] = ref[b,tok] + (q[p] - comp[p]) for the patch p that covers the token.
template <typename T, int MAXCH>
__global__ void __launch_bounds__(128)
unpool_region_kernel(const T* __restrict__ q, const T* __restrict__ comp, const T* ref, T* out, RegionGeom g,
                     const int32_t* __restrict__ idx, const int32_t* __restrict__ region_first,
                     const int32_t* __restrict__ offsets, Splits sp, NextBlock nx) {
    constexpr int VN = Vec<T>::N;
    extern __shared__ float part[];          // [4 grid rows][C] row sums of the output (next block's gate)
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int nchunks = g.C / VN;
    const int R = g.Hr * g.Wr;
    const int rid = blockIdx.x;

    if (rid >= g.B * R) {
        const int e = (rid - g.B * R) * RG + w;
        if (e >= g.B * g.num_extra) return;
        const int b = e / g.num_extra, t = e % g.num_extra;
        const size_t tok = (size_t)b * g.N + t;
        const size_t p = (size_t)(__ldg(offsets + b) + t);
        float e1 = 0.f, e2 = 0.f;
#pragma unroll
        for (int ch = 0; ch < MAXCH; ++ch) {
            const int chunk = lane + 32 * ch;
            if (chunk < nchunks) {
                Vec<T> qv, cv, rv;
                float qf[VN], cf[VN], rf[VN];
                qv.load(q + p * g.C + chunk * VN);
                cv.load(comp + p * g.C + chunk * VN);
                rv.load(ref + tok * g.C + chunk * VN);
                qv.to_float(qf); cv.to_float(cf); rv.to_float(rf);
#pragma unroll
                for (int i = 0; i < VN; ++i) rf[i] = (qf[i] - cf[i]) + rf[i];
                rv.from_float(rf);
                rv.store(out + tok * g.C + chunk * VN);
                if (nx.stats_x) {
                    rv.to_float(rf);
#pragma unroll
                    for (int i = 0; i < VN; ++i) { e1 += rf[i]; e2 = fmaf(rf[i], rf[i], e2); }
                }
            }
        }
        if (nx.stats_x) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                e1 += __shfl_xor_sync(0xffffffffu, e1, o);
                e2 += __shfl_xor_sync(0xffffffffu, e2, o);
            }
            const float mean = e1 / (float)g.C;
            if (lane == 0) nx.stats_x[tok] = make_float2(mean, rsqrtf(fmaxf(e2 / (float)g.C - mean * mean, 0.f) + nx.eps));
        }
        return;
    }
    const int b = rid / R, rr = rid % R;
    const int ry = rr / g.Wr, rx = rr % g.Wr;
    int k = __ldg(idx + rid);
    k = min(max(k, 0), sp.n - 1);
    const int s = sp.v[k];
    const int step = RG / s;
    const int first = __ldg(region_first + rid);
    const size_t tok0 = (size_t)b * g.N + g.num_extra + (size_t)(ry * RG + w) * g.W + rx * RG;
    const int prow = first + (w / step) * s;            // packed row of this grid row's first patch
    float rowsum[MAXCH][VN];                            // sum of this grid row's four output tokens
#pragma unroll
    for (int ch = 0; ch < MAXCH; ++ch)
#pragma unroll
        for (int i = 0; i < VN; ++i) rowsum[ch][i] = 0.f;

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        // two tokens per pass: their reference rows and the one or two patch rows they map to
        const int j0 = 2 * h;
        const int p0 = prow + j0 / step, p1 = prow + (j0 + 1) / step;
        float s1a = 0.f, s2a = 0.f, s1b = 0.f, s2b = 0.f;
        Vec<T> r0[MAXCH], r1[MAXCH], q0[MAXCH], c0[MAXCH], q1[MAXCH], c1[MAXCH];
#pragma unroll
        for (int ch = 0; ch < MAXCH; ++ch) {
            const int chunk = lane + 32 * ch;
            if (chunk < nchunks) {
                r0[ch].load(ref + (tok0 + j0) * g.C + chunk * VN);
                r1[ch].load(ref + (tok0 + j0 + 1) * g.C + chunk * VN);
                q0[ch].load(q + (size_t)p0 * g.C + chunk * VN);
                c0[ch].load(comp + (size_t)p0 * g.C + chunk * VN);
                if (p1 != p0) {
                    q1[ch].load(q + (size_t)p1 * g.C + chunk * VN);
                    c1[ch].load(comp + (size_t)p1 * g.C + chunk * VN);
                }
            }
        }
#pragma unroll
        for (int ch = 0; ch < MAXCH; ++ch) {
            const int chunk = lane + 32 * ch;
            if (chunk < nchunks) {
                float d0[VN], d1[VN], t[VN], a[VN];
                q0[ch].to_float(d0); c0[ch].to_float(t);
#pragma unroll
                for (int i = 0; i < VN; ++i) d0[i] -= t[i];
                if (p1 != p0) {
                    q1[ch].to_float(d1); c1[ch].to_float(t);
#pragma unroll
                    for (int i = 0; i < VN; ++i) d1[i] -= t[i];
                } else {
#pragma unroll
                    for (int i = 0; i < VN; ++i) d1[i] = d0[i];
                }
                r0[ch].to_float(a);
#pragma unroll
                for (int i = 0; i < VN; ++i) a[i] = d0[i] + a[i];
                Vec<T> o;
                o.from_float(a);
                o.store(out + (tok0 + j0) * g.C + chunk * VN);
                if (nx.stats_x) {
                    o.to_float(a);                      // the rounded values the next block will read
#pragma unroll
                    for (int i = 0; i < VN; ++i) { s1a += a[i]; s2a = fmaf(a[i], a[i], s2a); rowsum[ch][i] += a[i]; }
                }
                r1[ch].to_float(a);
#pragma unroll
                for (int i = 0; i < VN; ++i) a[i] = d1[i] + a[i];
                o.from_float(a);
                o.store(out + (tok0 + j0 + 1) * g.C + chunk * VN);
                if (nx.stats_x) {
                    o.to_float(a);
#pragma unroll
                    for (int i = 0; i < VN; ++i) { s1b += a[i]; s2b = fmaf(a[i], a[i], s2b); rowsum[ch][i] += a[i]; }
                }
            }
        }
        if (nx.stats_x) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                s1a += __shfl_xor_sync(0xffffffffu, s1a, o);
                s2a += __shfl_xor_sync(0xffffffffu, s2a, o);
                s1b += __shfl_xor_sync(0xffffffffu, s1b, o);
                s2b += __shfl_xor_sync(0xffffffffu, s2b, o);
            }
            if (lane < 2) {
                const float e1 = lane == 0 ? s1a : s1b, e2 = lane == 0 ? s2a : s2b;
                const float mean = e1 / (float)g.C;
                nx.stats_x[tok0 + j0 + lane] = make_float2(mean, rsqrtf(fmaxf(e2 / (float)g.C - mean * mean, 0.f) + nx.eps));
            }
        }
    }
    if (!nx.gw) return;
    // ---- the next block's router gate on the region this CTA has just written
#pragma unroll
    for (int ch = 0; ch < MAXCH; ++ch) {
        const int chunk = lane + 32 * ch;
        if (chunk < nchunks)
#pragma unroll
            for (int i = 0; i < VN; ++i) part[(size_t)w * g.C + chunk * VN + i] = rowsum[ch][i];
    }
    __syncthreads();
    if (w != 0) return;
    gate_from_row_sums<T, MAXCH>(part, g.C, lane, nchunks, nx.gw, nx.gb, nx.S, nx.logits, nx.idx, rid,
                                 nx.counts ? nx.counts + b : nullptr, sp);
}

// ------------------------------------------------------------------------ router gate
// Region mean of the raw tokens (each grid row summed in order, rows added top to bottom,
// then / 16), n_splits fp32 dot products, argmax with the lowest index winning ties.
// `part` holds the four grid-row sums [4][C]; executed by one warp.
template <typename T, int MAXCH>
__device__ __forceinline__ void gate_from_row_sums(const float* part, int C, int lane, int nchunks,
                                                   const float* __restrict__ gw, const float* __restrict__ gb, int S,
                                                   float* __restrict__ logits_out, int32_t* __restrict__ idx_out,
                                                   int rid, int32_t* counts_img, const Splits& sp) {
    constexpr int VN = Vec<T>::N;
    float acc[MAXCH][VN];
#pragma unroll
    for (int ch = 0; ch < MAXCH; ++ch)
#pragma unroll
        for (int i = 0; i < VN; ++i) acc[ch][i] = 0.f;
    for (int p = 0; p < RG; ++p) {
#pragma unroll
        for (int ch = 0; ch < MAXCH; ++ch) {
            const int chunk = lane + 32 * ch;
            if (chunk < nchunks)
#pragma unroll
                for (int i = 0; i < VN; ++i) acc[ch][i] += part[(size_t)p * C + chunk * VN + i];
        }
    }
    const float denom = (float)(RG * RG);
    float best = 0.f;
    int best_i = 0;
    for (int sI = 0; sI < S; ++sI) {
        float pdot = 0.f;
#pragma unroll
        for (int ch = 0; ch < MAXCH; ++ch) {
            const int chunk = lane + 32 * ch;
            if (chunk < nchunks) {
                const float4* wp = reinterpret_cast<const float4*>(gw + (size_t)sI * C + chunk * VN);
#pragma unroll
                for (int i4 = 0; i4 < VN / 4; ++i4) {
                    const float4 w4 = __ldg(wp + i4);
                    pdot = fmaf(acc[ch][4 * i4 + 0] / denom, w4.x, pdot);
                    pdot = fmaf(acc[ch][4 * i4 + 1] / denom, w4.y, pdot);
                    pdot = fmaf(acc[ch][4 * i4 + 2] / denom, w4.z, pdot);
                    pdot = fmaf(acc[ch][4 * i4 + 3] / denom, w4.w, pdot);
                }
            }
        }
        pdot = warp_sum(pdot) + __ldg(gb + sI);
        if (lane == 0 && logits_out) logits_out[(size_t)rid * S + sI] = pdot;
        if (sI == 0 || pdot > best) { best = pdot; best_i = sI; }
    }
    if (lane == 0) {
        idx_out[rid] = best_i;
        // queries this region contributes to its image (the image's slot starts at num_extra)
        if (counts_img) atomicAdd(counts_img, sp.v[min(best_i, sp.n - 1)] * sp.v[min(best_i, sp.n - 1)]);
    }
}

// Stand-alone gate (first block of a model, or a block called on its own); optionally also
// writes the LayerNorm statistics of every token row it reads.
template <typename T, int MAXCH>
__global__ void __launch_bounds__(128)
gate_region_kernel(const T* __restrict__ x, RegionGeom g, const float* __restrict__ gw,
                   const float* __restrict__ gb, int S, float* __restrict__ logits_out,
                   int32_t* __restrict__ idx_out, float2* __restrict__ stats_x, float eps) {
    constexpr int VN = Vec<T>::N;
    extern __shared__ float part[];          // [4][C]
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int nchunks = g.C / VN;
    const int R = g.Hr * g.Wr;
    const int rid = blockIdx.x;
    if (rid >= g.B * R) {
        // extra (cls) tokens only matter for the statistics
        const int e = (rid - g.B * R) * RG + w;
        if (!stats_x || e >= g.B * g.num_extra) return;
        const size_t tok = (size_t)(e / g.num_extra) * g.N + e % g.num_extra;
        Vec<T> row[MAXCH];
#pragma unroll
        for (int ch = 0; ch < MAXCH; ++ch)
            if (lane + 32 * ch < nchunks) row[ch].load(x + tok * g.C + (lane + 32 * ch) * VN);
        float f[MAXCH][VN];
        row_to_float<T, MAXCH>(f, row, lane, nchunks);
        const float2 st = row_stats_1pass<MAXCH, VN>(f, lane, nchunks, g.C, eps);
        if (lane == 0) stats_x[tok] = st;
        return;
    }
    const int b = rid / R, rr = rid % R;
    const int ry = rr / g.Wr, rx = rr % g.Wr;
    const size_t tok0 = (size_t)b * g.N + g.num_extra + (size_t)(ry * RG + w) * g.W + rx * RG;
    Rows4<T, MAXCH> rows;
    rows.load(x + tok0 * g.C, g.C, lane, nchunks);
    float acc[MAXCH][VN];
#pragma unroll
    for (int ch = 0; ch < MAXCH; ++ch)
#pragma unroll
        for (int i = 0; i < VN; ++i) acc[ch][i] = 0.f;
#pragma unroll
    for (int j = 0; j < RG; ++j) {
        add_row<T, MAXCH>(acc, rows.raw[j], lane, nchunks);
        if (stats_x) {
            float f[MAXCH][VN];
            row_to_float<T, MAXCH>(f, rows.raw[j], lane, nchunks);
            const float2 st = row_stats_1pass<MAXCH, VN>(f, lane, nchunks, g.C, eps);
            if (lane == 0) stats_x[tok0 + j] = st;
        }
    }
#pragma unroll
    for (int ch = 0; ch < MAXCH; ++ch) {
        const int chunk = lane + 32 * ch;
        if (chunk < nchunks)
#pragma unroll
            for (int i = 0; i < VN; ++i) part[(size_t)w * g.C + chunk * VN + i] = acc[ch][i];
    }
    __syncthreads();
    if (w != 0) return;
    Splits none;
    none.n = 1; none.v[0] = 0;
    gate_from_row_sums<T, MAXCH>(part, g.C, lane, nchunks, gw, gb, S, logits_out, idx_out, rid, nullptr, none);
}

// ------------------------------------------------------------------------------- host

template <typename T, int MAXCH>
static void launch_pool_t(const RegionPoolArgs& a, cudaStream_t st) {
    const int R = a.g.Hr * a.g.Wr;
    const int grid = a.g.B * R + ceil_div(a.g.B * a.g.num_extra, RG);
    const size_t smem = (size_t)8 * a.g.C * sizeof(float);
    if (a.stats_q)
        pool_region_kernel<T, MAXCH, true><<<grid, 128, smem, st>>>(
            (const T*)a.x, a.g, a.idx, a.region_first, a.offsets, a.counts, a.offsets_out, a.region_first_out, a.counts_next, a.sp,
            (T*)a.comp, a.stats_x, a.stats_q, a.stats_acc, a.stats_x_ready ? 0 : 1, nullptr, nullptr, a.eps, nullptr,
            nullptr);
    else
        pool_region_kernel<T, MAXCH, false><<<grid, 128, smem, st>>>(
            (const T*)a.x, a.g, a.idx, a.region_first, a.offsets, a.counts, a.offsets_out, a.region_first_out, a.counts_next, a.sp,
            (T*)a.comp, nullptr, nullptr, nullptr, 0, a.lnw, a.lnb, a.eps, (T*)a.xn, (T*)a.qn);
}

template <typename T, int MAXCH>
static void launch_unpool_t(const RegionUnpoolArgs& a, cudaStream_t st) {
    const int R = a.g.Hr * a.g.Wr;
    const int grid = a.g.B * R + ceil_div(a.g.B * a.g.num_extra, RG);
    unpool_region_kernel<T, MAXCH><<<grid, 128, (size_t)4 * a.g.C * sizeof(float), st>>>(
        (const T*)a.q, (const T*)a.comp, (const T*)a.ref, (T*)a.out, a.g, a.idx, a.region_first, a.offsets, a.sp, a.next);
}

template <typename T, int MAXCH>
static void launch_gate_t(const RegionGateArgs& a, cudaStream_t st) {
    const int R = a.g.Hr * a.g.Wr;
    const int grid = a.g.B * R + (a.stats_x ? ceil_div(a.g.B * a.g.num_extra, RG) : 0);
    gate_region_kernel<T, MAXCH><<<grid, 128, (size_t)4 * a.g.C * sizeof(float), st>>>(
        (const T*)a.x, a.g, a.gw, a.gb, a.S, a.logits_out, a.idx_out, a.stats_x, a.eps);
}

#define VTP_DISPATCH_MAXCH(FN, T, ARGS, ST)                      \
    do {                                                         \
        const int maxch = ceil_div((ARGS).g.C / Vec<T>::N, 32);  \
        if (maxch <= 1) FN<T, 1>(ARGS, ST);                      \
        else if (maxch == 2) FN<T, 2>(ARGS, ST);                 \
        else if (maxch == 3) FN<T, 3>(ARGS, ST);                 \
        else if (maxch == 4) FN<T, 4>(ARGS, ST);                 \
        else if (maxch <= 6) FN<T, 6>(ARGS, ST);                 \
        else return fail(VTP_ERR_SHAPE, "C=%d too large", (ARGS).g.C); \
    } while (0)

bool region_ops_supported(const RegionGeom& g, int dtype) {
    const int vn = dtype == VTP_BF16 ? 8 : 4;
    return g.region == RG && g.C % vn == 0 && g.C / vn <= 192 && g.B > 0 && g.Hr > 0 && g.Wr > 0;
}

int region_pool(const RegionPoolArgs& a, int dtype, cudaStream_t st) {
    if (dtype == VTP_F32) VTP_DISPATCH_MAXCH(launch_pool_t, float, a, st);
    else VTP_DISPATCH_MAXCH(launch_pool_t, bf16, a, st);
    return check_launch("pool (region)");
}

int region_unpool(const RegionUnpoolArgs& a, int dtype, cudaStream_t st) {
    if (dtype == VTP_F32) VTP_DISPATCH_MAXCH(launch_unpool_t, float, a, st);
    else VTP_DISPATCH_MAXCH(launch_unpool_t, bf16, a, st);
    return check_launch("unpool (region)");
}

int region_gate(const RegionGateArgs& a, int dtype, cudaStream_t st) {
    if (dtype == VTP_F32) VTP_DISPATCH_MAXCH(launch_gate_t, float, a, st);
    else VTP_DISPATCH_MAXCH(launch_gate_t, bf16, a, st);
    return check_launch("router gate (region)");
}

}  // namespace vtp
