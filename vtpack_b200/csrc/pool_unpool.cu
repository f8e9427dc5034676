// HBM-bound token movers: multi-grain pooling (+ fused LayerNorms), replicate-unpool with
// residual, and a stand-alone LayerNorm.  One warp owns one packed query row (pool/unpool)
// or one token row (LayerNorm); lanes stride over 16-byte channel chunks so every global
// access is a full, coalesced 16-byte vector.
//
// Replaces grained_sample_compress / grained_sample_decompress
// (vtpack/layers/csrc/grained_sample/grained_sample.cu:31-69, 71-144) and the nn.LayerNorm
// calls of Block.forward (vtpack/models/dge/deit_dge.py:127-128).
#include "common.cuh"
#include "region_ops.h"
#include "runtime.h"

namespace vtp {

// True when every token a patch row [b, y, x, step] names lies inside the declared [B, N] token array
// (N = num_extra + H*W); extra-token rows are [b, -idx-1, *, 1].
__device__ __forceinline__ bool patch_in_range(const int4& pt, int B, int N, int W, int num_extra) {
#if VTP_INDEX_GUARDS
    if ((unsigned)pt.x >= (unsigned)B) return false;
    if (pt.y < 0) return -(long long)pt.y - 1 < (long long)num_extra;
    const int H = (N - num_extra) / W;
    return pt.w >= 1 && pt.w <= H && pt.y <= H - pt.w && pt.z >= 0 && pt.w <= W && pt.z <= W - pt.w;
#else
    return true;
#endif
}
__device__ __forceinline__ void flag_bad_index(int* status) {
    if (status) atomicOr(status, STATUS_BAD_INDEX);
}

template <typename T, int MAXCH>
struct RowRegs {
    static constexpr int VN = Vec<T>::N;
    float f[MAXCH][VN];
};

// LayerNorm of one row held across the warp (two-pass: mean, then centred variance).
template <typename T, int MAXCH>
__device__ __forceinline__ void ln_row_store(const float (&f)[MAXCH][Vec<T>::N], int lane,
                                             int nchunks, int C, const float (&w)[MAXCH][Vec<T>::N],
                                             const float (&bb)[MAXCH][Vec<T>::N], float eps,
                                             T* __restrict__ dst, const T* __restrict__ add_row = nullptr) {
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
            for (int i = 0; i < VN; ++i) o[i] = (f[ch][i] - mean) * rstd * w[ch][i] + bb[ch][i];
            if (add_row) {
                Vec<T> av;
                float af[VN];
                av.load(add_row + chunk * VN);
                av.to_float(af);
#pragma unroll
                for (int i = 0; i < VN; ++i) o[i] += af[i];
            }
            Vec<T> ov;
            ov.from_float(o);
            ov.store(dst + chunk * VN);
        }
    }
}

template <typename T, int MAXCH>
__device__ __forceinline__ void load_vecs(float (&dst)[MAXCH][Vec<T>::N], const float* __restrict__ src,
                                          int lane, int nchunks) {
    constexpr int VN = Vec<T>::N;
#pragma unroll
    for (int ch = 0; ch < MAXCH; ++ch) {
        const int chunk = lane + 32 * ch;
#pragma unroll
        for (int i = 0; i < VN; ++i) dst[ch][i] = (chunk < nchunks) ? __ldg(src + chunk * VN + i) : 0.f;
    }
}

// ------------------------------------------------------------------------------- pool
// comp[p] = mean of the patch's tokens (sum in (dy,dx) order, then divide; mean = 0 keeps the
// sum, which is the gradient of the replicate-unpool with respect to its packed rows);  optionally
// xn[b,tok] = LN(x[b,tok]) for every token read and qn[p] = LN(comp[p]).  Every token
// belongs to exactly one patch, so x is read once.
// Algorithmic bytes: (B*N + L)*C*e  (+ (B*N + L)*C*e when the LayerNorm outputs are on).
// Three blocks per SM (85 registers instead of 106): the kernel waits on its row loads, and the sum
// form measured 40 us instead of 50 us at DeiT-S batch 256; four blocks were no better.
template <typename T, int MAXCH, bool WITH_LN>
__global__ void __launch_bounds__(256, 3)
pool_kernel(const T* __restrict__ x, int B, int N, int C, int W, int num_extra,
            const int4* __restrict__ patches, const int32_t* __restrict__ n_dev, int n_max,
            T* __restrict__ comp, const float* __restrict__ lnw, const float* __restrict__ lnb,
            float eps, T* __restrict__ xn, T* __restrict__ qn, int mean, int* status) {
    constexpr int VN = Vec<T>::N;
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int nchunks = C / VN;
    int L = n_max;
    if (n_dev) L = min(__ldg(n_dev), n_max);

    float w[MAXCH][VN], bb[MAXCH][VN];
    if (WITH_LN) {
        load_vecs<T, MAXCH>(w, lnw, lane, nchunks);
        load_vecs<T, MAXCH>(bb, lnb, lane, nchunks);
    }

    for (int p = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; p < L; p += warps) {
        const int4 pt = __ldg(patches + p);
        if (!patch_in_range(pt, B, N, W, num_extra)) {      // skip the row, leave a mark for the host
            if (lane == 0) flag_bad_index(status);
            continue;
        }
        const bool extra = pt.y < 0;
        const int step = extra ? 1 : pt.w;
        const int tok0 = extra ? (-pt.y - 1) : (num_extra + pt.y * W + pt.z);
        const size_t row0 = (size_t)pt.x * N + tok0;

        float sum[MAXCH][VN];
#pragma unroll
        for (int ch = 0; ch < MAXCH; ++ch)
#pragma unroll
            for (int i = 0; i < VN; ++i) sum[ch][i] = 0.f;

        for (int dy = 0; dy < step; ++dy) {
            for (int dx0 = 0; dx0 < step; dx0 += 4) {
                // up to four rows in flight before any arithmetic
                Vec<T> raw[4][MAXCH];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (dx0 + j < step) {
                        const T* src = x + (row0 + (size_t)dy * W + dx0 + j) * C;
#pragma unroll
                        for (int ch = 0; ch < MAXCH; ++ch)
                            if (lane + 32 * ch < nchunks) raw[j][ch].load(src + (lane + 32 * ch) * VN);
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (dx0 + j < step) {
                        float f[MAXCH][VN];
#pragma unroll
                        for (int ch = 0; ch < MAXCH; ++ch) {
                            if (lane + 32 * ch < nchunks) raw[j][ch].to_float(f[ch]);
                            else
#pragma unroll
                                for (int i = 0; i < VN; ++i) f[ch][i] = 0.f;
#pragma unroll
                            for (int i = 0; i < VN; ++i) sum[ch][i] += f[ch][i];
                        }
                        if (WITH_LN && xn)
                            ln_row_store<T, MAXCH>(f, lane, nchunks, C, w, bb, eps,
                                                   xn + (row0 + (size_t)dy * W + dx0 + j) * C);
                    }
                }
            }
        }
        const float denom = mean ? (float)(step * step) : 1.0f;   // 1: the plain sum (gradient of the unpool)
#pragma unroll
        for (int ch = 0; ch < MAXCH; ++ch) {
            const int chunk = lane + 32 * ch;
#pragma unroll
            for (int i = 0; i < VN; ++i) sum[ch][i] = sum[ch][i] / denom;
            if (chunk < nchunks) {
                Vec<T> ov;
                ov.from_float(sum[ch]);
                ov.store(comp + (size_t)p * C + chunk * VN);
            }
        }
        if (WITH_LN && qn) ln_row_store<T, MAXCH>(sum, lane, nchunks, C, w, bb, eps, qn + (size_t)p * C);
    }
}

// ----------------------------------------------------------------------------- unpool
// out[b,tok] = (q[p] - comp[p]) + ref[b,tok] for every token of patch p; inv_area = 1 scales the
// replicated row by 1/step^2 (the gradient of the mean pooling with respect to its tokens).
// Algorithmic bytes: (2*B*N + L)*C*e (+ L*C*e for comp).
template <typename T, int MAXCH>
__global__ void __launch_bounds__(256)
unpool_kernel(const T* __restrict__ q, const T* __restrict__ comp, int B, int N, int C, int W,
              int num_extra, const int4* __restrict__ patches, const int32_t* __restrict__ n_dev,
              int n_max, const T* ref, T* out, int inv_area, int* status) {
    constexpr int VN = Vec<T>::N;
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int nchunks = C / VN;
    int L = n_max;
    if (n_dev) L = min(__ldg(n_dev), n_max);

    for (int p = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; p < L; p += warps) {
        const int4 pt = __ldg(patches + p);
        if (!patch_in_range(pt, B, N, W, num_extra)) {      // skip the row, leave a mark for the host
            if (lane == 0) flag_bad_index(status);
            continue;
        }
        const bool extra = pt.y < 0;
        const int step = extra ? 1 : pt.w;
        const int tok0 = extra ? (-pt.y - 1) : (num_extra + pt.y * W + pt.z);
        const size_t row0 = (size_t)pt.x * N + tok0;

        float d[MAXCH][VN];
#pragma unroll
        for (int ch = 0; ch < MAXCH; ++ch) {
            const int chunk = lane + 32 * ch;
            if (chunk < nchunks) {
                Vec<T> qv;
                qv.load(q + (size_t)p * C + chunk * VN);
                qv.to_float(d[ch]);
                if (comp) {
                    Vec<T> cv;
                    float c[VN];
                    cv.load(comp + (size_t)p * C + chunk * VN);
                    cv.to_float(c);
#pragma unroll
                    for (int i = 0; i < VN; ++i) d[ch][i] -= c[i];
                }
                if (inv_area) {
                    // gradient of the mean pooling: every token of the patch receives 1/step^2 of the row
                    const float sc = 1.0f / (float)(step * step);
#pragma unroll
                    for (int i = 0; i < VN; ++i) d[ch][i] *= sc;
                }
            }
        }
        for (int dy = 0; dy < step; ++dy) {
            for (int dx0 = 0; dx0 < step; dx0 += 4) {
                Vec<T> raw[4][MAXCH];
                if (ref) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (dx0 + j < step) {
                            const T* src = ref + (row0 + (size_t)dy * W + dx0 + j) * C;
#pragma unroll
                            for (int ch = 0; ch < MAXCH; ++ch)
                                if (lane + 32 * ch < nchunks) raw[j][ch].load(src + (lane + 32 * ch) * VN);
                        }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (dx0 + j < step) {
                        T* dst = out + (row0 + (size_t)dy * W + dx0 + j) * C;
#pragma unroll
                        for (int ch = 0; ch < MAXCH; ++ch) {
                            const int chunk = lane + 32 * ch;
                            if (chunk < nchunks) {
                                float o[VN];
                                if (ref) {
                                    raw[j][ch].to_float(o);
#pragma unroll
                                    for (int i = 0; i < VN; ++i) o[i] = d[ch][i] + o[i];
                                } else {
#pragma unroll
                                    for (int i = 0; i < VN; ++i) o[i] = d[ch][i];
                                }
                                Vec<T> ov;
                                ov.from_float(o);
                                ov.store(dst + chunk * VN);
                            }
                        }
                    }
            }
        }
    }
}

// ------------------------------------------------- any channel count (one thread per element)
// The vector kernels above need rows of whole 16-byte chunks.  Training also pools narrow
// tensors (the per-token gate value, one channel: vtpack/layers/dge.py:104-110); those rows
// take the element-wise form of the same arithmetic, one thread per (packed row, channel) as in
// grained_sample.cu:31-69 and :107-144.
template <typename T>
__global__ void __launch_bounds__(256)
pool_any_c_kernel(const T* __restrict__ x, int B, int N, int C, int W, int num_extra,
                  const int4* __restrict__ patches, const int32_t* __restrict__ n_dev, int n_max,
                  T* __restrict__ comp, int mean, int* status) {
    int L = n_max;
    if (n_dev) L = min(__ldg(n_dev), n_max);
    const long long total = (long long)L * C;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (long long)gridDim.x * blockDim.x) {
        const int p = (int)(e / C), c = (int)(e % C);
        const int4 pt = __ldg(patches + p);
        if (!patch_in_range(pt, B, N, W, num_extra)) {      // skip the row, leave a mark for the host
            if (c == 0) flag_bad_index(status);
            continue;
        }
        const bool extra = pt.y < 0;
        const int step = extra ? 1 : pt.w;
        const int tok0 = extra ? (-pt.y - 1) : (num_extra + pt.y * W + pt.z);
        const size_t row0 = (size_t)pt.x * N + tok0;
        float sum = 0.f;
        for (int dy = 0; dy < step; ++dy)
            for (int dx = 0; dx < step; ++dx) sum += to_f32(x[(row0 + (size_t)dy * W + dx) * C + c]);
        if (mean) sum = sum / (float)(step * step);
        comp[e] = from_f32<T>(sum);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
unpool_any_c_kernel(const T* __restrict__ q, const T* __restrict__ comp, int B, int N, int C, int W, int num_extra,
                    const int4* __restrict__ patches, const int32_t* __restrict__ n_dev, int n_max,
                    const T* ref, T* out, int inv_area, int* status) {
    int L = n_max;
    if (n_dev) L = min(__ldg(n_dev), n_max);
    const long long total = (long long)L * C;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (long long)gridDim.x * blockDim.x) {
        const int p = (int)(e / C), c = (int)(e % C);
        const int4 pt = __ldg(patches + p);
        if (!patch_in_range(pt, B, N, W, num_extra)) {      // skip the row, leave a mark for the host
            if (c == 0) flag_bad_index(status);
            continue;
        }
        const bool extra = pt.y < 0;
        const int step = extra ? 1 : pt.w;
        const int tok0 = extra ? (-pt.y - 1) : (num_extra + pt.y * W + pt.z);
        const size_t row0 = (size_t)pt.x * N + tok0;
        float d = to_f32(q[e]);
        if (comp) d -= to_f32(comp[e]);
        if (inv_area) d *= 1.0f / (float)(step * step);
        for (int dy = 0; dy < step; ++dy)
            for (int dx = 0; dx < step; ++dx) {
                const size_t o = (row0 + (size_t)dy * W + dx) * C + c;
                out[o] = from_f32<T>(ref ? d + to_f32(ref[o]) : d);
            }
    }
}

static int elem_grid(long long elems) {
    const long long want = (elems + 255) / 256;
    const long long cap = (long long)sm_count() * 8;
    return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

// -------------------------------------------------------------------------- layernorm
// Optional second half of a LayerNorm launch: y[orow(r)] = LN(x[r]) + addend[r % a_mod + a_off] with
// orow(r) = (r / out_grp) * out_stride + out_off + r % out_grp (a stage's position-embedding add, written
// behind a cls slot when there is one).  addend == null: dense output rows, nothing added.
struct RowAdd {
    const void* addend = nullptr;
    int a_mod = 1, a_off = 0, out_grp = 1, out_stride = 1, out_off = 0;
};

template <typename T, int MAXCH>
__global__ void __launch_bounds__(256)
layernorm_kernel(const T* __restrict__ x, int rows_max, const int32_t* __restrict__ rows_dev, int C,
                 long long in_stride, const float* __restrict__ lnw, const float* __restrict__ lnb,
                 float eps, T* __restrict__ y, RowAdd add) {
    constexpr int VN = Vec<T>::N;
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int nchunks = C / VN;
    int rows = rows_max;
    if (rows_dev) rows = min(__ldg(rows_dev), rows_max);
    float w[MAXCH][VN], bb[MAXCH][VN];
    load_vecs<T, MAXCH>(w, lnw, lane, nchunks);
    load_vecs<T, MAXCH>(bb, lnb, lane, nchunks);
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        float f[MAXCH][VN];
#pragma unroll
        for (int ch = 0; ch < MAXCH; ++ch) {
            const int chunk = lane + 32 * ch;
            if (chunk < nchunks) {
                Vec<T> v;
                v.load(x + (size_t)r * in_stride + chunk * VN);
                v.to_float(f[ch]);
            } else {
#pragma unroll
                for (int i = 0; i < VN; ++i) f[ch][i] = 0.f;
            }
        }
        if (add.addend) {
            const size_t orow = (size_t)(r / add.out_grp) * add.out_stride + add.out_off + r % add.out_grp;
            ln_row_store<T, MAXCH>(f, lane, nchunks, C, w, bb, eps, y + orow * C,
                                   static_cast<const T*>(add.addend) + ((size_t)(r % add.a_mod) + add.a_off) * C);
        } else {
            ln_row_store<T, MAXCH>(f, lane, nchunks, C, w, bb, eps, y + (size_t)r * C);
        }
    }
}

// Rows of at most 16 chunks of 16 bytes (C <= 128 in bf16, 64 in fp32): G = 8 or 16 lanes share a row and a
// warp normalises 32 / G rows at a time; with a warp per row three quarters of its lanes would have nothing to
// load.  Same two-pass arithmetic as ln_row_store.
template <typename T, int G>
__global__ void __launch_bounds__(256)
layernorm_narrow_kernel(const T* __restrict__ x, int rows_max, const int32_t* __restrict__ rows_dev, int C,
                        long long in_stride, const float* __restrict__ lnw, const float* __restrict__ lnb,
                        float eps, T* __restrict__ y, RowAdd add) {
    constexpr int VN = Vec<T>::N, RPW = 32 / G;
    const int lane = threadIdx.x & 31, sub = lane % G, grp = lane / G;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int nchunks = C / VN;
    const bool has = sub < nchunks;
    int rows = rows_max;
    if (rows_dev) rows = min(__ldg(rows_dev), rows_max);
    float w[VN], bb[VN];
#pragma unroll
    for (int i = 0; i < VN; ++i) {
        w[i] = has ? __ldg(lnw + sub * VN + i) : 0.f;
        bb[i] = has ? __ldg(lnb + sub * VN + i) : 0.f;
    }
    // (every lane of a warp goes round the loop the same number of times: the shuffles name the whole warp)
    for (int r0 = ((blockIdx.x * blockDim.x + threadIdx.x) >> 5) * RPW; r0 < rows; r0 += warps * RPW) {
        const int r = r0 + grp;
        const bool live = has && r < rows;
        float f[VN];
#pragma unroll
        for (int i = 0; i < VN; ++i) f[i] = 0.f;
        if (live) {
            Vec<T> v;
            v.load(x + (size_t)r * in_stride + sub * VN);
            v.to_float(f);
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < VN; ++i) s += f[i];
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float mean = s / (float)C;
        float v2 = 0.f;
        if (has) {
#pragma unroll
            for (int i = 0; i < VN; ++i) { const float d = f[i] - mean; v2 = fmaf(d, d, v2); }
        }
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) v2 += __shfl_xor_sync(0xffffffffu, v2, o);
        const float rstd = rsqrtf(v2 / (float)C + eps);
        if (live) {
            float o[VN];
#pragma unroll
            for (int i = 0; i < VN; ++i) o[i] = (f[i] - mean) * rstd * w[i] + bb[i];
            size_t orow = (size_t)r;
            if (add.addend) {
                Vec<T> av;
                float af[VN];
                av.load(static_cast<const T*>(add.addend) + ((size_t)(r % add.a_mod) + add.a_off) * C + sub * VN);
                av.to_float(af);
#pragma unroll
                for (int i = 0; i < VN; ++i) o[i] += af[i];
                orow = (size_t)(r / add.out_grp) * add.out_stride + add.out_off + r % add.out_grp;
            }
            Vec<T> ov;
            ov.from_float(o);
            ov.store(y + orow * C + sub * VN);
        }
    }
}

static int row_grid(int rows) {
    const int per_block = 8;   // warps per 256-thread block
    const int want = ceil_div(rows, per_block);
    const int cap = sm_count() * 8;
    return want < 1 ? 1 : (want < cap ? want : cap);
}

template <typename T>
static int launch_pool(const void* x, int B, int N, int C, int W, int num_extra, const int32_t* patches,
                       const int32_t* n_dev, int n_max, void* comp, const float* lnw,
                       const float* lnb, float eps, void* xn, void* qn, int mean, cudaStream_t st) {
    if (C % Vec<T>::N != 0) {
        if (lnw) return fail(VTP_ERR_SHAPE, "pool: fused LayerNorm needs C=%d in whole 16-byte chunks", C);
        pool_any_c_kernel<T><<<elem_grid((long long)n_max * C), 256, 0, st>>>(
            (const T*)x, B, N, C, W, num_extra, (const int4*)patches, n_dev, n_max, (T*)comp, mean, device_status_ptr());
        return check_launch("pool");
    }
    const int maxch = ceil_div(C / Vec<T>::N, 32);
    const int grid = row_grid(n_max);
    const bool ln = lnw != nullptr;
#define VTP_POOL(M)                                                                                  \
    do {                                                                                             \
        if (ln)                                                                                      \
            pool_kernel<T, M, true><<<grid, 256, 0, st>>>(                                           \
                (const T*)x, B, N, C, W, num_extra, (const int4*)patches, n_dev, n_max, (T*)comp, lnw,  \
                lnb, eps, (T*)xn, (T*)qn, mean, device_status_ptr());                                \
        else                                                                                         \
            pool_kernel<T, M, false><<<grid, 256, 0, st>>>(                                          \
                (const T*)x, B, N, C, W, num_extra, (const int4*)patches, n_dev, n_max, (T*)comp,    \
                nullptr, nullptr, eps, nullptr, nullptr, mean, device_status_ptr());                 \
    } while (0)
    if (maxch <= 1) VTP_POOL(1);
    else if (maxch == 2) VTP_POOL(2);
    else if (maxch == 3) VTP_POOL(3);
    else if (maxch == 4) VTP_POOL(4);
    else if (maxch <= 6) VTP_POOL(6);
    else return fail(VTP_ERR_SHAPE, "pool: C=%d too large", C);
#undef VTP_POOL
    return check_launch("pool");
}

template <typename T>
static int launch_unpool(const void* q, const void* comp, int B, int N, int C, int W, int num_extra,
                         const int32_t* patches, const int32_t* n_dev, int n_max, const void* ref,
                         void* out, int inv_area, cudaStream_t st) {
    if (C % Vec<T>::N != 0) {
        unpool_any_c_kernel<T><<<elem_grid((long long)n_max * C), 256, 0, st>>>(
            (const T*)q, (const T*)comp, B, N, C, W, num_extra, (const int4*)patches, n_dev, n_max, (const T*)ref,
            (T*)out, inv_area, device_status_ptr());
        return check_launch("unpool_add");
    }
    const int maxch = ceil_div(C / Vec<T>::N, 32);
    const int grid = row_grid(n_max);
#define VTP_UNPOOL(M)                                                                           \
    unpool_kernel<T, M><<<grid, 256, 0, st>>>((const T*)q, (const T*)comp, B, N, C, W, num_extra,  \
                                              (const int4*)patches, n_dev, n_max, (const T*)ref,      \
                                              (T*)out, inv_area, device_status_ptr())
    if (maxch <= 1) VTP_UNPOOL(1);
    else if (maxch == 2) VTP_UNPOOL(2);
    else if (maxch == 3) VTP_UNPOOL(3);
    else if (maxch == 4) VTP_UNPOOL(4);
    else if (maxch <= 6) VTP_UNPOOL(6);
    else return fail(VTP_ERR_SHAPE, "unpool: C=%d too large", C);
#undef VTP_UNPOOL
    return check_launch("unpool_add");
}

template <typename T>
static int launch_ln(const void* x, int rows_max, const int32_t* rows_dev, int C, long long stride,
                     const float* w, const float* b, float eps, void* y, cudaStream_t st, const RowAdd& add = RowAdd()) {
    const int maxch = ceil_div(C / Vec<T>::N, 32);
    const int nchunks = C / Vec<T>::N;
    if (nchunks <= 16) {
        const int rpw = nchunks <= 8 ? 4 : 2;
        const int g = row_grid(ceil_div(rows_max, rpw));
        if (nchunks <= 8)
            layernorm_narrow_kernel<T, 8><<<g, 256, 0, st>>>((const T*)x, rows_max, rows_dev, C, stride, w, b, eps, (T*)y, add);
        else
            layernorm_narrow_kernel<T, 16><<<g, 256, 0, st>>>((const T*)x, rows_max, rows_dev, C, stride, w, b, eps, (T*)y, add);
        return check_launch("layernorm");
    }
    const int grid = row_grid(rows_max);
#define VTP_LN(M)                                                                                 \
    layernorm_kernel<T, M><<<grid, 256, 0, st>>>((const T*)x, rows_max, rows_dev, C, stride, w, b, \
                                                 eps, (T*)y, add)
    if (maxch <= 1) VTP_LN(1);
    else if (maxch == 2) VTP_LN(2);
    else if (maxch == 3) VTP_LN(3);
    else if (maxch == 4) VTP_LN(4);
    else if (maxch <= 6) VTP_LN(6);
    else return fail(VTP_ERR_SHAPE, "layernorm: C=%d too large", C);
#undef VTP_LN
    return check_launch("layernorm");
}

static int check_rows(const char* what, int dtype, int C, const void* a, const void* b) {
    VTP_REQUIRE(dtype == VTP_F32 || dtype == VTP_BF16, VTP_ERR_DTYPE, "%s: dtype %d", what, dtype);
    VTP_REQUIRE(C > 0 && C % (16 / (int)elem_size(dtype)) == 0 && C % 4 == 0, VTP_ERR_SHAPE,
                "%s: C=%d must be a multiple of 16 bytes", what, C);
    VTP_REQUIRE(aligned16(a) && aligned16(b), VTP_ERR_ALIGN, "%s: unaligned pointer", what);
    return VTP_OK;
}

// pool / unpool rows: any C > 0; rows of whole 16-byte chunks take the vector kernels, which need
// 16-byte aligned pointers
static bool vector_rows(int dtype, int C) { return C % (16 / (int)elem_size(dtype)) == 0; }
static int check_token_rows(const char* what, int dtype, int C, const void* a, const void* b, const void* c,
                            const void* d) {
    VTP_REQUIRE(dtype == VTP_F32 || dtype == VTP_BF16, VTP_ERR_DTYPE, "%s: dtype %d", what, dtype);
    VTP_REQUIRE(C > 0, VTP_ERR_SHAPE, "%s: C=%d", what, C);
    if (vector_rows(dtype, C))
        VTP_REQUIRE(aligned16(a) && aligned16(b) && aligned16(c) && aligned16(d), VTP_ERR_ALIGN,
                    "%s: unaligned pointer", what);
    return VTP_OK;
}

}  // namespace vtp

using namespace vtp;

extern "C" int vtp_pool(const void* x, int dtype, int B, int N, int C, int W, int num_extra,
                        const int32_t* patches, const int32_t* n_patches_dev, int n_patches_max,
                        void* comp, const float* ln_w, const float* ln_b, float eps, void* xn,
                        void* qn, void* stream) {
    VTP_REQUIRE(x && patches && comp, VTP_ERR_NULL, "pool: null pointer");
    VTP_REQUIRE((ln_w == nullptr) == (ln_b == nullptr), VTP_ERR_NULL, "pool: ln_w and ln_b go together");
    VTP_REQUIRE(ln_w || (!xn && !qn), VTP_ERR_NULL, "pool: xn/qn need LayerNorm weights");
    VTP_REQUIRE(B > 0 && N > 0 && W > 0 && num_extra >= 0 && n_patches_max >= 0, VTP_ERR_SHAPE,
                "pool: bad shape");
    VTP_REQUIRE(N > num_extra && (N - num_extra) % W == 0, VTP_ERR_SHAPE, "pool: N - num_extra = %d is not a whole number of grid rows of %d tokens", N - num_extra, W);
    if (int rc = check_token_rows("pool", dtype, C, x, comp, xn, qn)) return rc;
    VTP_REQUIRE(aligned16(patches), VTP_ERR_ALIGN, "pool: unaligned patch list");
    if (n_patches_max == 0) return VTP_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == VTP_F32)
        return launch_pool<float>(x, B, N, C, W, num_extra, patches, n_patches_dev, n_patches_max, comp,
                                  ln_w, ln_b, eps, xn, qn, 1, st);
    return launch_pool<bf16>(x, B, N, C, W, num_extra, patches, n_patches_dev, n_patches_max, comp, ln_w,
                             ln_b, eps, xn, qn, 1, st);
}

extern "C" int vtp_unpool_add(const void* q, const void* comp, int dtype, int B, int N, int C, int W,
                              int num_extra, const int32_t* patches, const int32_t* n_patches_dev,
                              int n_patches_max, const void* ref, void* out, void* stream) {
    VTP_REQUIRE(q && patches && out, VTP_ERR_NULL, "unpool: null pointer");
    VTP_REQUIRE(B > 0 && N > 0 && W > 0 && num_extra >= 0 && n_patches_max >= 0, VTP_ERR_SHAPE,
                "unpool: bad shape");
    VTP_REQUIRE(N > num_extra && (N - num_extra) % W == 0, VTP_ERR_SHAPE, "unpool: N - num_extra = %d is not a whole number of grid rows of %d tokens", N - num_extra, W);
    if (int rc = check_token_rows("unpool", dtype, C, q, out, comp, ref)) return rc;
    VTP_REQUIRE(aligned16(patches), VTP_ERR_ALIGN, "unpool: unaligned patch list");
    if (n_patches_max == 0) return VTP_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == VTP_F32)
        return launch_unpool<float>(q, comp, B, N, C, W, num_extra, patches, n_patches_dev, n_patches_max,
                                    ref, out, 0, st);
    return launch_unpool<bf16>(q, comp, B, N, C, W, num_extra, patches, n_patches_dev, n_patches_max, ref,
                               out, 0, st);
}

// Gradients of the two movers; each is the other kernel with a different scale
// (vtpack/layers/grained_sample.py:26-38 and :61-78).
extern "C" int vtp_pool_grad(const void* grad_comp, int dtype, int B, int N, int C, int W, int num_extra,
                             const int32_t* patches, const int32_t* n_patches_dev, int n_patches_max,
                             void* grad_x, void* stream) {
    VTP_REQUIRE(grad_comp && patches && grad_x, VTP_ERR_NULL, "pool_grad: null pointer");
    VTP_REQUIRE(B > 0 && N > 0 && W > 0 && num_extra >= 0 && n_patches_max >= 0, VTP_ERR_SHAPE,
                "pool_grad: bad shape");
    VTP_REQUIRE(N > num_extra && (N - num_extra) % W == 0, VTP_ERR_SHAPE, "pool_grad: N - num_extra = %d is not a whole number of grid rows of %d tokens", N - num_extra, W);
    if (int rc = check_token_rows("pool_grad", dtype, C, grad_comp, grad_x, nullptr, nullptr)) return rc;
    VTP_REQUIRE(aligned16(patches), VTP_ERR_ALIGN, "pool_grad: unaligned patch list");
    if (n_patches_max == 0) return VTP_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == VTP_F32)
        return launch_unpool<float>(grad_comp, nullptr, B, N, C, W, num_extra, patches, n_patches_dev,
                                    n_patches_max, nullptr, grad_x, 1, st);
    return launch_unpool<bf16>(grad_comp, nullptr, B, N, C, W, num_extra, patches, n_patches_dev, n_patches_max,
                               nullptr, grad_x, 1, st);
}

extern "C" int vtp_unpool_grad(const void* grad_out, int dtype, int B, int N, int C, int W, int num_extra,
                               const int32_t* patches, const int32_t* n_patches_dev, int n_patches_max,
                               void* grad_q, void* stream) {
    VTP_REQUIRE(grad_out && patches && grad_q, VTP_ERR_NULL, "unpool_grad: null pointer");
    VTP_REQUIRE(B > 0 && N > 0 && W > 0 && num_extra >= 0 && n_patches_max >= 0, VTP_ERR_SHAPE,
                "unpool_grad: bad shape");
    VTP_REQUIRE(N > num_extra && (N - num_extra) % W == 0, VTP_ERR_SHAPE, "unpool_grad: N - num_extra = %d is not a whole number of grid rows of %d tokens", N - num_extra, W);
    if (int rc = check_token_rows("unpool_grad", dtype, C, grad_out, grad_q, nullptr, nullptr)) return rc;
    VTP_REQUIRE(aligned16(patches), VTP_ERR_ALIGN, "unpool_grad: unaligned patch list");
    if (n_patches_max == 0) return VTP_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == VTP_F32)
        return launch_pool<float>(grad_out, B, N, C, W, num_extra, patches, n_patches_dev, n_patches_max, grad_q,
                                  nullptr, nullptr, 0.f, nullptr, nullptr, 0, st);
    return launch_pool<bf16>(grad_out, B, N, C, W, num_extra, patches, n_patches_dev, n_patches_max, grad_q,
                             nullptr, nullptr, 0.f, nullptr, nullptr, 0, st);
}

// The same gradient for a patch list that was made from grain indices: one CTA per region, every token
// row of the region requested before any arithmetic, no walk over the list (region_ops.cu).
extern "C" int vtp_region_layout_supported(int dtype, int C) {
    RegionGeom g{};
    g.B = g.Hr = g.Wr = 1; g.C = C; g.region = 4;
    return (dtype == VTP_F32 || dtype == VTP_BF16) && C > 0 && region_ops_supported(g, dtype) ? 1 : 0;
}

extern "C" int vtp_unpool_grad_regions(const void* grad_out, int dtype, int B, int Hr, int Wr, int region_size,
                                       int C, int num_extra, const int32_t* indices, const int* splits,
                                       int n_splits, const int32_t* region_first, const int32_t* offsets,
                                       int n_patches, void* grad_q, void* stream) {
    VTP_REQUIRE(grad_out && indices && splits && region_first && offsets && grad_q, VTP_ERR_NULL,
                "unpool_grad (regions): null pointer");
    VTP_REQUIRE(dtype == VTP_F32 || dtype == VTP_BF16, VTP_ERR_DTYPE, "unpool_grad (regions): dtype %d", dtype);
    VTP_REQUIRE(B > 0 && Hr > 0 && Wr > 0 && C > 0 && num_extra >= 0 && n_patches >= 0, VTP_ERR_SHAPE,
                "unpool_grad (regions): bad shape");
    if (n_patches == 0) return VTP_OK;
    RegionPoolArgs a;
    if (int rc = make_splits(&a.sp, splits, n_splits, region_size)) return rc;
    a.g.B = B; a.g.Hr = Hr; a.g.Wr = Wr; a.g.W = Wr * region_size; a.g.C = C; a.g.num_extra = num_extra;
    a.g.region = region_size;
    a.g.N = num_extra + Hr * Wr * region_size * region_size;
    VTP_REQUIRE(region_ops_supported(a.g, dtype), VTP_ERR_SHAPE,
                "unpool_grad (regions): region size %d / C=%d have no region kernel (use vtp_unpool_grad)", region_size, C);
    VTP_REQUIRE(aligned16(grad_out) && aligned16(grad_q), VTP_ERR_ALIGN, "unpool_grad (regions): unaligned rows");
    a.x = grad_out; a.idx = indices; a.region_first = region_first; a.offsets = offsets; a.comp = grad_q;
    a.sum_only = true;
    a.g.l_max = n_patches;       // regions whose rows would not fit grad_q are skipped and flagged
    return region_pool(a, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int vtp_layernorm_add_rows(const void* x, int dtype, int rows, int C, long long in_row_stride, const float* w,
                                      const float* b, float eps, const void* addend, int a_mod, int a_off, void* out,
                                      int out_grp, int out_stride, int out_off, void* stream) {
    VTP_REQUIRE(x && w && b && addend && out, VTP_ERR_NULL, "layernorm + add rows: null pointer");
    VTP_REQUIRE(rows >= 0 && in_row_stride >= C && a_mod > 0 && a_off >= 0 && out_grp > 0 && out_stride >= out_grp &&
                    out_off >= 0,
                VTP_ERR_SHAPE, "layernorm + add rows: bad shape");
    if (int rc = check_rows("layernorm + add rows", dtype, C, x, out)) return rc;
    VTP_REQUIRE(aligned16(addend), VTP_ERR_ALIGN, "layernorm + add rows: unaligned pointer");
    VTP_REQUIRE((in_row_stride * (long long)elem_size(dtype)) % 16 == 0, VTP_ERR_ALIGN,
                "layernorm + add rows: row stride not 16-byte aligned");
    if (rows == 0) return VTP_OK;
    RowAdd add;
    add.addend = addend; add.a_mod = a_mod; add.a_off = a_off; add.out_grp = out_grp; add.out_stride = out_stride;
    add.out_off = out_off;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == VTP_F32) return launch_ln<float>(x, rows, nullptr, C, in_row_stride, w, b, eps, out, st, add);
    return launch_ln<bf16>(x, rows, nullptr, C, in_row_stride, w, b, eps, out, st, add);
}

extern "C" int vtp_layernorm(const void* x, int dtype, int rows_max, const int32_t* rows_dev, int C,
                             long long in_row_stride, const float* w, const float* b, float eps,
                             void* y, void* stream) {
    VTP_REQUIRE(x && w && b && y, VTP_ERR_NULL, "layernorm: null pointer");
    VTP_REQUIRE(rows_max >= 0 && in_row_stride >= C, VTP_ERR_SHAPE, "layernorm: bad shape");
    if (int rc = check_rows("layernorm", dtype, C, x, y)) return rc;
    VTP_REQUIRE((in_row_stride * (long long)elem_size(dtype)) % 16 == 0, VTP_ERR_ALIGN,
                "layernorm: row stride not 16-byte aligned");
    if (rows_max == 0) return VTP_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == VTP_F32)
        return launch_ln<float>(x, rows_max, rows_dev, C, in_row_stride, w, b, eps, y, st);
    return launch_ln<bf16>(x, rows_max, rows_dev, C, in_row_stride, w, b, eps, y, st);
}
