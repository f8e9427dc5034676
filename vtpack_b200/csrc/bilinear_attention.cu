// Bilinear-sampling attention of the deformable PVT (vtpack/models/standard/dpvt.py:92-115):
// every query position g of a feature map [B, H, W, C] looks at P sampling points given in pixel
// coordinates (x, y), reads the map there by bilinear interpolation (zero outside the map) and
//   "point"   mode: out[b,g,c] = sum_p weight[b,g,p] * sample(b, p, c)         weight [B,G,P]
//   "channel" mode: out[b,g,p] = sum_c weight[b,g,c] * sample(b, p, c)         weight [B,G,C]
// Replaces bilinear_attention_{pointwise,channelwise}_{forward,backward}
// (vtpack/layers/csrc/bilinear_attention/bilinear_attention.cu:88-132, :134-232, :234-268, :270-362).
//
// The reference runs one thread per (b, g) that walks the channels serially, so neighbouring
// threads read addresses C elements apart.  Here one warp owns a (b, g) instance and its lanes walk
// the channels: every corner read, every atomic of the input gradient and every output row is a
// run of consecutive addresses; with an even C a lane takes two neighbouring channels, which halves
// the loads and (packed float2 / bf16x2 atomics) the atomic traffic of the input gradient.  All four
// kernels are bound by those gathers (4 corner rows per point), not by arithmetic.
#include <initializer_list>

#include "common.cuh"

namespace vtp {

constexpr int BA_WARPS = 8;           // instances per 256-thread block
constexpr int BA_MAXCH = 8;           // channel-mode backward keeps C / 32 weight gradients per lane

struct Corner {
    int x0, y0;
    float w_lt, w_rt, w_lb, w_rb, tx, ty;
    bool in_lt, in_rt, in_lb, in_rb;
};

__device__ __forceinline__ Corner corners_of(float x, float y, int H, int W) {
    Corner c;
    const float fx = floorf(x), fy = floorf(y);
    c.x0 = (int)fx;
    c.y0 = (int)fy;
    c.tx = x - fx;
    c.ty = y - fy;
    c.w_lt = (1.f - c.tx) * (1.f - c.ty);
    c.w_rt = c.tx * (1.f - c.ty);
    c.w_lb = (1.f - c.tx) * c.ty;
    c.w_rb = c.tx * c.ty;
    const bool xl = c.x0 >= 0 && c.x0 < W, xr = c.x0 + 1 >= 0 && c.x0 + 1 < W;
    const bool yt = c.y0 >= 0 && c.y0 < H, yb = c.y0 + 1 >= 0 && c.y0 + 1 < H;
    c.in_lt = xl && yt; c.in_rt = xr && yt; c.in_lb = xl && yb; c.in_rb = xr && yb;
    return c;
}

// a coordinate far outside the map (or not finite) touches no pixel; clamp it so the int casts stay defined
__device__ __forceinline__ float sane(float v, int extent) {
    return (v > -4.f && v < (float)extent + 4.f) ? v : -4.f;
}

// V consecutive channels per lane (2 when C is even: half the loads and half the atomics)
template <typename T, int V> struct Pack;
template <> struct Pack<float, 1> {
    static __device__ __forceinline__ void load(const float* p, float (&f)[1]) { f[0] = *p; }
    static __device__ __forceinline__ void store(float* p, const float (&f)[1]) { *p = f[0]; }
    static __device__ __forceinline__ void atomic_add(float* p, const float (&f)[1]) { atomicAdd(p, f[0]); }
};
template <> struct Pack<float, 2> {
    static __device__ __forceinline__ void load(const float* p, float (&f)[2]) {
        const float2 v = *reinterpret_cast<const float2*>(p);
        f[0] = v.x; f[1] = v.y;
    }
    static __device__ __forceinline__ void store(float* p, const float (&f)[2]) {
        *reinterpret_cast<float2*>(p) = make_float2(f[0], f[1]);
    }
    static __device__ __forceinline__ void atomic_add(float* p, const float (&f)[2]) {
        atomicAdd(reinterpret_cast<float2*>(p), make_float2(f[0], f[1]));
    }
};
template <> struct Pack<bf16, 1> {
    static __device__ __forceinline__ void load(const bf16* p, float (&f)[1]) { f[0] = __bfloat162float(*p); }
    static __device__ __forceinline__ void store(bf16* p, const float (&f)[1]) { *p = __float2bfloat16_rn(f[0]); }
    static __device__ __forceinline__ void atomic_add(bf16* p, const float (&f)[1]) {
        atomicAdd(p, __float2bfloat16_rn(f[0]));
    }
};
template <> struct Pack<bf16, 2> {
    static __device__ __forceinline__ void load(const bf16* p, float (&f)[2]) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
        f[0] = v.x; f[1] = v.y;
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&f)[2]) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(f[0], f[1]);
    }
    static __device__ __forceinline__ void atomic_add(bf16* p, const float (&f)[2]) {
        atomicAdd(reinterpret_cast<__nv_bfloat162*>(p), __floats2bfloat162_rn(f[0], f[1]));
    }
};

template <typename T, int V>
struct Taps {
    float lt[V], rt[V], lb[V], rb[V];
    __device__ __forceinline__ void load(const T* __restrict__ img, const Corner& k, int W, int C, int c) {
        const size_t o = ((size_t)k.y0 * W + k.x0) * C + c;   // only dereferenced where in-bounds
#pragma unroll
        for (int v = 0; v < V; ++v) lt[v] = rt[v] = lb[v] = rb[v] = 0.f;
        if (k.in_lt) Pack<T, V>::load(img + o, lt);
        if (k.in_rt) Pack<T, V>::load(img + o + C, rt);
        if (k.in_lb) Pack<T, V>::load(img + o + (size_t)W * C, lb);
        if (k.in_rb) Pack<T, V>::load(img + o + (size_t)W * C + C, rb);
    }
    __device__ __forceinline__ float value(const Corner& k, int v) const {
        return k.w_lt * lt[v] + k.w_rt * rt[v] + k.w_lb * lb[v] + k.w_rb * rb[v];
    }
};

template <typename T, int V>
__device__ __forceinline__ void scatter(T* __restrict__ gimg, const Corner& k, int W, int C, int c, const float (&g)[V]) {
    const size_t o = ((size_t)k.y0 * W + k.x0) * C + c;
    float t[V];
#define VTP_BA_SCATTER(IN, OFF, WT)                              \
    if (IN) {                                                    \
        _Pragma("unroll") for (int v = 0; v < V; ++v) t[v] = g[v] * (WT); \
        Pack<T, V>::atomic_add(gimg + o + (OFF), t);             \
    }
    VTP_BA_SCATTER(k.in_lt, 0, k.w_lt)
    VTP_BA_SCATTER(k.in_rt, C, k.w_rt)
    VTP_BA_SCATTER(k.in_lb, (size_t)W * C, k.w_lb)
    VTP_BA_SCATTER(k.in_rb, (size_t)W * C + C, k.w_rb)
#undef VTP_BA_SCATTER
}

// ---------------------------------------------------------------------------- forward
template <typename T, bool POINT, int V>
__global__ void __launch_bounds__(BA_WARPS * 32)
bilinear_attention_fwd_kernel(const T* __restrict__ input, const T* __restrict__ grid, const T* __restrict__ weight,
                              T* __restrict__ out, int B, int H, int W, int C, int G, int P,
                              const long long* __restrict__ batch_of) {
    // batch_of == null: B * G instances, G per image; else G packed instances, instance i reads image batch_of[i]
    const int lane = threadIdx.x & 31;
    const long long n_inst = batch_of ? (long long)G : (long long)B * G;
    for (long long inst = (long long)blockIdx.x * BA_WARPS + (threadIdx.x >> 5); inst < n_inst;
         inst += (long long)gridDim.x * BA_WARPS) {
        long long b = batch_of ? batch_of[inst] : inst / G;
        const bool image_ok = b >= 0 && b < B;          // an instance naming no image reads zeros
        if (!image_ok) b = 0;
        const int Hb = image_ok ? H : 0;                 // no pixel is in bounds
        const T* img = input + (size_t)b * H * W * C;
        const T* pts = grid + (size_t)inst * P * 2;
        if (POINT) {
            const T* wt = weight + (size_t)inst * P;
            for (int c = lane * V; c < C; c += 32 * V) {
                float acc[V];
#pragma unroll
                for (int v = 0; v < V; ++v) acc[v] = 0.f;
                for (int p = 0; p < P; ++p) {
                    const Corner k = corners_of(sane(to_f32(pts[2 * p]), W), sane(to_f32(pts[2 * p + 1]), H), Hb, W);
                    Taps<T, V> t;
                    t.load(img, k, W, C, c);
                    const float wp = to_f32(wt[p]);
#pragma unroll
                    for (int v = 0; v < V; ++v) acc[v] = fmaf(t.value(k, v), wp, acc[v]);
                }
                Pack<T, V>::store(out + (size_t)inst * C + c, acc);
            }
        } else {
            const T* wt = weight + (size_t)inst * C;
            for (int p = 0; p < P; ++p) {
                const Corner k = corners_of(sane(to_f32(pts[2 * p]), W), sane(to_f32(pts[2 * p + 1]), H), Hb, W);
                float acc = 0.f;
                for (int c = lane * V; c < C; c += 32 * V) {
                    Taps<T, V> t;
                    t.load(img, k, W, C, c);
                    float wc[V];
                    Pack<T, V>::load(wt + c, wc);
#pragma unroll
                    for (int v = 0; v < V; ++v) acc = fmaf(t.value(k, v), wc[v], acc);
                }
                acc = warp_sum(acc);
                if (lane == 0) out[(size_t)inst * P + p] = from_f32<T>(acc);
            }
        }
    }
}

// --------------------------------------------------------------------------- backward
// grad_input must be zero on entry (the host wrapper clears it on the same stream).
template <typename T, bool POINT, int V>
__global__ void __launch_bounds__(BA_WARPS * 32)
bilinear_attention_bwd_kernel(const T* __restrict__ grad_out, const T* __restrict__ input, const T* __restrict__ grid,
                              const T* __restrict__ weight, T* __restrict__ grad_input, T* __restrict__ grad_grid,
                              T* __restrict__ grad_weight, int B, int H, int W, int C, int G, int P) {
    constexpr int J = BA_MAXCH / V;                        // channel groups per lane
    const int lane = threadIdx.x & 31;
    const long long n_inst = (long long)B * G;
    for (long long inst = (long long)blockIdx.x * BA_WARPS + (threadIdx.x >> 5); inst < n_inst;
         inst += (long long)gridDim.x * BA_WARPS) {
        const int b = (int)(inst / G);
        const T* img = input + (size_t)b * H * W * C;
        T* gimg = grad_input + (size_t)b * H * W * C;
        const T* pts = grid + (size_t)inst * P * 2;
        // per lane and channel group: the upstream gradient (point mode) or the weight (channel mode),
        // read once, and in channel mode the weight gradient accumulated over the points
        float up[J][V], gw_c[J][V];
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const int c = (lane + 32 * j) * V;
#pragma unroll
            for (int v = 0; v < V; ++v) up[j][v] = gw_c[j][v] = 0.f;
            if (c < C) Pack<T, V>::load((POINT ? grad_out : weight) + (size_t)inst * C + c, up[j]);
        }
        for (int p = 0; p < P; ++p) {
            const Corner k = corners_of(sane(to_f32(pts[2 * p]), W), sane(to_f32(pts[2 * p + 1]), H), H, W);
            // scale turning up[] into g = d(loss) / d(sample(b, p, c))
            const float sc = POINT ? to_f32(weight[(size_t)inst * P + p]) : to_f32(grad_out[(size_t)inst * P + p]);
            float gix = 0.f, giy = 0.f, giw = 0.f;
#pragma unroll
            for (int j = 0; j < J; ++j) {
                const int c = (lane + 32 * j) * V;
                if (c < C) {
                    float g[V];
#pragma unroll
                    for (int v = 0; v < V; ++v) g[v] = up[j][v] * sc;
                    scatter<T, V>(gimg, k, W, C, c, g);
                    Taps<T, V> t;
                    t.load(img, k, W, C, c);
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        // d(sample)/dx and d(sample)/dy of the bilinear form
                        gix += g[v] * ((t.rt[v] - t.lt[v]) * (1.f - k.ty) + (t.rb[v] - t.lb[v]) * k.ty);
                        giy += g[v] * ((t.lb[v] - t.lt[v]) * (1.f - k.tx) + (t.rb[v] - t.rt[v]) * k.tx);
                        if (POINT) giw += t.value(k, v) * up[j][v];
                        else gw_c[j][v] += t.value(k, v) * sc;
                    }
                }
            }
            gix = warp_sum(gix);
            giy = warp_sum(giy);
            if (POINT) giw = warp_sum(giw);
            if (lane == 0) {
                grad_grid[((size_t)inst * P + p) * 2] = from_f32<T>(gix);
                grad_grid[((size_t)inst * P + p) * 2 + 1] = from_f32<T>(giy);
                if (POINT) grad_weight[(size_t)inst * P + p] = from_f32<T>(giw);
            }
        }
        if (!POINT) {
#pragma unroll
            for (int j = 0; j < J; ++j) {
                const int c = (lane + 32 * j) * V;
                if (c < C) Pack<T, V>::store(grad_weight + (size_t)inst * C + c, gw_c[j]);
            }
        }
    }
}

static int ba_grid(long long instances) {
    const long long want = (instances + BA_WARPS - 1) / BA_WARPS;
    const long long cap = (long long)sm_count() * 16;
    return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

static int ba_check(const char* what, int dtype, int mode, int B, int H, int W, int C, int G, int P) {
    VTP_REQUIRE(dtype == VTP_F32 || dtype == VTP_BF16, VTP_ERR_DTYPE, "%s: dtype %d", what, dtype);
    VTP_REQUIRE(mode == 0 || mode == 1, VTP_ERR_SHAPE, "%s: mode %d (0 = point, 1 = channel)", what, mode);
    VTP_REQUIRE(B > 0 && H > 0 && W > 0 && C > 0 && G > 0 && P > 0, VTP_ERR_SHAPE, "%s: bad shape", what);
    return VTP_OK;
}

// channel pairs need an even C and every channel-indexed pointer aligned to a pair
static bool ba_pairs(int dtype, int C, std::initializer_list<const void*> ptrs) {
    if (C % 2) return false;
    const uintptr_t mask = 2 * elem_size(dtype) - 1;
    for (const void* p : ptrs)
        if (reinterpret_cast<uintptr_t>(p) & mask) return false;
    return true;
}

}  // namespace vtp

using namespace vtp;

static int ba_forward(const void* input, const void* grid, const void* weight, void* out, int dtype, int mode, int B,
                      int H, int W, int C, int G, int P, const long long* batch_of, void* stream) {
    VTP_REQUIRE(input && grid && weight && out, VTP_ERR_NULL, "bilinear_attention: null pointer");
    if (int rc = ba_check("bilinear_attention", dtype, mode, B, H, W, C, G, P)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int blocks = ba_grid(batch_of ? (long long)G : (long long)B * G);
    const bool pairs = ba_pairs(dtype, C, {input, weight, out});
#define VTP_BA_FWD(T, PT)                                                                                    \
    do {                                                                                                     \
        if (pairs)                                                                                           \
            bilinear_attention_fwd_kernel<T, PT, 2><<<blocks, BA_WARPS * 32, 0, st>>>(                       \
                (const T*)input, (const T*)grid, (const T*)weight, (T*)out, B, H, W, C, G, P, batch_of);     \
        else                                                                                                 \
            bilinear_attention_fwd_kernel<T, PT, 1><<<blocks, BA_WARPS * 32, 0, st>>>(                       \
                (const T*)input, (const T*)grid, (const T*)weight, (T*)out, B, H, W, C, G, P, batch_of);     \
    } while (0)
    if (dtype == VTP_F32) { if (mode == 0) VTP_BA_FWD(float, true); else VTP_BA_FWD(float, false); }
    else { if (mode == 0) VTP_BA_FWD(bf16, true); else VTP_BA_FWD(bf16, false); }
#undef VTP_BA_FWD
    return check_launch("bilinear_attention_forward");
}

extern "C" int vtp_bilinear_attention_forward(const void* input, const void* grid, const void* weight, void* out,
                                              int dtype, int mode, int B, int H, int W, int C, int G, int P,
                                              void* stream) {
    return ba_forward(input, grid, weight, out, dtype, mode, B, H, W, C, G, P, nullptr, stream);
}

extern "C" int vtp_sparse_bilinear_attention_forward(const void* input, const void* grid, const void* weight,
                                                     const long long* batches, void* out, int dtype, int B, int H,
                                                     int W, int C, int L, int P, void* stream) {
    VTP_REQUIRE(batches, VTP_ERR_NULL, "sparse_bilinear_attention: null batches");
    if (L == 0) return VTP_OK;
    return ba_forward(input, grid, weight, out, dtype, 0, B, H, W, C, L, P, batches, stream);
}

extern "C" int vtp_bilinear_attention_backward(const void* grad_out, const void* input, const void* grid,
                                               const void* weight, void* grad_input, void* grad_grid,
                                               void* grad_weight, int dtype, int mode, int B, int H, int W, int C,
                                               int G, int P, void* stream) {
    VTP_REQUIRE(grad_out && input && grid && weight && grad_input && grad_grid && grad_weight, VTP_ERR_NULL,
                "bilinear_attention_backward: null pointer");
    if (int rc = ba_check("bilinear_attention_backward", dtype, mode, B, H, W, C, G, P)) return rc;
    VTP_REQUIRE(C <= 32 * BA_MAXCH, VTP_ERR_SHAPE, "bilinear_attention_backward: C=%d above %d", C, 32 * BA_MAXCH);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(grad_input, 0, (size_t)B * H * W * C * elem_size(dtype), st);
    if (e != cudaSuccess) return fail((int)e, "bilinear_attention_backward: clearing grad_input: %s", cudaGetErrorString(e));
    const int blocks = ba_grid((long long)B * G);
    const bool pairs = ba_pairs(dtype, C, {grad_out, input, weight, grad_input, grad_weight});
#define VTP_BA_BWD(T, PT)                                                                                    \
    do {                                                                                                     \
        if (pairs)                                                                                           \
            bilinear_attention_bwd_kernel<T, PT, 2><<<blocks, BA_WARPS * 32, 0, st>>>(                       \
                (const T*)grad_out, (const T*)input, (const T*)grid, (const T*)weight, (T*)grad_input,       \
                (T*)grad_grid, (T*)grad_weight, B, H, W, C, G, P);                                           \
        else                                                                                                 \
            bilinear_attention_bwd_kernel<T, PT, 1><<<blocks, BA_WARPS * 32, 0, st>>>(                       \
                (const T*)grad_out, (const T*)input, (const T*)grid, (const T*)weight, (T*)grad_input,       \
                (T*)grad_grid, (T*)grad_weight, B, H, W, C, G, P);                                           \
    } while (0)
    if (dtype == VTP_F32) { if (mode == 0) VTP_BA_BWD(float, true); else VTP_BA_BWD(float, false); }
    else { if (mode == 0) VTP_BA_BWD(bf16, true); else VTP_BA_BWD(bf16, false); }
#undef VTP_BA_BWD
    return check_launch("bilinear_attention_backward");
}
