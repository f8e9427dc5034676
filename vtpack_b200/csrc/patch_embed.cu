// Patch-embedding front end: im2col of the fp32 images into GEMM rows, and the cls rows.
// The 16x16/16 convolution is then one Linear (column = c*P*P + py*P + px matches the
// flattened conv weight [C, 3, P, P]).
//
// Replaces PatchEmbed, the cls-token concat and the position-embedding add of
// VisionTransformer.forward_features (vtpack/models/dge/deit_dge.py:268-275).
#include "common.cuh"

namespace vtp {

// One thread moves 8 horizontally adjacent pixels: two coalesced float4 loads, one
// 16-byte (bf16) or two 16-byte (fp32) stores.
// 8 consecutive pixels as floats, from fp32 or bf16 images
__device__ __forceinline__ void load8(const float* p, float* f) {
    const float4 v0 = __ldg(reinterpret_cast<const float4*>(p));
    const float4 v1 = __ldg(reinterpret_cast<const float4*>(p) + 1);
    f[0] = v0.x; f[1] = v0.y; f[2] = v0.z; f[3] = v0.w; f[4] = v1.x; f[5] = v1.y; f[6] = v1.z; f[7] = v1.w;
}
__device__ __forceinline__ void load8(const bf16* p, float* f) {
    Vec<bf16> v;
    v.raw = __ldg(reinterpret_cast<const uint4*>(p));
    v.to_float(f);
}

// Patches narrower than 8 pixels (PVT's first stage: 4 x 4): one thread moves 4 adjacent pixels.
template <typename I, typename T>
__global__ void __launch_bounds__(256)
im2col4_kernel(const I* __restrict__ img, long long total4, int S, int P, T* __restrict__ cols) {
    const int G = S / P;
    const int KP = 3 * P * P;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total4;
         e += (long long)gridDim.x * blockDim.x) {
        const long long pix = e * 4;
        const int ix = (int)(pix % S);
        const int iy = (int)((pix / S) % S);
        const int c = (int)((pix / ((long long)S * S)) % 3);
        const long long b = pix / ((long long)3 * S * S);
        float f[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = to_f32(img[pix + i]);
        const int gy = iy / P, py = iy % P, gx = ix / P, px = ix % P;
        T* dst = cols + ((b * G + gy) * G + gx) * KP + c * P * P + py * P + px;
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = from_f32<T>(f[i]);
    }
}

template <typename I, typename T>
__global__ void __launch_bounds__(256)
im2col_kernel(const I* __restrict__ img, long long total8, int S, int P, T* __restrict__ cols) {
    const int G = S / P;
    const int KP = 3 * P * P;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total8;
         e += (long long)gridDim.x * blockDim.x) {
        const long long pix = e * 8;
        const int ix = (int)(pix % S);
        const int iy = (int)((pix / S) % S);
        const int c = (int)((pix / ((long long)S * S)) % 3);
        const long long b = pix / ((long long)3 * S * S);
        float f[8];
        load8(img + pix, f);
        const int gy = iy / P, py = iy % P, gx = ix / P, px = ix % P;
        T* dst = cols + ((b * G + gy) * G + gx) * KP + c * P * P + py * P + px;
        if (sizeof(T) == 2) {
            Vec<bf16> o;
            o.from_float(f);
            o.store(reinterpret_cast<bf16*>(dst));
        } else {
            reinterpret_cast<float4*>(dst)[0] = make_float4(f[0], f[1], f[2], f[3]);
            reinterpret_cast<float4*>(dst)[1] = make_float4(f[4], f[5], f[6], f[7]);
        }
    }
}

template <typename T>
__global__ void cls_row_kernel(const T* __restrict__ cls, const T* __restrict__ pos, int C, long long row_stride,
                               T* __restrict__ x) {
    const int b = blockIdx.x;
    for (int c = threadIdx.x; c < C; c += blockDim.x)
        x[(size_t)b * row_stride + c] = from_f32<T>(to_f32(cls[c]) + to_f32(pos[c]));
}

// Rows of the stride-sr reduction convolution of a PVT block as a GEMM operand: row (b, oy, ox) is
// the sr x sr window of tokens, column (dy, dx, c).  A window row (fixed dy) is sr consecutive
// tokens = sr*C contiguous elements on both sides; one thread moves 16 bytes.
// Replaces the permute / reshape in front of attn.sr (vtpack/models/dge/pvt_dge.py:82-83).
template <typename T>
__global__ void __launch_bounds__(256)
token_im2col_kernel(const T* __restrict__ x, long long total_vec, int H, int W, int C, int sr, T* __restrict__ cols,
                    const float2* __restrict__ stats, const float* __restrict__ lnw, const float* __restrict__ lnb) {
    // stats != null: the rows gathered are LayerNorm(x), normalised on the way from each token's (mean, rstd)
    constexpr int VN = Vec<T>::N;
    const int run = sr * C / VN;                  // 16-byte vectors per window row
    const int Wo = W / sr, Ho = H / sr;
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total_vec;
         v += (long long)gridDim.x * blockDim.x) {
        const int i = (int)(v % run);
        long long r = v / run;                    // (b, oy, ox, dy) with dy fastest
        const int dy = (int)(r % sr); r /= sr;
        const int ox = (int)(r % Wo); r /= Wo;
        const int oy = (int)(r % Ho);
        const long long b = r / Ho;
        const long long tok = (b * H + (long long)oy * sr + dy) * W + (long long)ox * sr;
        Vec<T> t;
        t.load(x + tok * C + (long long)i * VN);
        if (stats) {
            const int e0 = i * VN;                        // element of the window row: token e0 / C, channel e0 % C
            const float2 ms = stats[tok + e0 / C];
            const int ch = e0 % C;
            float f[VN];
            t.to_float(f);
#pragma unroll
            for (int k = 0; k < VN; ++k) f[k] = (f[k] - ms.x) * ms.y * __ldg(lnw + ch + k) + __ldg(lnb + ch + k);
            t.from_float(f);
        }
        t.store(cols + ((((b * Ho + oy) * Wo + ox) * sr + dy) * (long long)run + i) * VN);
    }
}

int token_im2col(const void* x, int dtype, int B, int H, int W, int C, int sr, void* cols, cudaStream_t st,
                 const float2* stats, const float* lnw, const float* lnb) {
    const int vn = dtype == VTP_BF16 ? 8 : 4;
    VTP_REQUIRE(C % vn == 0, VTP_ERR_SHAPE, "spatial reduction: C=%d must be a multiple of %d", C, vn);
    const long long total = (long long)B * H * W * C / vn;
    if (total == 0) return VTP_OK;
    const int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (dtype == VTP_BF16)
        token_im2col_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)x, total, H, W, C, sr, (bf16*)cols, stats, lnw, lnb);
    else
        token_im2col_kernel<float><<<grid, 256, 0, st>>>((const float*)x, total, H, W, C, sr, (float*)cols, stats, lnw, lnb);
    return check_launch("spatial reduction im2col");
}

// out[orow(r)] = x[r % x_mod] + addend[r % a_mod + a_off], orow(r) = (r / out_grp) * out_stride + out_off + r % out_grp:
// the position-embedding add of a token stage, and (x_mod = a_mod = out_grp = 1) the cls rows put in front of it.
template <typename T>
__global__ void __launch_bounds__(256)
add_rows_kernel(const T* __restrict__ x, int x_mod, const T* __restrict__ addend, int a_mod, int a_off,
                T* __restrict__ out, int out_grp, int out_stride, int out_off, long long total_vec, int C) {
    constexpr int VN = Vec<T>::N;
    const int cv = C / VN;
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total_vec;
         v += (long long)gridDim.x * blockDim.x) {
        const long long r = v / cv;
        const int i = (int)(v % cv) * VN;
        Vec<T> a, p;
        float fa[VN], fp[VN];
        a.load(x + (r % x_mod) * C + i);
        p.load(addend + (r % a_mod + a_off) * C + i);
        a.to_float(fa);
        p.to_float(fp);
#pragma unroll
        for (int k = 0; k < VN; ++k) fa[k] += fp[k];
        a.from_float(fa);
        a.store(out + ((r / out_grp) * out_stride + out_off + r % out_grp) * C + i);
    }
}

}  // namespace vtp

using namespace vtp;

extern "C" int vtp_token_im2col(const void* x, int dtype, int B, int H, int W, int C, int ratio, void* cols,
                                void* stream) {
    VTP_REQUIRE(x && cols, VTP_ERR_NULL, "token im2col: null pointer");
    VTP_REQUIRE(dtype == VTP_F32 || dtype == VTP_BF16, VTP_ERR_DTYPE, "token im2col: dtype %d", dtype);
    VTP_REQUIRE(B > 0 && H > 0 && W > 0 && C > 0 && ratio > 0 && H % ratio == 0 && W % ratio == 0, VTP_ERR_SHAPE,
                "token im2col: grid %dx%d / ratio %d", H, W, ratio);
    VTP_REQUIRE(aligned16(x) && aligned16(cols), VTP_ERR_ALIGN, "token im2col: unaligned pointer");
    return token_im2col(x, dtype, B, H, W, C, ratio, cols, static_cast<cudaStream_t>(stream), nullptr, nullptr, nullptr);
}

extern "C" int vtp_add_rows(const void* x, int x_mod, const void* addend, int a_mod, int a_off, void* out, int out_grp,
                            int out_stride, int out_off, int dtype, long long rows, int C, void* stream) {
    VTP_REQUIRE(x && addend && out, VTP_ERR_NULL, "add rows: null pointer");
    VTP_REQUIRE(dtype == VTP_F32 || dtype == VTP_BF16, VTP_ERR_DTYPE, "add rows: dtype %d", dtype);
    const int vn = dtype == VTP_BF16 ? 8 : 4;
    VTP_REQUIRE(rows >= 0 && C > 0 && C % vn == 0 && x_mod > 0 && a_mod > 0 && a_off >= 0 && out_grp > 0 &&
                    out_stride >= out_grp && out_off >= 0,
                VTP_ERR_SHAPE, "add rows: bad shape");
    VTP_REQUIRE(aligned16(x) && aligned16(addend) && aligned16(out), VTP_ERR_ALIGN, "add rows: unaligned pointer");
    const long long total = rows * (C / vn);
    if (total == 0) return VTP_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = (int)((total + 255) / 256 < (long long)sm_count() * 16 ? (total + 255) / 256 : (long long)sm_count() * 16);
    if (dtype == VTP_BF16)
        add_rows_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)x, x_mod, (const bf16*)addend, a_mod, a_off, (bf16*)out,
                                                   out_grp, out_stride, out_off, total, C);
    else
        add_rows_kernel<float><<<grid, 256, 0, st>>>((const float*)x, x_mod, (const float*)addend, a_mod, a_off,
                                                    (float*)out, out_grp, out_stride, out_off, total, C);
    return check_launch("add rows");
}

extern "C" int vtp_patch_im2col(const void* images, int image_dtype, int B, int S, int P, int dtype, void* cols,
                                const void* cls_token, const void* pos_embed, int C, void* x, void* stream) {
    VTP_REQUIRE(images && cols, VTP_ERR_NULL, "im2col: null pointer");
    VTP_REQUIRE(dtype == VTP_F32 || dtype == VTP_BF16, VTP_ERR_DTYPE, "im2col: dtype %d", dtype);
    VTP_REQUIRE(image_dtype == VTP_F32 || image_dtype == VTP_BF16, VTP_ERR_DTYPE, "im2col: image dtype %d", image_dtype);
    VTP_REQUIRE(B > 0 && S > 0 && P > 0 && S % P == 0 && P % 4 == 0, VTP_ERR_SHAPE,
                "im2col: image %d / patch %d (patch must be a multiple of 4)", S, P);
    VTP_REQUIRE(aligned16(images) && aligned16(cols), VTP_ERR_ALIGN, "im2col: unaligned pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (P % 8 != 0) {
        VTP_REQUIRE(!x, VTP_ERR_UNSUPPORTED, "im2col: the cls row is written for patches that are multiples of 8 only");
        const long long total4 = (long long)B * 3 * S * S / 4;
        const int g4 = (int)((total4 + 255) / 256 < (long long)sm_count() * 16 ? (total4 + 255) / 256
                                                                                : (long long)sm_count() * 16);
        if (image_dtype == VTP_F32 && dtype == VTP_F32)
            im2col4_kernel<float, float><<<g4, 256, 0, st>>>((const float*)images, total4, S, P, (float*)cols);
        else if (image_dtype == VTP_F32)
            im2col4_kernel<float, bf16><<<g4, 256, 0, st>>>((const float*)images, total4, S, P, (bf16*)cols);
        else if (dtype == VTP_F32)
            im2col4_kernel<bf16, float><<<g4, 256, 0, st>>>((const bf16*)images, total4, S, P, (float*)cols);
        else
            im2col4_kernel<bf16, bf16><<<g4, 256, 0, st>>>((const bf16*)images, total4, S, P, (bf16*)cols);
        return check_launch("im2col");
    }
    const long long total8 = (long long)B * 3 * S * S / 8;
    const int grid = (int)((total8 + 255) / 256 < (long long)sm_count() * 16 ? (total8 + 255) / 256
                                                                             : (long long)sm_count() * 16);
    if (image_dtype == VTP_F32 && dtype == VTP_F32)
        im2col_kernel<float, float><<<grid, 256, 0, st>>>((const float*)images, total8, S, P, (float*)cols);
    else if (image_dtype == VTP_F32)
        im2col_kernel<float, bf16><<<grid, 256, 0, st>>>((const float*)images, total8, S, P, (bf16*)cols);
    else if (dtype == VTP_F32)
        im2col_kernel<bf16, float><<<grid, 256, 0, st>>>((const bf16*)images, total8, S, P, (float*)cols);
    else
        im2col_kernel<bf16, bf16><<<grid, 256, 0, st>>>((const bf16*)images, total8, S, P, (bf16*)cols);
    if (int rc = check_launch("im2col")) return rc;
    if (x) {
        VTP_REQUIRE(cls_token && pos_embed && C > 0, VTP_ERR_NULL, "im2col: cls row needs cls_token and pos_embed");
        const int G = S / P;
        const long long row_stride = (long long)(G * G + 1) * C;
        if (dtype == VTP_F32)
            cls_row_kernel<float><<<B, 128, 0, st>>>((const float*)cls_token, (const float*)pos_embed, C,
                                                     row_stride, (float*)x);
        else
            cls_row_kernel<bf16><<<B, 128, 0, st>>>((const bf16*)cls_token, (const bf16*)pos_embed, C, row_stride,
                                                    (bf16*)x);
        return check_launch("cls row");
    }
    return VTP_OK;
}
