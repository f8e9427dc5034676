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

// Patches narrower than 8 pixels (PVT's first stage: 4 x 4): one thread moves 4 adjacent pixels, one vector
// load and one vector store.  Rows of `cols` are `ld` elements apart; the thread that moves a patch's first
// pixels also zeroes the row's tail beyond 3 * P * P (ld > 3 * P * P pads the reduction for the tensor-core GEMM).
__device__ __forceinline__ void load4(const float* p, float* f) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(p));
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
__device__ __forceinline__ void load4(const bf16* p, float* f) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float* f) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    uint2 v;
    v.x = *reinterpret_cast<const uint32_t*>(&a);
    v.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = v;
}
// (IDX: unsigned when every element index fits 32 bits — the index arithmetic is most of this kernel's
// instructions, and 64-bit divisions cost several times the 32-bit ones — else long long)
template <typename I, typename T, typename IDX>
__global__ void __launch_bounds__(256)
im2col4_kernel(const I* __restrict__ img, long long total4, int S, int P, T* __restrict__ cols, int ld) {
    const int G = S / P;
    const int KP = 3 * P * P;
    const IDX uS = (IDX)S, plane = (IDX)S * (IDX)S;
    for (IDX e = (IDX)blockIdx.x * blockDim.x + threadIdx.x; e < (IDX)total4; e += (IDX)gridDim.x * blockDim.x) {
        const IDX pix = e * 4;
        const int ix = (int)(pix % uS);
        const int iy = (int)((pix / uS) % uS);
        const int c = (int)((pix / plane) % 3);
        const long long b = (long long)(pix / (plane * 3));
        float f[4];
        load4(img + pix, f);
        const int gy = iy / P, py = iy % P, gx = ix / P, px = ix % P;
        T* row = cols + ((b * G + gy) * G + gx) * (long long)ld;
        store4(row + c * P * P + py * P + px, f);
        if (c == 0 && py == 0 && px == 0) {
            const float z[4] = {0.f, 0.f, 0.f, 0.f};
            for (int t = KP; t < ld; t += 4) store4(row + t, z);
        }
    }
}

// 4 x 4 patches, one CTA per (image, patch row): the twelve image rows (3 channels x 4) of the patch row are
// read as whole rows, scattered into a shared-memory copy of the S/4 output rows, and those leave as one
// contiguous range of 16-byte stores (the direct kernel above writes 8-byte pieces 96 or 128 bytes apart).
template <typename I, typename T>
__global__ void __launch_bounds__(256)
im2col_p4_kernel(const I* __restrict__ img, int S, T* __restrict__ cols, int ld) {
    constexpr int P = 4, KP = 48, VT = 16 / (int)sizeof(T);     // VT: elements of a 16-byte store
    extern __shared__ __align__(16) unsigned char tile_raw[];
    T* tile = reinterpret_cast<T*>(tile_raw);
    const int G = S / P, pitch = ld + VT;                        // one store of padding per row spreads the banks
    const int b = blockIdx.x / G, gy = blockIdx.x % G;
    const int per_row = S / 4;
    // tails beyond the 48 columns
    for (int i = threadIdx.x; i < G * ((ld - KP) / 4); i += blockDim.x) {
        const float z[4] = {0.f, 0.f, 0.f, 0.f};
        store4(tile + (i / ((ld - KP) / 4)) * pitch + KP + (i % ((ld - KP) / 4)) * 4, z);
    }
    for (int v = threadIdx.x; v < 12 * per_row; v += blockDim.x) {
        const int r = v / per_row, gx = v % per_row;             // r = c * 4 + py; four pixels = the patch's row
        const int c = r >> 2, py = r & 3;
        float f[4];
        load4(img + (((size_t)b * 3 + c) * S + (size_t)gy * P + py) * S + (size_t)gx * 4, f);
        store4(tile + gx * pitch + r * 4, f);
    }
    __syncthreads();
    const int vec_per_row = ld / VT;
    T* out = cols + ((size_t)b * G + gy) * G * (size_t)ld;
    for (int v = threadIdx.x; v < G * vec_per_row; v += blockDim.x) {
        const int row = v / vec_per_row, i = v % vec_per_row;
        *reinterpret_cast<uint4*>(out + (size_t)row * ld + i * VT) = *reinterpret_cast<const uint4*>(tile + row * pitch + i * VT);
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
template <typename T, typename IDX>
__global__ void __launch_bounds__(256)
token_im2col_kernel(const T* __restrict__ x, long long total_vec, int H, int W, int C, int sr, T* __restrict__ cols,
                    const float2* __restrict__ stats, const float* __restrict__ lnw, const float* __restrict__ lnb) {
    // stats != null: the rows gathered are LayerNorm(x), normalised on the way from each token's (mean, rstd)
    // (IDX: unsigned when the vector count fits 32 bits, see im2col4_kernel)
    constexpr int VN = Vec<T>::N;
    const int run = sr * C / VN;                  // 16-byte vectors per window row
    const int Wo = W / sr, Ho = H / sr;
    for (IDX v = (IDX)blockIdx.x * blockDim.x + threadIdx.x; v < (IDX)total_vec; v += (IDX)gridDim.x * blockDim.x) {
        const int i = (int)(v % (IDX)run);
        IDX r = v / (IDX)run;                     // (b, oy, ox, dy) with dy fastest
        const int dy = (int)(r % (IDX)sr); r /= (IDX)sr;
        const int ox = (int)(r % (IDX)Wo); r /= (IDX)Wo;
        const int oy = (int)(r % (IDX)Ho);
        const long long b = (long long)(r / (IDX)Ho);
        const long long tok = (b * H + (long long)oy * sr + dy) * W + (long long)ox * sr;
        Vec<T> t;
        t.load(x + tok * C + (long long)i * VN);
        if (stats) {
            const int e0 = i * VN;                        // element of the window row: token e0 / C, channel e0 % C
            const float2 ms = stats[tok + e0 / C];
            const int ch = e0 % C;
            float f[VN], gw[VN], gb[VN];
            t.to_float(f);
#pragma unroll
            for (int k4 = 0; k4 < VN / 4; ++k4) {          // ch is a multiple of VN: 16-byte loads of the LayerNorm vectors
                const float4 w4 = __ldg(reinterpret_cast<const float4*>(lnw + ch) + k4);
                const float4 b4 = __ldg(reinterpret_cast<const float4*>(lnb + ch) + k4);
                gw[4 * k4] = w4.x; gw[4 * k4 + 1] = w4.y; gw[4 * k4 + 2] = w4.z; gw[4 * k4 + 3] = w4.w;
                gb[4 * k4] = b4.x; gb[4 * k4 + 1] = b4.y; gb[4 * k4 + 2] = b4.z; gb[4 * k4 + 3] = b4.w;
            }
#pragma unroll
            for (int k = 0; k < VN; ++k) f[k] = (f[k] - ms.x) * ms.y * gw[k] + gb[k];
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
    const bool small = total < (1ll << 31);
    if (dtype == VTP_BF16) {
        if (small) token_im2col_kernel<bf16, unsigned><<<grid, 256, 0, st>>>((const bf16*)x, total, H, W, C, sr, (bf16*)cols, stats, lnw, lnb);
        else token_im2col_kernel<bf16, long long><<<grid, 256, 0, st>>>((const bf16*)x, total, H, W, C, sr, (bf16*)cols, stats, lnw, lnb);
    } else {
        if (small) token_im2col_kernel<float, unsigned><<<grid, 256, 0, st>>>((const float*)x, total, H, W, C, sr, (float*)cols, stats, lnw, lnb);
        else token_im2col_kernel<float, long long><<<grid, 256, 0, st>>>((const float*)x, total, H, W, C, sr, (float*)cols, stats, lnw, lnb);
    }
    return check_launch("spatial reduction im2col");
}

// out[orow(r)] = x[r % x_mod] + addend[r % a_mod + a_off], orow(r) = (r / out_grp) * out_stride + out_off + r % out_grp:
// the position-embedding add of a token stage, and (x_mod = a_mod = out_grp = 1) the cls rows put in front of it.
template <typename T, typename IDX>
__global__ void __launch_bounds__(256)
add_rows_kernel(const T* __restrict__ x, int x_mod, const T* __restrict__ addend, int a_mod, int a_off,
                T* __restrict__ out, int out_grp, int out_stride, int out_off, long long total_vec, int C) {
    // (IDX: unsigned when the vector count fits 32 bits, see im2col4_kernel)
    constexpr int VN = Vec<T>::N;
    const int cv = C / VN;
    for (IDX v = (IDX)blockIdx.x * blockDim.x + threadIdx.x; v < (IDX)total_vec; v += (IDX)gridDim.x * blockDim.x) {
        const IDX r = v / (IDX)cv;
        const int i = (int)(v % (IDX)cv) * VN;
        Vec<T> a, p;
        float fa[VN], fp[VN];
        a.load(x + (long long)(r % (IDX)x_mod) * C + i);
        p.load(addend + ((long long)(r % (IDX)a_mod) + a_off) * C + i);
        a.to_float(fa);
        p.to_float(fp);
#pragma unroll
        for (int k = 0; k < VN; ++k) fa[k] += fp[k];
        a.from_float(fa);
        a.store(out + ((long long)(r / (IDX)out_grp) * out_stride + out_off + (long long)(r % (IDX)out_grp)) * C + i);
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
    const bool small = total < (1ll << 31);
#define VTP_ADD_ROWS(T, IDX)                                                                                  \
    add_rows_kernel<T, IDX><<<grid, 256, 0, st>>>((const T*)x, x_mod, (const T*)addend, a_mod, a_off, (T*)out, \
                                                  out_grp, out_stride, out_off, total, C)
    if (dtype == VTP_BF16) { if (small) VTP_ADD_ROWS(bf16, unsigned); else VTP_ADD_ROWS(bf16, long long); }
    else { if (small) VTP_ADD_ROWS(float, unsigned); else VTP_ADD_ROWS(float, long long); }
#undef VTP_ADD_ROWS
    return check_launch("add rows");
}

static int patch_im2col(const void* images, int image_dtype, int B, int S, int P, int dtype, void* cols, int ld,
                        const void* cls_token, const void* pos_embed, int C, void* x, void* stream);

extern "C" int vtp_patch_im2col(const void* images, int image_dtype, int B, int S, int P, int dtype, void* cols,
                                const void* cls_token, const void* pos_embed, int C, void* x, void* stream) {
    return patch_im2col(images, image_dtype, B, S, P, dtype, cols, 3 * P * P, cls_token, pos_embed, C, x, stream);
}

extern "C" int vtp_patch_im2col_padded(const void* images, int image_dtype, int B, int S, int P, int dtype, void* cols,
                                       int ld_cols, void* stream) {
    VTP_REQUIRE(P > 0 && P % 8 != 0, VTP_ERR_UNSUPPORTED,
                "im2col (padded rows): for patches that are not multiples of 8 pixels; others need no padding");
    VTP_REQUIRE(ld_cols >= 3 * P * P && ld_cols % 8 == 0, VTP_ERR_SHAPE,
                "im2col (padded rows): row pitch %d for %d columns (a multiple of 8, at least the columns)", ld_cols,
                3 * P * P);
    return patch_im2col(images, image_dtype, B, S, P, dtype, cols, ld_cols, nullptr, nullptr, 0, nullptr, stream);
}

static int patch_im2col(const void* images, int image_dtype, int B, int S, int P, int dtype, void* cols, int ld,
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
        const size_t p4_smem = (size_t)(S / 4) * (ld + 16 / elem_size(dtype)) * elem_size(dtype);
        if (P == 4 && ld % (16 / (int)elem_size(dtype)) == 0 && p4_smem <= 48 * 1024) {
            const int grid = B * (S / 4);
            if (image_dtype == VTP_F32 && dtype == VTP_F32)
                im2col_p4_kernel<float, float><<<grid, 256, p4_smem, st>>>((const float*)images, S, (float*)cols, ld);
            else if (image_dtype == VTP_F32)
                im2col_p4_kernel<float, bf16><<<grid, 256, p4_smem, st>>>((const float*)images, S, (bf16*)cols, ld);
            else if (dtype == VTP_F32)
                im2col_p4_kernel<bf16, float><<<grid, 256, p4_smem, st>>>((const bf16*)images, S, (float*)cols, ld);
            else
                im2col_p4_kernel<bf16, bf16><<<grid, 256, p4_smem, st>>>((const bf16*)images, S, (bf16*)cols, ld);
            return check_launch("im2col");
        }
        // 32-bit indices when the pixel count and the padded output both fit
        const bool small = (long long)B * 3 * S * S < (1ll << 31) && (long long)B * (S / P) * (S / P) * ld < (1ll << 31);
#define VTP_IM2COL4(I, T, ARGS)                                                              \
    do {                                                                                     \
        if (small) im2col4_kernel<I, T, unsigned><<<g4, 256, 0, st>>> ARGS;                   \
        else im2col4_kernel<I, T, long long><<<g4, 256, 0, st>>> ARGS;                        \
    } while (0)
        if (image_dtype == VTP_F32 && dtype == VTP_F32)
            VTP_IM2COL4(float, float, ((const float*)images, total4, S, P, (float*)cols, ld));
        else if (image_dtype == VTP_F32)
            VTP_IM2COL4(float, bf16, ((const float*)images, total4, S, P, (bf16*)cols, ld));
        else if (dtype == VTP_F32)
            VTP_IM2COL4(bf16, float, ((const bf16*)images, total4, S, P, (float*)cols, ld));
        else
            VTP_IM2COL4(bf16, bf16, ((const bf16*)images, total4, S, P, (bf16*)cols, ld));
#undef VTP_IM2COL4
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
