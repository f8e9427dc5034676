/*
 * vtpack_b200 — C ABI of the B200 (sm_100a) Dynamic Grained Encoder eval path.
 *
 * Conventions for every entry point
 *   - plain device pointers, explicit sizes, `void* stream` = the caller's cudaStream_t;
 *   - returns int: 0 ok; <0 an invalid argument found on the host before any launch
 *     (VTP_ERR_*); >0 a cudaError_t / CUresult reported by the launch;
 *   - never allocates device memory, never synchronises, never creates streams: the
 *     caller owns every buffer, including worst-case sized scratch (L_max = B*N rows);
 *   - element type is VTP_F32 or VTP_BF16; small per-channel vectors (biases, LayerNorm
 *     weight/bias, gate weights) are always fp32;
 *   - counts that are only known on the device (number of queries L) are read by the
 *     kernels from `offsets[B]`; no entry point copies them to the host unless it says so.
 *
 * Each declaration cites the reference interface it replaces (paths inside the
 * StevenGrove/vtpack tree).  The reference binds these through pybind11
 * (vtpack/layers/csrc/vision.cpp:9-29) with at::Tensor arguments.
 */
#ifndef VTPACK_B200_H
#define VTPACK_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VTP_F32 0
#define VTP_BF16 1

#define VTP_OK 0
#define VTP_ERR_NULL -1        /* required pointer is null */
#define VTP_ERR_SHAPE -2       /* size out of the supported range */
#define VTP_ERR_DTYPE -3       /* unknown element type */
#define VTP_ERR_ALIGN -4       /* pointer or stride not 16-byte aligned */
#define VTP_ERR_UNSUPPORTED -5 /* combination not implemented */
#define VTP_ERR_DRIVER -6      /* driver entry point unavailable */

/* flags for vtp_linear / vtp_sparse_attention / block + model forward */
#define VTP_FLAG_GELU 1u        /* erf GELU on (acc + bias) */
#define VTP_FLAG_OUT_F32 2u     /* write fp32 even when inputs are bf16 */
#define VTP_FLAG_CUDA_CORES 4u  /* bf16 inputs: use the CUDA-core kernel instead of tcgen05 */

/* Library version, 1000*major + minor. */
int vtp_version(void);

/* Text of the last error raised on the calling thread ("" if none). */
const char* vtp_last_error_string(void);

/*
 * Device status word: kernels that wait on mbarriers give up after a bounded time and
 * OR a code into a per-device word instead of hanging.  Reads it back (synchronises the
 * device); `reset` != 0 clears it.  0 = no kernel gave up.
 */
int vtp_device_status(int* value, int reset);

/*
 * Router gate: mean of each region's raw tokens, Linear(C -> n_splits) in fp32, argmax
 * with the lowest index winning ties.
 * Replaces DynamicRouter.forward + gate.argmax (vtpack/layers/dge.py:145-150, :75).
 *   x           [B, num_extra + H*W, C]
 *   gate_w/b    fp32 [n_splits, C] / [n_splits]
 *   logits_out  fp32 [B, H/region, W/region, n_splits] or null
 *   grain_idx   int32 [B, H/region, W/region]
 */
int vtp_router_gate(const void* x, int dtype, int B, int H, int W, int C, int num_extra,
                    int region, const float* gate_w, const float* gate_b, int n_splits,
                    float* logits_out, int32_t* grain_idx, void* stream);

/* argmax over the last axis of fp32 logits [rows, n_splits] (first maximum wins), for
 * teacher-forced gates.  Replaces gate.argmax(dim=-1) (vtpack/layers/dge.py:75). */
int vtp_gate_argmax(const float* logits, int rows, int n_splits, int32_t* grain_idx,
                    void* stream);

/*
 * Patch list from grain indices.
 * Replaces grained_sample_index_to_patch (grained_sample.cu:302-345, kernel :146-196),
 * without its device-to-host copy.
 *   indices     [B, Hr, Wr] int32 (idx_is_i64 = 0) or int64 (1): index into splits
 *   splits      HOST array, n_splits entries (e.g. 4,2,1): sub-patches per region side
 *   counts      int32 [B]     queries per image = num_extra + sum(split^2)
 *   offsets     int32 [B+1]   exclusive prefix of counts; offsets[B] = L
 *   patches     int32 [L_max,4] rows [b, y, x, step]; extra tokens [b, -idx-1, 0, 1]
 *   patches64   int64 [L_max,4] mirror in the reference's dtype, or null
 */
int vtp_index_to_patch(const void* indices, int idx_is_i64, const int* splits, int n_splits,
                       int B, int Hr, int Wr, int region, int num_extra, int32_t* counts,
                       int32_t* offsets, int32_t* patches, int64_t* patches64, void* stream);

/*
 * vtp_router_gate + vtp_index_to_patch in one call that needs no scratch from the caller.
 * It has no counterpart in the reference.  It exists for hosts that can hand over input and
 * output buffers but cannot allocate device memory themselves: a plugin inside an inference
 * server that only receives its tensors, a host runtime in another language whose FFI can
 * pass device pointers but has no CUDA allocator, or a real-time loop where cudaMalloc (which
 * synchronises the device) is off limits.  The grain index of every region and the query
 * count of every image are kept in a fixed array inside the library's device image instead:
 *   - limits: B <= 4096 images and B*(H/region)*(W/region) <= 65536 regions; larger calls
 *     return VTP_ERR_SHAPE and launch nothing;
 *   - the array (278,528 bytes) occupies device memory on every GPU that loads the library
 *     until the process exits;
 *   - the first call on each device looks up the array's device address; make that first
 *     call outside any stream capture;
 *   - all calls share the array and it keeps the last call's contents.  Nothing in it needs
 *     clearing (every entry is written before it is read), but two calls whose kernels can
 *     run at the same time (different streams, different host threads) race on it: order
 *     them on one stream or with events;
 *   - no cudaMalloc / cudaFree or other allocating call is made.
 * Inputs and outputs as in vtp_router_gate / vtp_index_to_patch: x [B, num_extra+H*W, C],
 * gate_w/gate_b fp32, splits a HOST array; offsets int32 [B+1] and patches int32 [L_max,4]
 * (L_max = B*(num_extra+H*W)) are written.
 */
int vtp_gate_compact_static(const void* x, int dtype, int B, int H, int W, int C, int num_extra,
                            int region, const float* gate_w, const float* gate_b,
                            const int* splits, int n_splits, int32_t* offsets, int32_t* patches,
                            void* stream);

/*
 * Multi-grain average pooling, optionally fused with the two LayerNorms that follow it.
 * Replaces grained_sample_compress (grained_sample.cu:198-239, kernel :31-69) and, when
 * ln_w != null, norm1(x) and norm1(q) (vtpack/models/dge/deit_dge.py:127).
 *   x [B,N,C]; patches int32 [L,4]; n_patches_dev -> device int32 holding L (e.g.
 *   offsets + B), or null to use n_patches_max as L.
 *   comp [L_max,C];  xn [B,N,C] = LN(x) or null;  qn [L_max,C] = LN(comp) or null.
 */
int vtp_pool(const void* x, int dtype, int B, int N, int C, int W, int num_extra,
             const int32_t* patches, const int32_t* n_patches_dev, int n_patches_max,
             void* comp, const float* ln_w, const float* ln_b, float eps, void* xn, void* qn,
             void* stream);

/*
 * Replicate-unpool with residual: out[b,tok,:] = q[p,:] - comp[p,:] + ref[b,tok,:] for
 * every token of patch p.  comp may be null (q is already a delta); ref may be null
 * (no residual).  out may alias ref.
 * Replaces DynamicGrainedEncoder.decompress (vtpack/layers/dge.py:87-112) and
 * grained_sample_decompress (grained_sample.cu:241-300, kernels :71-144).
 */
int vtp_unpool_add(const void* q, const void* comp, int dtype, int B, int N, int C, int W,
                   int num_extra, const int32_t* patches, const int32_t* n_patches_dev,
                   int n_patches_max, const void* ref, void* out, void* stream);

/*
 * Gradients of the two movers (training path).  Each is the other mover with another scale:
 *   vtp_pool_grad:   grad_x[b,tok,:] = grad_comp[p,:] / step(p)^2 for every token of patch p
 *                    (backward of grained_sample_compress, vtpack/layers/grained_sample.py:26-38);
 *   vtp_unpool_grad: grad_q[p,:] = sum over the tokens of patch p of grad_out[b,tok,:]
 *                    (backward of grained_sample_decompress with respect to its packed input,
 *                    grained_sample.py:61-72; the gradient with respect to ref_input is grad_out
 *                    itself, :74-77).
 * Shapes as in vtp_pool / vtp_unpool_add.  C may be any positive count for all four movers: rows of
 * whole 16-byte chunks take the vector kernels (16-byte aligned pointers required), other widths
 * (the one-channel gate tensor of vtpack/layers/dge.py:104-110) an element-wise kernel.
 */
int vtp_pool_grad(const void* grad_comp, int dtype, int B, int N, int C, int W, int num_extra,
                  const int32_t* patches, const int32_t* n_patches_dev, int n_patches_max,
                  void* grad_x, void* stream);
int vtp_unpool_grad(const void* grad_out, int dtype, int B, int N, int C, int W, int num_extra,
                    const int32_t* patches, const int32_t* n_patches_dev, int n_patches_max,
                    void* grad_q, void* stream);

/*
 * vtp_unpool_grad for a patch list that was made from grain indices (vtp_index_to_patch), region-parallel:
 * one thread block per region reads the region's region_size^2 rows of grad_out at once and writes the sums
 * of its patches; nothing walks the list.  indices int32 [B, Hr*Wr] (values clamped to the split table),
 * region_first int32 [B*Hr*Wr] = packed row of each region's first patch, offsets int32 [B+1] = packed row
 * of each image's first extra token; grad_out [B, num_extra + Hr*Wr*region_size^2, C], grad_q [n_patches, C]
 * (a region or extra token whose rows would fall outside grad_q is skipped and STATUS_BAD_INDEX set).
 * The sums are taken in fp32 per grid row and then over the rows (the list-walking form adds in (dy, dx)
 * order; the two agree to fp32 rounding).  Region size 4 and a C whose row is 8..192 16-byte chunks in one of
 * the kernel's lane layouts: vtp_region_layout_supported(dtype, C) says whether; otherwise VTP_ERR_SHAPE,
 * and vtp_unpool_grad is the general form.
 */
int vtp_region_layout_supported(int dtype, int C);
int vtp_unpool_grad_regions(const void* grad_out, int dtype, int B, int Hr, int Wr, int region_size, int C,
                            int num_extra, const int32_t* indices, const int* splits, int n_splits,
                            const int32_t* region_first, const int32_t* offsets, int n_patches, void* grad_q,
                            void* stream);

/*
 * Ragged batched matrix product of the training path.  For image i and head h
 *   out_i = op(a_i) * op(b_i),  a_i = a[h, a_offsets[i] : a_offsets[i+1], :],  b_i likewise,
 * op = transpose when the matching flag is non-zero; the out_i are stacked along the row axis: image i
 * starts at row a_offsets[i] (a not transposed) or i*a_cols (a transposed).
 *   a [heads, a_rows, a_cols], b [heads, b_rows, b_cols], out [heads, out_rows, out_cols], dense;
 *   a_offsets / b_offsets device int32 [n_images+1]; max_a_len / max_b_len bound the per-image row
 *   counts (they size the launch); when b is transposed every image must have out_cols rows of b.
 * Replaces batched_sparse_gemm_forward (vtpack/layers/csrc/batched_sparse_gemm/
 * batched_sparse_gemm.cu:150-196), the one native call behind batched_sparse_gemm and its backward
 * (vtpack/layers/sparse_ops.py:11-57).
 */
int vtp_batched_sparse_gemm(const void* a, const void* b, void* out, int dtype, int heads, int n_images,
                            long long a_rows, int a_cols, long long b_rows, int b_cols,
                            const int32_t* a_offsets, const int32_t* b_offsets, int max_a_len,
                            int max_b_len, int a_transposed, int b_transposed, long long out_rows,
                            int out_cols, void* stream);

/*
 * Bilinear-sampling attention of the deformable PVT (vtpack/models/standard/dpvt.py:92-115).
 *   input [B,H,W,C] feature map; grid [B,G,P,2] sampling points in pixel coordinates (x, y);
 *   a sample is the bilinear interpolation of the map at the point, zero outside the map.
 *   mode 0 ("point"):   weight [B,G,P], out [B,G,C] = sum_p weight * sample;
 *   mode 1 ("channel"): weight [B,G,C], out [B,G,P] = sum_c weight * sample.
 * All tensors dense and of the one dtype.  The backward call writes grad_input [B,H,W,C] (cleared
 * on the stream first, then accumulated with atomics), grad_grid [B,G,P,2] and grad_weight (shape of
 * weight); it needs C <= 256.
 * Replace bilinear_attention_{pointwise,channelwise}_{forward,backward}
 * (vtpack/layers/csrc/bilinear_attention/bilinear_attention.cu:364-536, kernels :88-362).
 */
int vtp_bilinear_attention_forward(const void* input, const void* grid, const void* weight, void* out,
                                   int dtype, int mode, int B, int H, int W, int C, int G, int P,
                                   void* stream);
int vtp_bilinear_attention_backward(const void* grad_out, const void* input, const void* grid,
                                    const void* weight, void* grad_input, void* grad_grid,
                                    void* grad_weight, int dtype, int mode, int B, int H, int W, int C,
                                    int G, int P, void* stream);

/*
 * Point-mode bilinear attention over PACKED queries (the variable-length layout of the DGE path):
 *   grid [L,P,2], weight [L,P], batches int64 [L] = the image each query samples, out [L,C].
 * A query whose image index is outside [0, B) reads zeros.
 * Replaces sparse_bilinear_attention_pointwise_forward
 * (vtpack/layers/csrc/sparse_bilinear_attention/sparse_bilinear_attention.cu:88-171; forward only
 * in the reference as well).
 */
int vtp_sparse_bilinear_attention_forward(const void* input, const void* grid, const void* weight,
                                          const long long* batches, void* out, int dtype, int B, int H,
                                          int W, int C, int L, int P, void* stream);

/*
 * LayerNorm over the last axis.  Row r of the input starts at x + r*in_row_stride
 * elements; output rows are dense.  rows_dev (device int32) overrides rows_max when set.
 * Replaces nn.LayerNorm norm2 / norm (vtpack/models/dge/deit_dge.py:128, :277).
 */
int vtp_layernorm(const void* x, int dtype, int rows_max, const int32_t* rows_dev, int C,
                  long long in_row_stride, const float* w, const float* b, float eps, void* y,
                  void* stream);

/*
 * LayerNorm and a row-wise add in one pass: out[orow(r)] = LN(x[r]) + addend[r % a_mod + a_off] with
 * orow(r) = (r / out_grp) * out_stride + out_off + r % out_grp, for r < rows (the row maps are those of
 * vtp_add_rows).  One rounding of the sum instead of two.  Replaces a stage embedding's norm followed by
 * the position-embedding add, written behind the cls slot in the last stage
 * (vtpack/models/dge/pvt_dge.py:177, 307-316).
 */
int vtp_layernorm_add_rows(const void* x, int dtype, int rows, int C, long long in_row_stride, const float* w,
                           const float* b, float eps, const void* addend, int a_mod, int a_off, void* out,
                           int out_grp, int out_stride, int out_off, void* stream);

/*
 * y[m, n] = act(sum_k a[m,k] * w[n,k] + bias[n]) + residual[m,n]
 * a [M,K] (row stride lda elements), w [N,K] dense, bias fp32 [N] or null,
 * residual [M,N] (row stride ldr) or null, y [M,N] (row stride ldy).
 * m_dev (device int32) overrides m_max when set.  bf16 inputs run on tcgen05 tensor
 * cores (K % 64 == 0, 16-byte aligned rows); fp32 inputs on CUDA cores.
 * Replaces nn.Linear q/kv/proj/fc1/fc2/head (vtpack/models/dge/deit_dge.py:27-29,55-58,216)
 * with the GELU (:40) and the residual adds (:127-128) as epilogues.
 */
int vtp_linear(const void* a, long long lda, const void* w, const float* bias,
               const void* residual, long long ldr, void* y, long long ldy, int dtype,
               int m_max, const int32_t* m_dev, int N, int K, unsigned flags, void* stream);

/*
 * Weight preparation for a Linear that follows a LayerNorm (run once per model):
 *   w_out[n,k] = W[n,k]*gamma[k] (rounded to dtype), s[n] = sum_k w_out[n,k],
 *   c[n] = sum_k beta[k]*W[n,k] + bias[n]   (bias may be null).
 * Then LN(x) W^T + b = rstd*(x w_out^T - mean*s) + c, which is what the block forward
 * evaluates when vtp_block_weights carries the folded fields.  The reference keeps
 * nn.LayerNorm and nn.Linear separate (vtpack/models/dge/deit_dge.py:127-128).
 */
int vtp_fold_layernorm(const void* w, int dtype, int N, int K, const float* gamma,
                       const float* beta, const float* bias, void* w_out, float* s_out,
                       float* c_out, void* stream);

/*
 * Variable-length-query attention: for image i, head h,
 *   out[rows of i] = softmax(scale * Q_i K_i^T) V_i   over all n_keys keys.
 * q/out rows are the packed queries (offsets[i] .. offsets[i+1]); strides are in
 * elements; the head dim is contiguous.  Accepts the Linear outputs in place:
 * q [L, h*d] -> q_row_stride = h*d, q_head_stride = d;  kv [B, N, 2, h, d] ->
 * k = kv, v = kv + h*d, kv_batch_stride = N*2*h*d, kv_row_stride = 2*h*d.
 * offsets int32 [B+1] (device): first packed row of each image; l_max rows are allocated
 * in q/out; max_q_per_image bounds the queries of any one image (it sizes the grid).
 * Replaces batched_sparse_attention_forward (batched_sparse_gemm.cu:219-305) and the
 * .contiguous() copies in front of it (vtpack/layers/sparse_ops.py:60-78).
 */
int vtp_sparse_attention(const void* q, long long q_row_stride, long long q_head_stride,
                         const void* k, const void* v, long long kv_batch_stride,
                         long long kv_row_stride, long long kv_head_stride, void* out,
                         long long o_row_stride, long long o_head_stride, int dtype, int B,
                         int n_keys, int heads, int head_dim, const int32_t* offsets,
                         int l_max, int max_q_per_image, float scale, unsigned flags,
                         void* stream);

/*
 * Patch embedding front end: images [B,3,S,S] (fp32 or bf16, image_dtype) -> im2col rows [B*(S/P)^2, 3*P*P] in
 * `dtype` (column = c*P*P + py*P + px, the flattening of the conv weight), and writes the
 * cls row x[b,0,:] = cls_token + pos_embed[0].  The GEMM itself is vtp_linear.
 * Replaces PatchEmbed + cls/pos add (vtpack/models/dge/deit_dge.py:268-275).
 */
int vtp_patch_im2col(const void* images, int image_dtype, int B, int S, int P, int dtype, void* cols,
                     const void* cls_token, const void* pos_embed, int C, void* x,
                     void* stream);

/*
 * The same im2col for patches that are not multiples of 8 pixels (PVT+DGE's 4 x 4 first stage,
 * vtpack/models/dge/pvt_dge.py:160-179), with rows `ld_cols` elements apart (a multiple of 8, at least
 * 3*P*P) and the tail of every row zeroed: 48 columns padded to 64 make the reduction a whole 64-element
 * block, so the patch-embedding GEMM runs on the tensor-core vtp_linear with K = ld_cols and the conv
 * weight [C, 3*P*P] padded with zero columns.  No cls row.
 */
int vtp_patch_im2col_padded(const void* images, int image_dtype, int B, int S, int P, int dtype, void* cols,
                            int ld_cols, void* stream);

/*
 * Stride-`ratio` window gather on a token grid: x [B, H*W, C] -> cols [B*(H/ratio)*(W/ratio), ratio*ratio*C],
 * column (dy, dx, c).  With vtp_linear it is a convolution of kernel = stride = ratio whose weight
 * [C_out, C_in, ratio, ratio] was reordered once to [C_out, (dy, dx, c_in)]: the spatial reduction of a
 * PVT block (vtpack/models/dge/pvt_dge.py:82-83) and the patch embedding between PVT stages
 * (PatchEmbed, pvt_dge.py:149-179; there the tokens stand for the [B, C, H, W] map of pvt_dge.py:315).
 */
int vtp_token_im2col(const void* x, int dtype, int B, int H, int W, int C, int ratio, void* cols, void* stream);

/*
 * out[orow(r), :] = x[r % x_mod, :] + addend[r % a_mod + a_off, :] for r < rows, with
 * orow(r) = (r / out_grp) * out_stride + out_off + r % out_grp.  The position-embedding add of a stage
 * (x_mod = rows, a_mod = tokens per image) and, with x_mod = a_mod = out_grp = 1, the cls rows that go in
 * front of each image's tokens (pvt_dge.py:306-313; deit_dge.py:271-275).
 */
int vtp_add_rows(const void* x, int x_mod, const void* addend, int a_mod, int a_off, void* out, int out_grp,
                 int out_stride, int out_off, int dtype, long long rows, int C, void* stream);

/* Pointers to one block's parameters (device memory).  Matrices are in the model dtype,
 * vectors fp32.  Keys are the reference's state_dict names below blocks.{i}. */
typedef struct {
    const float* norm1_w; const float* norm1_b;
    const void* q_w; const float* q_b;          /* attn.q    [C, C]  */
    const void* kv_w; const float* kv_b;        /* attn.kv   [2C, C] */
    const void* proj_w; const float* proj_b;    /* attn.proj [C, C]  */
    const float* norm2_w; const float* norm2_b;
    const void* fc1_w; const float* fc1_b;      /* mlp.fc1   [hidden, C] */
    const void* fc2_w; const float* fc2_b;      /* mlp.fc2   [C, hidden] */
    const float* gate_w; const float* gate_b;   /* dge.router.gate [n_splits, C] fp32 */
    /* Optional (bf16 tensor-core path): the three Linears that follow a LayerNorm with the
     * LayerNorm folded in by vtp_fold_layernorm (norm1 -> q, norm1 -> kv, norm2 -> fc1).
     * *_wf = W*diag(gamma) in the model dtype, *_s / *_c fp32 [out features].  When all nine
     * are set the block never materialises normalised rows: its GEMMs read raw rows and apply
     * rstd*(acc - mean*s) + c in their epilogues.  Leave null to run explicit LayerNorms. */
    const void* q_wf; const float* q_s; const float* q_c;
    const void* kv_wf; const float* kv_s; const float* kv_c;
    const void* fc1_wf; const float* fc1_s; const float* fc1_c;
    /* PVT+DGE blocks (shape sr_ratio > 1; vtpack/models/dge/pvt_dge.py:59-63,81-85): keys and values
     * come from the normed tokens reduced by a stride-sr convolution and a LayerNorm.
     * sr_w = attn.sr.weight as a matrix [C, sr*sr*C] in the model dtype with columns ordered
     * (dy, dx, c_in), i.e. weight.permute(0, 2, 3, 1).reshape(C, -1); sr_b = attn.sr.bias;
     * sr_norm_* = attn.norm (its epsilon is the shape's sr_eps, 1e-5 in the reference). */
    const void* sr_w; const float* sr_b; const float* sr_norm_w; const float* sr_norm_b;
} vtp_block_weights;

/* Shapes shared by the block and model entry points. */
typedef struct {
    int dtype;       /* VTP_F32 / VTP_BF16 */
    int B, H, W;     /* images, token grid */
    int num_extra;   /* cls tokens in front of the grid (1) */
    int C, heads, hidden;
    int region;      /* tokens per region side (4) */
    int n_splits;    /* entries of splits */
    int splits[8];   /* sub-patches per region side, e.g. 4,2,1 */
    float eps;       /* LayerNorm epsilon */
    unsigned flags;  /* VTP_FLAG_CUDA_CORES */
    int sr_ratio;    /* 0 or 1: keys = tokens (DeiT).  > 1: PVT spatial reduction, needs num_extra = 0,
                        H and W multiples of it; the block then has H*W/sr^2 keys per image */
    float sr_eps;    /* epsilon of the LayerNorm after the reduction */
    float attn_scale; /* softmax scale of the attention (Attention.scale = qk_scale or head_dim^-0.5,
                         vtpack/models/dge/deit_dge.py:52-53); 0 selects head_dim^-0.5 */
} vtp_dge_shape;

/* Scratch bytes vtp_dge_block_forward needs for this shape (16-byte aligned slices). */
long long vtp_block_workspace_bytes(const vtp_dge_shape* s);

/*
 * Eval forward of one DeiT+DGE block, x_in [B,N,C] -> x_out [B,N,C] (may alias).
 * forced_logits (fp32 [B,Hr,Wr,n_splits]) replaces the router output when non-null.
 * counts_out (int32 [B], optional) receives the per-image query counts.
 * Replaces Block.forward (vtpack/models/dge/deit_dge.py:123-130).
 */
int vtp_dge_block_forward(const vtp_dge_shape* s, const vtp_block_weights* w, const void* x_in,
                          void* x_out, const float* forced_logits, int32_t* counts_out,
                          void* workspace, long long workspace_bytes, void* stream);

/*
 * Eval forward of n_blocks consecutive DGE blocks of ONE shape, w[0 .. n_blocks-1]: a stage of the pyramid
 * model (the `for blk in block: x = blk(x, H, W)` loop, vtpack/models/dge/pvt_dge.py:318-319) or any run
 * of DeiT+DGE blocks (vtpack/models/dge/deit_dge.py:291-292).  x_in [B,N,C] -> x_out [B,N,C] (may alias);
 * blocks after the first work on x_out in place.  Same results as n_blocks calls of
 * vtp_dge_block_forward; where two neighbours both run with folded LayerNorms, the first one's unpool
 * also leaves the second one's token statistics, router decisions and per-image counts, so the second
 * starts at its pooling.  counts_out (int32 [n_blocks, B], optional) receives the per-image query
 * counts of every block.  The workspace is one block's (vtp_block_workspace_bytes).
 */
int vtp_dge_blocks_forward(const vtp_dge_shape* s, const vtp_block_weights* w, int n_blocks,
                           const void* x_in, void* x_out, int32_t* counts_out, void* workspace,
                           long long workspace_bytes, void* stream);

/*
 * Same as vtp_dge_block_forward, and records events[i] (cudaEvent_t created by the caller,
 * null entries skipped) on the stream after stage i:
 *   0 start, 1 router gate, 2 patch list, 3 pool+LN1, 4 q proj, 5 kv proj, 6 attention,
 *   7 out proj+residual, 8 LN2, 9 fc1+GELU, 10 fc2+residual, 11 unpool+residual.
 * For per-kernel timing; the reference has no counterpart (it logs wall-clock time per
 * iteration only, vtpack/engine/utils.py:128-172).
 */
#define VTP_BLOCK_STAGES 12
int vtp_dge_block_forward_timed(const vtp_dge_shape* s, const vtp_block_weights* w,
                                const void* x_in, void* x_out, const float* forced_logits,
                                int32_t* counts_out, void* workspace, long long workspace_bytes,
                                void* const* events, int n_events, void* stream);

/* Dense DeiT block from the same weights (q and kv applied to every token), the
 * comparison baseline.  Replaces Block.forward of vtpack/models/standard/deit.py:79-83. */
int vtp_dense_block_forward(const vtp_dge_shape* s, const vtp_block_weights* w, const void* x_in,
                            void* x_out, void* workspace, long long workspace_bytes,
                            void* stream);

/* Model-level parameters outside the blocks. */
typedef struct {
    const void* patch_w; const float* patch_b;  /* patch_embed.proj [C, 3*P*P] */
    const void* cls_token;                      /* [C]    model dtype */
    const void* pos_embed;                      /* [N, C] model dtype */
    const float* norm_w; const float* norm_b;
    const void* head_w; const float* head_b;    /* head [classes, C] */
    int depth, patch, img_size, num_classes;
    int image_dtype;                            /* VTP_F32 or VTP_BF16: element type of the images */
} vtp_model_weights;

long long vtp_model_workspace_bytes(const vtp_dge_shape* s, const vtp_model_weights* m);

/*
 * Eval forward of DeiT+DGE: images [B,3,S,S] (device; fp32, or bf16 when
 * m->image_dtype = VTP_BF16) -> logits fp32 [B,classes].
 * counts_out int32 [depth,B] optional.
 * Replaces VisionTransformer.forward (vtpack/models/dge/deit_dge.py:267-299).
 */
int vtp_deit_dge_forward(const vtp_dge_shape* s, const vtp_model_weights* m,
                         const vtp_block_weights* blocks, const void* images, float* logits,
                         int32_t* counts_out, void* workspace, long long workspace_bytes,
                         void* stream);

/* Optional inputs and outputs of vtp_deit_dge_forward_ex; every pointer may be null. */
typedef struct {
    /* fp32 [B, n_splits], added to the router logits of every region of image b in every block before the
     * argmax.  Large offsets force an image to one grain whatever its content: the measurement
     * configuration with half the images all-coarse and half all-fine is set up this way.  The reference
     * has one gate bias per grain for all images (vtpack/layers/dge.py:125). */
    const float* gate_image_bias;
    /* model dtype [depth, B, N, C]: the tokens each block received (block 0: patch embedding + position) */
    void* tokens_trace;
    /* int32 [depth, B, (H/region)*(W/region)]: the grain index each block's gate chose per region */
    int32_t* grain_trace;
} vtp_forward_options;

/*
 * vtp_deit_dge_forward with the options above (opt may be null).  The traces let a test feed the
 * reference's router (vtpack/layers/dge.py:61-76,145-150) the very activations the device gate saw and
 * compare decisions layer by layer; they cost one device-to-device copy per block.
 */
int vtp_deit_dge_forward_ex(const vtp_dge_shape* s, const vtp_model_weights* m,
                            const vtp_block_weights* blocks, const void* images, float* logits,
                            int32_t* counts_out, const vtp_forward_options* opt, void* workspace,
                            long long workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VTPACK_B200_H */
