// Whole-block and whole-model eval forwards: the host-side sequencing of the kernels on
// one stream, with every intermediate in a caller-provided workspace and every
// data-dependent size (the number of packed queries L) left on the device.
//
// Replaces Block.forward and VisionTransformer.forward
// (vtpack/models/dge/deit_dge.py:123-130, 267-299) and, for the comparison baseline,
// Block.forward of vtpack/models/standard/deit.py:79-83.
#include "attention.h"
#include "linear.h"
#include "region_ops.h"

namespace vtp {

int token_im2col(const void* x, int dtype, int B, int H, int W, int C, int sr, void* cols, cudaStream_t st,
                 const float2* stats = nullptr, const float* lnw = nullptr, const float* lnb = nullptr);  // patch_embed.cu

struct Carver {
    char* base;
    long long off = 0;
    explicit Carver(void* p) : base(static_cast<char*>(p)) {}
    void* take(long long bytes) {
        void* r = base ? base + off : nullptr;
        off += round_up(bytes, 256);
        return r;
    }
};

struct BlockScratch {
    int32_t *idx[2], *counts[2], *offsets, *patches, *region_first; // idx / counts / logits / stats_x: this block's and the
    float* logits[2];                                              // next block's (written by this block's unpool)
    float2 *stats_x[2], *stats_q, *stats_acc;
    void *comp, *xn, *qn, *qp, *kv, *ao, *q1, *hid;
    void *sr_cols, *sr_out, *sr_norm;       // spatial reduction (PVT blocks): im2col rows, reduced tokens, their LayerNorm
    long long bytes;
};

// keys per image: the tokens, or the grid reduced by sr_ratio in each direction
static int keys_per_image(const vtp_dge_shape& s) {
    return s.sr_ratio > 1 ? (s.H / s.sr_ratio) * (s.W / s.sr_ratio) : s.num_extra + s.H * s.W;
}

static BlockScratch carve_block(const vtp_dge_shape& s, void* ws) {
    const long long e = (long long)elem_size(s.dtype);
    const int N = s.num_extra + s.H * s.W;
    const long long rows = (long long)s.B * N;            // worst case: every region at the finest grain
    const int R = (s.H / s.region) * (s.W / s.region);
    Carver c(ws);
    BlockScratch b;
    b.idx[0] = (int32_t*)c.take((long long)s.B * R * 4);
    b.idx[1] = (int32_t*)c.take((long long)s.B * R * 4);
    b.counts[0] = (int32_t*)c.take((long long)s.B * 4);
    b.counts[1] = (int32_t*)c.take((long long)s.B * 4);
    b.offsets = (int32_t*)c.take((long long)(s.B + 1) * 4);
    b.patches = (int32_t*)c.take(rows * 16);
    b.region_first = (int32_t*)c.take((long long)s.B * R * 4);
    b.logits[0] = (float*)c.take((long long)s.B * R * s.n_splits * 4);
    b.logits[1] = (float*)c.take((long long)s.B * R * s.n_splits * 4);
    b.stats_x[0] = (float2*)c.take(rows * 8);
    b.stats_x[1] = (float2*)c.take(rows * 8);
    b.stats_q = (float2*)c.take(rows * 8);
    b.stats_acc = (float2*)c.take(rows * 8 * STAT_SLOTS);
    b.comp = c.take(rows * s.C * e);
    b.xn = c.take(rows * s.C * e);
    b.qn = c.take(rows * s.C * e);
    b.qp = c.take(rows * s.C * e);
    b.kv = c.take(rows * 2 * s.C * e);
    b.ao = c.take(rows * s.C * e);
    b.q1 = c.take(rows * s.C * e);
    b.hid = c.take(rows * s.hidden * e);
    b.sr_cols = b.sr_out = b.sr_norm = nullptr;
    if (s.sr_ratio > 1) {
        const long long krows = (long long)s.B * keys_per_image(s);
        b.sr_cols = c.take(rows * s.C * e);             // [B*keys, sr*sr*C] = as many elements as the tokens
        b.sr_out = c.take(krows * s.C * e);
        b.sr_norm = c.take(krows * s.C * e);
    }
    b.bytes = c.off;
    return b;
}

static int check_shape(const vtp_dge_shape* s) {
    VTP_REQUIRE(s, VTP_ERR_NULL, "block: null shape");
    VTP_REQUIRE(s->dtype == VTP_F32 || s->dtype == VTP_BF16, VTP_ERR_DTYPE, "block: dtype %d", s->dtype);
    VTP_REQUIRE(s->B > 0 && s->H > 0 && s->W > 0 && s->C > 0 && s->heads > 0 && s->hidden > 0 && s->num_extra >= 0,
                VTP_ERR_SHAPE, "block: bad shape");
    VTP_REQUIRE(s->C % s->heads == 0, VTP_ERR_SHAPE, "block: C=%d not divisible by %d heads", s->C, s->heads);
    VTP_REQUIRE(s->region > 0 && s->H % s->region == 0 && s->W % s->region == 0, VTP_ERR_SHAPE,
                "block: grid %dx%d not divisible by region %d", s->H, s->W, s->region);
    VTP_REQUIRE(s->n_splits >= 1 && s->n_splits <= 8, VTP_ERR_SHAPE, "block: n_splits %d", s->n_splits);
    VTP_REQUIRE((long long)s->B * (s->num_extra + s->H * s->W) < (1ll << 30), VTP_ERR_SHAPE, "block: too many tokens");
    if (s->sr_ratio > 1) {
        // the reference reshapes the tokens to [B, C, H, W] before the reduction (pvt_dge.py:82)
        VTP_REQUIRE(s->num_extra == 0, VTP_ERR_SHAPE, "block: spatial reduction needs a grid without extra tokens");
        VTP_REQUIRE(s->H % s->sr_ratio == 0 && s->W % s->sr_ratio == 0, VTP_ERR_SHAPE,
                    "block: grid %dx%d not divisible by the reduction ratio %d", s->H, s->W, s->sr_ratio);
    }
    return VTP_OK;
}

// Records events[i] on the stream after stage i when the caller asked for stage timing.
struct StageMarks {
    void* const* events = nullptr;
    int n = 0;
    cudaStream_t st = nullptr;
    int mark(int i) const {
        if (!events || i >= n || !events[i]) return VTP_OK;
        const cudaError_t e = cudaEventRecord(static_cast<cudaEvent_t>(events[i]), st);
        return e == cudaSuccess ? VTP_OK : fail((int)e, "stage event %d: %s", i, cudaGetErrorString(e));
    }
};

__global__ void fill_i32_kernel(int32_t* p, int n, int v) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

static bool has_folded_weights(const vtp_block_weights& w) {
    return w.q_wf && w.q_s && w.q_c && w.kv_wf && w.kv_s && w.kv_c && w.fc1_wf && w.fc1_s && w.fc1_c;
}

static bool has_folded_q_fc1(const vtp_block_weights& w) {
    return w.q_wf && w.q_s && w.q_c && w.fc1_wf && w.fc1_s && w.fc1_c;
}

static RegionGeom region_geom(const vtp_dge_shape& s) {
    RegionGeom g;
    g.B = s.B; g.Hr = s.H / s.region; g.Wr = s.W / s.region; g.W = s.W; g.N = s.num_extra + s.H * s.W; g.C = s.C;
    g.num_extra = s.num_extra; g.region = s.region;
    return g;
}

// Whether a block of this shape runs with norm1 folded into q and norm2 into fc1 (bf16 tensor-core path,
// region-parallel token movers, prepared weights).  A block without a spatial reduction folds kv too.  Only
// such blocks hand the next block its gate decisions and token statistics from their unpool.
static bool block_folds(const vtp_dge_shape& s, const vtp_block_weights& w) {
    if (!region_ops_supported(region_geom(s), s.dtype) || s.dtype != VTP_BF16 || (s.flags & VTP_FLAG_CUDA_CORES))
        return false;
    return s.sr_ratio > 1 ? has_folded_q_fc1(w) : has_folded_weights(w);
}

// Position of a block inside a model forward: whether the previous block's unpool already
// produced this block's gate decisions and token statistics (in scratch slot `parity`), and
// the block that follows, whose gate and statistics this block's unpool can produce.
struct BlockChain {
    bool have_gate = false;
    int parity = 0;
    const vtp_block_weights* next = nullptr;
    const float* image_bias = nullptr;   // fp32 [B, n_splits] added to this and the next block's router logits
};

// softmax scale of the attention: the shape's attn_scale, or head_dim^-0.5 when it is 0
static float attn_scale(const vtp_dge_shape& s) {
    return s.attn_scale != 0.f ? s.attn_scale : 1.0f / sqrtf((float)(s.C / s.heads));
}

static int block_forward(const vtp_dge_shape& s, const vtp_block_weights& w, const void* x_in, void* x_out,
                         const float* forced_logits, int32_t* counts_out, void* ws, cudaStream_t st,
                         const StageMarks& marks = StageMarks(), const BlockChain& chain = BlockChain()) {
    const int N = s.num_extra + s.H * s.W;
    const int rows = s.B * N;
    const int Hr = s.H / s.region, Wr = s.W / s.region;
    const int C = s.C, d = C / s.heads;
    const unsigned kflag = s.flags & VTP_FLAG_CUDA_CORES;
    BlockScratch b = carve_block(s, ws);
    const int32_t* L_dev = b.offsets + s.B;
    int rc;
    if ((rc = marks.mark(0))) return rc;

    Splits sp;
    if ((rc = make_splits(&sp, s.splits, s.n_splits, s.region))) return rc;
    const RegionGeom g = region_geom(s);
    // Region-parallel gate / pool / unpool when the region is 4x4 tokens, else one warp per patch.
    const bool by_region = region_ops_supported(g, s.dtype);
    const bool reduce = s.sr_ratio > 1;        // PVT block: keys from spatially reduced tokens (explicit LayerNorm rows)
    VTP_REQUIRE(!reduce || (w.sr_w && w.sr_norm_w && w.sr_norm_b), VTP_ERR_NULL,
                "block: spatial reduction needs the sr and sr_norm parameters");
    const int n_keys = keys_per_image(s);
    // LayerNorm folded into the GEMM epilogues (bf16 tensor-core path with prepared weights): norm1 into q and
    // norm2 into fc1.  A PVT block's keys need LayerNorm rows all the same; the im2col in front of the reducing
    // convolution normalises them on the way from the token statistics.  Without a reduction kv folds norm1 too.
    const bool fold_q = block_folds(s, w);
    const bool fold = fold_q && !reduce;
    // norm2 into fc1 only where the reduction is long enough to hide it: with K <= 128 the Linear is bound by its
    // epilogue, the fold adds a quarter to that, and the narrow-row LayerNorm pass costs less than it adds
    const bool fold_fc1 = fold_q && s.C > 128;
    const int par = chain.parity & 1;
    int32_t* idx = b.idx[par];
    int32_t* counts = b.counts[par];
    float2* stats_x = b.stats_x[par];
    bool stats_x_ready = false;
    // chained: gate decisions, per-image counts and token statistics came from the previous
    // block's unpool; the pool kernel then also derives the row offsets itself
    const bool chained = chain.have_gate && fold_q && !forced_logits;
    VTP_REQUIRE(!chain.image_bias || by_region, VTP_ERR_UNSUPPORTED,
                "block: a per-image gate bias needs the region-parallel gate (4x4-token regions)");

    if (chained) {
        stats_x_ready = true;
        rc = VTP_OK;
    } else if (forced_logits) {
        rc = vtp_gate_argmax(forced_logits, s.B * Hr * Wr, s.n_splits, idx, st);
    } else if (by_region) {
        RegionGateArgs ga;
        ga.g = g; ga.x = x_in; ga.gw = w.gate_w; ga.gb = w.gate_b; ga.S = s.n_splits; ga.logits_out = b.logits[par];
        ga.idx_out = idx; ga.eps = s.eps; ga.image_bias = chain.image_bias;
        if (fold_q) { ga.stats_x = stats_x; stats_x_ready = true; }
        rc = region_gate(ga, s.dtype, st);
    } else {
        rc = vtp_router_gate(x_in, s.dtype, s.B, s.H, s.W, C, s.num_extra, s.region, w.gate_w, w.gate_b,
                             s.n_splits, b.logits[par], idx, st);
    }
    if (rc || (rc = marks.mark(1))) return rc;
    if (!chained)
        rc = index_to_patch(idx, 0, sp, s.B, Hr, Wr, s.region, s.num_extra, counts, b.offsets,
                            by_region ? nullptr : b.patches, nullptr, b.region_first, st);
    if (rc || (rc = marks.mark(2))) return rc;
    if (counts_out) {
        const cudaError_t e = cudaMemcpyAsync(counts_out, counts, (size_t)s.B * 4, cudaMemcpyDeviceToDevice, st);
        if (e != cudaSuccess) return fail((int)e, "block: counts copy: %s", cudaGetErrorString(e));
    }
    if (by_region) {
        RegionPoolArgs pa;
        pa.g = g; pa.sp = sp; pa.x = x_in; pa.idx = idx; pa.comp = b.comp; pa.eps = s.eps;
        pa.region_first = chained ? nullptr : b.region_first;
        pa.offsets = b.offsets; pa.counts = counts; pa.offsets_out = b.offsets; pa.region_first_out = b.region_first;
        const bool will_chain = fold_q && chain.next && block_folds(s, *chain.next);
        pa.counts_next = (chained && will_chain) ? b.counts[par ^ 1] : nullptr;
        if (fold_q) {
            pa.stats_x = stats_x; pa.stats_q = b.stats_q;
            pa.stats_x_ready = stats_x_ready;
        }
        else { pa.lnw = w.norm1_w; pa.lnb = w.norm1_b; pa.xn = b.xn; pa.qn = b.qn; }
        rc = region_pool(pa, s.dtype, st);
    } else {
        rc = vtp_pool(x_in, s.dtype, s.B, N, C, s.W, s.num_extra, b.patches, L_dev, rows, b.comp, w.norm1_w,
                      w.norm1_b, s.eps, b.xn, b.qn, st);
    }
    if (rc || (rc = marks.mark(3))) return rc;

    LinearArgs lq;   // q = LN(comp) Wq^T + b
    lq.a = fold_q ? b.comp : b.qn; lq.lda = C; lq.w = fold_q ? w.q_wf : w.q_w; lq.bias = fold_q ? w.q_c : w.q_b;
    lq.y = b.qp; lq.ldy = C; lq.dtype = s.dtype; lq.m_max = rows; lq.m_dev = L_dev; lq.N = C; lq.K = C; lq.flags = kflag;
    if (fold_q) { lq.ln_mode = 1; lq.ln_stats = b.stats_q; lq.ln_s = w.q_s; }

    const void* keys_in = fold ? x_in : b.xn;
    if (reduce) {
        if ((rc = linear(lq, st)) || (rc = marks.mark(4))) return rc;
        // x_ = norm(sr(LN1(x) as [B,C,H,W])): the stride-sr convolution as im2col rows times a matrix
        const int krows = s.B * n_keys, KS = s.sr_ratio * s.sr_ratio * C;
        if (fold_q) rc = token_im2col(x_in, s.dtype, s.B, s.H, s.W, C, s.sr_ratio, b.sr_cols, st, stats_x, w.norm1_w, w.norm1_b);
        else rc = token_im2col(b.xn, s.dtype, s.B, s.H, s.W, C, s.sr_ratio, b.sr_cols, st);
        if (rc) return rc;
        LinearArgs lsr;
        lsr.a = b.sr_cols; lsr.lda = KS; lsr.w = w.sr_w; lsr.bias = w.sr_b; lsr.y = b.sr_out; lsr.ldy = C;
        lsr.dtype = s.dtype; lsr.m_max = krows; lsr.N = C; lsr.K = KS; lsr.flags = kflag;
        if ((rc = linear(lsr, st))) return rc;
        rc = vtp_layernorm(b.sr_out, s.dtype, krows, nullptr, C, C, w.sr_norm_w, w.sr_norm_b, s.sr_eps, b.sr_norm, st);
        if (rc) return rc;
        keys_in = b.sr_norm;
    }
    LinearArgs lkv;  // kv = LN(x) Wkv^T + b, rows stay [b, key, {k,v}, head, d]
    lkv.a = keys_in; lkv.lda = C; lkv.w = fold ? w.kv_wf : w.kv_w; lkv.bias = fold ? w.kv_c : w.kv_b;
    lkv.y = b.kv; lkv.ldy = 2 * C; lkv.dtype = s.dtype; lkv.m_max = s.B * n_keys; lkv.N = 2 * C; lkv.K = C; lkv.flags = kflag;
    if (fold) { lkv.ln_mode = 1; lkv.ln_stats = stats_x; lkv.ln_s = w.kv_s; }
    if (fold && !marks.events && linear_pair_supported(lkv, lq)) {
        // the two projections do not depend on each other: one launch, the q tiles fill the kv tail
        if ((rc = linear_tcgen05_pair(lkv, lq, st))) return rc;
    } else {
        if (!reduce && ((rc = linear(lq, st)) || (rc = marks.mark(4)))) return rc;
        if ((rc = linear(lkv, st)) || (rc = marks.mark(5))) return rc;
    }

    AttnArgs at;
    const long long e = (long long)elem_size(s.dtype);
    at.q = b.qp; at.q_rs = C; at.q_hs = d;
    at.k = b.kv; at.v = static_cast<const char*>(b.kv) + (long long)C * e;
    at.kv_bs = (long long)n_keys * 2 * C; at.kv_rs = 2 * C; at.kv_hs = d;
    at.out = b.ao; at.o_rs = C; at.o_hs = d;
    at.dtype = s.dtype; at.B = s.B; at.n_keys = n_keys; at.heads = s.heads; at.head_dim = d;
    at.offsets = b.offsets; at.l_max = rows; at.max_q = N; at.scale = attn_scale(s); at.flags = kflag;
    if ((rc = attention(at, st)) || (rc = marks.mark(6))) return rc;

    LinearArgs lp;   // q1 = comp + attn_out Wp^T + b   (and, when folding, the row sums LN2 needs)
    lp.a = b.ao; lp.lda = C; lp.w = w.proj_w; lp.bias = w.proj_b; lp.res = b.comp; lp.ldr = C; lp.y = b.q1;
    lp.ldy = C; lp.dtype = s.dtype; lp.m_max = rows; lp.m_dev = L_dev; lp.N = C; lp.K = C; lp.flags = kflag;
    if (fold_fc1) lp.emit_stats = b.stats_acc;
    if ((rc = linear(lp, st)) || (rc = marks.mark(7))) return rc;

    if (!fold_fc1) {
        rc = vtp_layernorm(b.q1, s.dtype, rows, L_dev, C, C, w.norm2_w, w.norm2_b, s.eps, b.qn, st);
        if (rc) return rc;
    }
    if ((rc = marks.mark(8))) return rc;

    LinearArgs l1;   // hid = GELU(LN2(q1) W1^T + b)
    l1.a = fold_fc1 ? b.q1 : b.qn; l1.lda = C; l1.w = fold_fc1 ? w.fc1_wf : w.fc1_w; l1.bias = fold_fc1 ? w.fc1_c : w.fc1_b;
    l1.y = b.hid; l1.ldy = s.hidden; l1.dtype = s.dtype; l1.m_max = rows; l1.m_dev = L_dev; l1.N = s.hidden; l1.K = C;
    l1.flags = kflag | VTP_FLAG_GELU;
    if (fold_fc1) { l1.ln_mode = 2; l1.ln_stats = b.stats_acc; l1.ln_s = w.fc1_s; l1.ln_dim = C; l1.ln_eps = s.eps;
                l1.ln_slots = linear_stat_slots(C); }
    if ((rc = linear(l1, st)) || (rc = marks.mark(9))) return rc;

    LinearArgs l2;   // q2 = q1 + hid W2^T + b   (into the q-projection buffer, dead by now)
    l2.a = b.hid; l2.lda = s.hidden; l2.w = w.fc2_w; l2.bias = w.fc2_b; l2.res = b.q1; l2.ldr = C; l2.y = b.qp;
    l2.ldy = C; l2.dtype = s.dtype; l2.m_max = rows; l2.m_dev = L_dev; l2.N = C; l2.K = s.hidden; l2.flags = kflag;
    if ((rc = linear(l2, st)) || (rc = marks.mark(10))) return rc;

    if (by_region) {
        RegionUnpoolArgs ua;
        ua.g = g; ua.sp = sp; ua.q = b.qp; ua.comp = b.comp; ua.ref = x_in; ua.out = x_out; ua.idx = idx;
        ua.region_first = b.region_first; ua.offsets = b.offsets;
        if (fold_q && chain.next && block_folds(s, *chain.next)) {
            // the rows being written are the next block's input: leave its LayerNorm statistics and
            // its router gate's decisions in the other scratch slot
            ua.next.stats_x = b.stats_x[par ^ 1]; ua.next.eps = s.eps;
            ua.next.gw = chain.next->gate_w; ua.next.gb = chain.next->gate_b; ua.next.S = s.n_splits;
            ua.next.logits = b.logits[par ^ 1]; ua.next.idx = b.idx[par ^ 1];
            ua.next.counts = b.counts[par ^ 1];
            ua.next.image_bias = chain.image_bias;
            if (!chained) {
                // this block's pool did not reset the next block's counts: start them at the extra tokens
                fill_i32_kernel<<<ceil_div(s.B, 256), 256, 0, st>>>(b.counts[par ^ 1], s.B, s.num_extra);
                if ((rc = check_launch("counts reset"))) return rc;
            }
        }
        rc = region_unpool(ua, s.dtype, st);
    } else {
        rc = vtp_unpool_add(b.qp, b.comp, s.dtype, s.B, N, C, s.W, s.num_extra, b.patches, L_dev, rows, x_in,
                            x_out, st);
    }
    if (rc) return rc;
    return marks.mark(11);
}

__global__ void dense_offsets_kernel(int32_t* offsets, int B, int N) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i <= B) offsets[i] = i * N;
}

static int dense_block_forward(const vtp_dge_shape& s, const vtp_block_weights& w, const void* x_in, void* x_out,
                               void* ws, cudaStream_t st) {
    const int N = s.num_extra + s.H * s.W;
    const int rows = s.B * N;
    const int C = s.C, d = C / s.heads;
    const unsigned kflag = s.flags & VTP_FLAG_CUDA_CORES;
    BlockScratch b = carve_block(s, ws);
    int rc;
    dense_offsets_kernel<<<ceil_div(s.B + 1, 128), 128, 0, st>>>(b.offsets, s.B, N);
    if ((rc = check_launch("dense offsets"))) return rc;
    rc = vtp_layernorm(x_in, s.dtype, rows, nullptr, C, C, w.norm1_w, w.norm1_b, s.eps, b.xn, st);
    if (rc) return rc;
    LinearArgs lq;
    lq.a = b.xn; lq.lda = C; lq.w = w.q_w; lq.bias = w.q_b; lq.y = b.qp; lq.ldy = C; lq.dtype = s.dtype;
    lq.m_max = rows; lq.N = C; lq.K = C; lq.flags = kflag;
    if ((rc = linear(lq, st))) return rc;
    LinearArgs lkv;
    lkv.a = b.xn; lkv.lda = C; lkv.w = w.kv_w; lkv.bias = w.kv_b; lkv.y = b.kv; lkv.ldy = 2 * C;
    lkv.dtype = s.dtype; lkv.m_max = rows; lkv.N = 2 * C; lkv.K = C; lkv.flags = kflag;
    if ((rc = linear(lkv, st))) return rc;
    AttnArgs at;
    const long long e = (long long)elem_size(s.dtype);
    at.q = b.qp; at.q_rs = C; at.q_hs = d;
    at.k = b.kv; at.v = static_cast<const char*>(b.kv) + (long long)C * e;
    at.kv_bs = (long long)N * 2 * C; at.kv_rs = 2 * C; at.kv_hs = d;
    at.out = b.ao; at.o_rs = C; at.o_hs = d;
    at.dtype = s.dtype; at.B = s.B; at.n_keys = N; at.heads = s.heads; at.head_dim = d;
    at.offsets = b.offsets; at.l_max = rows; at.max_q = N; at.scale = attn_scale(s); at.flags = kflag;
    if ((rc = attention(at, st))) return rc;
    LinearArgs lp;
    lp.a = b.ao; lp.lda = C; lp.w = w.proj_w; lp.bias = w.proj_b; lp.res = x_in; lp.ldr = C; lp.y = b.q1;
    lp.ldy = C; lp.dtype = s.dtype; lp.m_max = rows; lp.N = C; lp.K = C; lp.flags = kflag;
    if ((rc = linear(lp, st))) return rc;
    rc = vtp_layernorm(b.q1, s.dtype, rows, nullptr, C, C, w.norm2_w, w.norm2_b, s.eps, b.qn, st);
    if (rc) return rc;
    LinearArgs l1;
    l1.a = b.qn; l1.lda = C; l1.w = w.fc1_w; l1.bias = w.fc1_b; l1.y = b.hid; l1.ldy = s.hidden;
    l1.dtype = s.dtype; l1.m_max = rows; l1.N = s.hidden; l1.K = C; l1.flags = kflag | VTP_FLAG_GELU;
    if ((rc = linear(l1, st))) return rc;
    LinearArgs l2;
    l2.a = b.hid; l2.lda = s.hidden; l2.w = w.fc2_w; l2.bias = w.fc2_b; l2.res = b.q1; l2.ldr = C; l2.y = x_out;
    l2.ldy = C; l2.dtype = s.dtype; l2.m_max = rows; l2.N = C; l2.K = s.hidden; l2.flags = kflag;
    return linear(l2, st);
}

struct ModelScratch {
    void *cols, *x, *cls_n;
    void* block_ws;
    long long bytes;
};

static ModelScratch carve_model(const vtp_dge_shape& s, const vtp_model_weights& m, void* ws) {
    const long long e = (long long)elem_size(s.dtype);
    const int N = s.num_extra + s.H * s.W;
    Carver c(ws);
    ModelScratch r;
    r.cols = c.take((long long)s.B * s.H * s.W * 3 * m.patch * m.patch * e);
    r.x = c.take((long long)s.B * N * s.C * e);
    r.cls_n = c.take((long long)s.B * s.C * e);
    r.block_ws = c.take(carve_block(s, nullptr).bytes);
    r.bytes = c.off;
    return r;
}

}  // namespace vtp

using namespace vtp;

extern "C" long long vtp_block_workspace_bytes(const vtp_dge_shape* s) {
    if (check_shape(s)) return -1;
    return carve_block(*s, nullptr).bytes;
}

extern "C" int vtp_dge_block_forward(const vtp_dge_shape* s, const vtp_block_weights* w, const void* x_in,
                                     void* x_out, const float* forced_logits, int32_t* counts_out,
                                     void* workspace, long long workspace_bytes, void* stream) {
    if (int rc = check_shape(s)) return rc;
    VTP_REQUIRE(w && x_in && x_out && workspace, VTP_ERR_NULL, "block: null pointer");
    VTP_REQUIRE(aligned16(workspace), VTP_ERR_ALIGN, "block: workspace must be 16-byte aligned");
    VTP_REQUIRE(workspace_bytes >= carve_block(*s, nullptr).bytes, VTP_ERR_SHAPE,
                "block: workspace of %lld bytes is smaller than the %lld needed", workspace_bytes,
                carve_block(*s, nullptr).bytes);
    return block_forward(*s, *w, x_in, x_out, forced_logits, counts_out, workspace,
                         static_cast<cudaStream_t>(stream));
}

extern "C" int vtp_dge_blocks_forward(const vtp_dge_shape* s, const vtp_block_weights* w, int n_blocks,
                                      const void* x_in, void* x_out, int32_t* counts_out, void* workspace,
                                      long long workspace_bytes, void* stream) {
    if (int rc = check_shape(s)) return rc;
    VTP_REQUIRE(w && x_in && x_out && workspace, VTP_ERR_NULL, "blocks: null pointer");
    VTP_REQUIRE(n_blocks > 0, VTP_ERR_SHAPE, "blocks: n_blocks=%d", n_blocks);
    VTP_REQUIRE(aligned16(workspace), VTP_ERR_ALIGN, "blocks: workspace must be 16-byte aligned");
    VTP_REQUIRE(workspace_bytes >= carve_block(*s, nullptr).bytes, VTP_ERR_SHAPE,
                "blocks: workspace of %lld bytes is smaller than the %lld needed", workspace_bytes,
                carve_block(*s, nullptr).bytes);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    bool chained = false;      // block i-1's unpool prepared block i's gate
    for (int i = 0; i < n_blocks; ++i) {
        BlockChain chain;
        chain.have_gate = chained;
        chain.parity = i & 1;
        chain.next = (i + 1 < n_blocks) ? &w[i + 1] : nullptr;
        if (int rc = block_forward(*s, w[i], i == 0 ? x_in : x_out, x_out, nullptr,
                                   counts_out ? counts_out + (size_t)i * s->B : nullptr, workspace, st, StageMarks(),
                                   chain))
            return rc;
        chained = chain.next && block_folds(*s, w[i]) && block_folds(*s, *chain.next);
    }
    return VTP_OK;
}

extern "C" int vtp_dge_block_forward_timed(const vtp_dge_shape* s, const vtp_block_weights* w, const void* x_in,
                                           void* x_out, const float* forced_logits, int32_t* counts_out,
                                           void* workspace, long long workspace_bytes, void* const* events,
                                           int n_events, void* stream) {
    if (int rc = check_shape(s)) return rc;
    VTP_REQUIRE(w && x_in && x_out && workspace && events, VTP_ERR_NULL, "block: null pointer");
    VTP_REQUIRE(aligned16(workspace), VTP_ERR_ALIGN, "block: workspace must be 16-byte aligned");
    VTP_REQUIRE(workspace_bytes >= carve_block(*s, nullptr).bytes, VTP_ERR_SHAPE, "block: workspace too small");
    StageMarks marks;
    marks.events = events; marks.n = n_events; marks.st = static_cast<cudaStream_t>(stream);
    return block_forward(*s, *w, x_in, x_out, forced_logits, counts_out, workspace, marks.st, marks);
}

extern "C" int vtp_dense_block_forward(const vtp_dge_shape* s, const vtp_block_weights* w, const void* x_in,
                                       void* x_out, void* workspace, long long workspace_bytes, void* stream) {
    if (int rc = check_shape(s)) return rc;
    VTP_REQUIRE(w && x_in && x_out && workspace, VTP_ERR_NULL, "dense block: null pointer");
    VTP_REQUIRE(x_in != x_out, VTP_ERR_UNSUPPORTED, "dense block: x_out must not alias x_in");
    VTP_REQUIRE(workspace_bytes >= carve_block(*s, nullptr).bytes, VTP_ERR_SHAPE, "dense block: workspace too small");
    return dense_block_forward(*s, *w, x_in, x_out, workspace, static_cast<cudaStream_t>(stream));
}

extern "C" long long vtp_model_workspace_bytes(const vtp_dge_shape* s, const vtp_model_weights* m) {
    if (check_shape(s) || !m) return -1;
    return carve_model(*s, *m, nullptr).bytes;
}

extern "C" int vtp_deit_dge_forward(const vtp_dge_shape* s, const vtp_model_weights* m,
                                    const vtp_block_weights* blocks, const void* images, float* logits,
                                    int32_t* counts_out, void* workspace, long long workspace_bytes,
                                    void* stream) {
    return vtp_deit_dge_forward_ex(s, m, blocks, images, logits, counts_out, nullptr, workspace, workspace_bytes,
                                   stream);
}

extern "C" int vtp_deit_dge_forward_ex(const vtp_dge_shape* s, const vtp_model_weights* m,
                                       const vtp_block_weights* blocks, const void* images, float* logits,
                                       int32_t* counts_out, const vtp_forward_options* opt, void* workspace,
                                       long long workspace_bytes, void* stream) {
    if (int rc = check_shape(s)) return rc;
    VTP_REQUIRE(m && blocks && images && logits && workspace, VTP_ERR_NULL, "model: null pointer");
    VTP_REQUIRE(m->depth > 0 && m->patch > 0 && m->num_classes > 0, VTP_ERR_SHAPE, "model: bad shape");
    VTP_REQUIRE(m->img_size == s->H * m->patch && s->H == s->W && s->num_extra == 1, VTP_ERR_SHAPE,
                "model: image %d does not match a %dx%d grid of %d-pixel patches with one cls token",
                m->img_size, s->H, s->W, m->patch);
    VTP_REQUIRE(aligned16(workspace), VTP_ERR_ALIGN, "model: workspace must be 16-byte aligned");
    const ModelScratch ms = carve_model(*s, *m, workspace);
    VTP_REQUIRE(workspace_bytes >= ms.bytes, VTP_ERR_SHAPE, "model: workspace of %lld bytes, %lld needed",
                workspace_bytes, ms.bytes);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int HW = s->H * s->W, N = HW + 1, C = s->C;
    const int KP = 3 * m->patch * m->patch;
    const long long e = (long long)elem_size(s->dtype);
    int rc = vtp_patch_im2col(images, m->image_dtype, s->B, m->img_size, m->patch, s->dtype, ms.cols, m->cls_token,
                              m->pos_embed, C, ms.x, st);
    if (rc) return rc;
    LinearArgs pe;   // token (b, 1+t) = cols(b,t) Wp^T + bias + pos_embed[1+t]
    pe.a = ms.cols; pe.lda = KP; pe.w = m->patch_w; pe.bias = m->patch_b; pe.res = m->pos_embed; pe.ldr = C;
    pe.y = ms.x; pe.ldy = C; pe.dtype = s->dtype; pe.m_max = s->B * HW; pe.N = C; pe.K = KP;
    pe.flags = s->flags & VTP_FLAG_CUDA_CORES;
    pe.out_grp = HW; pe.out_skip = 1; pe.res_mod = HW; pe.res_off = 1;
    if ((rc = linear(pe, st))) return rc;
    bool chained = false;      // block i-1's unpool prepared block i's gate
    const BlockScratch bs = carve_block(*s, ms.block_ws);
    const long long R = (long long)(s->H / s->region) * (s->W / s->region);
    for (int i = 0; i < m->depth; ++i) {
        BlockChain chain;
        chain.have_gate = chained;
        chain.parity = i & 1;
        chain.next = (i + 1 < m->depth) ? &blocks[i + 1] : nullptr;
        chain.image_bias = opt ? opt->gate_image_bias : nullptr;
        if (opt && opt->tokens_trace) {
            const size_t nb = (size_t)s->B * N * C * e;
            const cudaError_t ce = cudaMemcpyAsync(static_cast<char*>(opt->tokens_trace) + (size_t)i * nb, ms.x, nb,
                                                   cudaMemcpyDeviceToDevice, st);
            if (ce != cudaSuccess) return fail((int)ce, "model: tokens trace copy: %s", cudaGetErrorString(ce));
        }
        rc = block_forward(*s, blocks[i], ms.x, ms.x, nullptr, counts_out ? counts_out + (size_t)i * s->B : nullptr,
                           ms.block_ws, st, StageMarks(), chain);
        if (rc) return rc;
        if (opt && opt->grain_trace) {
            // the block's grain indices stay in its slot of the scratch (its unpool writes the other slot)
            const size_t nb = (size_t)s->B * R * sizeof(int32_t);
            const cudaError_t ce = cudaMemcpyAsync(opt->grain_trace + (size_t)i * s->B * R, bs.idx[i & 1], nb,
                                                   cudaMemcpyDeviceToDevice, st);
            if (ce != cudaSuccess) return fail((int)ce, "model: grain trace copy: %s", cudaGetErrorString(ce));
        }
        chained = chain.next && block_folds(*s, blocks[i]) && block_folds(*s, *chain.next);
    }
    rc = vtp_layernorm(ms.x, s->dtype, s->B, nullptr, C, (long long)N * C, m->norm_w, m->norm_b, s->eps, ms.cls_n, st);
    if (rc) return rc;
    LinearArgs hd;
    hd.a = ms.cls_n; hd.lda = C; hd.w = m->head_w; hd.bias = m->head_b; hd.y = logits; hd.ldy = m->num_classes;
    hd.dtype = s->dtype; hd.m_max = s->B; hd.N = m->num_classes; hd.K = C;
    hd.flags = (s->flags & VTP_FLAG_CUDA_CORES) | VTP_FLAG_OUT_F32;
    return linear(hd, st);
}
