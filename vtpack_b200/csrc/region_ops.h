// Internal interface of the region-parallel kernels (router gate, pooling, unpooling).
#pragma once

#include "common.cuh"

namespace vtp {

struct Splits { int v[8]; int n; };

struct RegionGeom {
    int B, Hr, Wr;      // images, regions per column / row
    int W, N, C;        // token grid width, tokens per image (extra + H*W), channels
    int num_extra;      // cls tokens in front of the grid
    int region;         // tokens per region side
    int l_max = 0;      // rows of the packed array where the caller supplies each region's first row
                        // (0: the rows come from this library's own compaction and are not checked)
};

struct RegionPoolArgs {
    RegionGeom g; Splits sp;
    const void* x = nullptr;
    const int32_t* idx = nullptr;            // grain index per region
    const int32_t* region_first = nullptr;   // packed row of each region's first query; null: derive it
                                             //   in the kernel from `counts` and write `offsets_out`
    const int32_t* offsets = nullptr;        // packed row of each image's first query (with region_first)
    const int32_t* counts = nullptr;         // queries per image (without region_first)
    int32_t* offsets_out = nullptr;          // [B+1], written when region_first is null
    int32_t* region_first_out = nullptr;     // [B*R], written when region_first is null (for the unpool)
    int32_t* counts_next = nullptr;          // [B], reset to num_extra for the next block's gate
    void* comp = nullptr;
    // LayerNorm applied later, in a GEMM epilogue: per-row (mean, rstd) of x and of comp, and a
    // per-query accumulator to clear.  Leave null for explicit LayerNorm rows instead.
    float2* stats_x = nullptr; float2* stats_q = nullptr; float2* stats_acc = nullptr;
    bool stats_x_ready = false;              // stats_x was already written (by the previous block's unpool)
    const float* lnw = nullptr; const float* lnb = nullptr; float eps = 1e-6f;
    void* xn = nullptr; void* qn = nullptr;
    // With neither statistics nor LayerNorm rows asked for: plain pooled rows, as means or (sum_only) as the
    // sums of each patch's tokens, which is the gradient of the replicate-unpool for its packed rows.
    bool sum_only = false;
};

// What the unpool kernel can prepare for the block that follows, from the rows it has just
// written: their LayerNorm statistics and the next router gate's decisions.
struct NextBlock {
    float2* stats_x = nullptr; float eps = 1e-6f;
    const float* gw = nullptr; const float* gb = nullptr; int S = 0;
    float* logits = nullptr; int32_t* idx = nullptr;
    int32_t* counts = nullptr;               // [B] per-image query counts, accumulated with atomics
    const float* image_bias = nullptr;       // [B, S] added to the logits of every region of image b, or null
};

struct RegionUnpoolArgs {
    RegionGeom g; Splits sp;
    const void* q = nullptr; const void* comp = nullptr; const void* ref = nullptr; void* out = nullptr;
    const int32_t* idx = nullptr; const int32_t* region_first = nullptr; const int32_t* offsets = nullptr;
    NextBlock next;
};

struct RegionGateArgs {
    RegionGeom g;
    const void* x = nullptr;
    const float* gw = nullptr; const float* gb = nullptr; int S = 0;
    float* logits_out = nullptr; int32_t* idx_out = nullptr;
    float2* stats_x = nullptr; float eps = 1e-6f;     // optional: also the token rows' (mean, rstd)
    const float* image_bias = nullptr;                // [B, S] added to the logits of every region of image b, or null
};

bool region_ops_supported(const RegionGeom& g, int dtype);
int region_pool(const RegionPoolArgs& a, int dtype, cudaStream_t st);
int region_unpool(const RegionUnpoolArgs& a, int dtype, cudaStream_t st);
int region_gate(const RegionGateArgs& a, int dtype, cudaStream_t st);

// Patch list + per-region first rows (internal form of vtp_index_to_patch).
int index_to_patch(const void* indices, int idx_is_i64, const Splits& sp, int B, int Hr, int Wr, int region,
                   int num_extra, int32_t* counts, int32_t* offsets, int32_t* patches, int64_t* patches64,
                   int32_t* region_first, cudaStream_t st);

int make_splits(Splits* sp, const int* splits, int n_splits, int region);

}  // namespace vtp
