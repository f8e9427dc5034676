// Internal interface of the variable-length-query attention kernels.
#pragma once

#include "common.cuh"

namespace vtp {

struct AttnArgs {
    const void* q = nullptr; long long q_rs = 0, q_hs = 0;
    const void* k = nullptr; const void* v = nullptr;
    long long kv_bs = 0, kv_rs = 0, kv_hs = 0;
    void* out = nullptr; long long o_rs = 0, o_hs = 0;
    int dtype = VTP_F32;
    int B = 0, n_keys = 0, heads = 0, head_dim = 0;
    const int32_t* offsets = nullptr;   // device int32 [B+1]
    int l_max = 0;                      // rows the q / out buffers hold
    int max_q = 0;                      // upper bound of the queries of one image
    float scale = 1.f;
    unsigned flags = 0;
};

int attention_cuda_cores(const AttnArgs& p, cudaStream_t st);
int attention_tcgen05(const AttnArgs& p, cudaStream_t st);
int attention_tcgen05_max_images();   // images per call the tensor-core kernel's shared-memory tile table holds
int attention(const AttnArgs& p, cudaStream_t st);

}  // namespace vtp
