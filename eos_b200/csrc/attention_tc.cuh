// Host-side interface of the tcgen05 attention kernel (attention_tc.cu).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <string>

#include "encoder_kernels.cuh"

namespace eosb {

struct AttnTcPlan {
    CUtensorMap tm_qkv;  // [M, 3*hidden] f16, box 64 x 128, 128B swizzle
};

// Usable when head_dim == 64; any sequence length; window <= 0 means full attention.
std::string attn_tc_make_plan(AttnTcPlan* plan, const __half* qkv, int m_alloc, int hidden);
void attn_tc_launch(const AttnTcPlan& plan, const SeqLayout& lay, int batch, int tokens, int hidden, int heads,
                    int window, __half* ctx, int* status, int sm_count, cudaStream_t stream);
std::string attn_tc_global_init();

}  // namespace eosb
