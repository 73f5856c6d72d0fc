// Host-side interface of the sparse attention kernels (sparse_attention.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "turboquant.cuh"

namespace eosb {

constexpr int kSaMaxBudget = 128;   // most keys (and most route blocks) a query row may select

cudaError_t sparse_attention_init();
size_t sparse_attention_smem_bytes(int dim);
// query [batches, q_len, dim], key [batches, k_len, dim], value [batches, k_len, vdim] -> out [batches, q_len, vdim],
// all fp32 on the device; budget <= kSaMaxBudget; block_size, top_blocks (<= kSaMaxBudget) > 0 select block-anchor
// routing (already normalised against k_len).
void launch_sparse_attention(const float* q, const float* k, const float* v, int batches, int q_len, int k_len, int dim,
                             int vdim, int budget, int block_size, int top_blocks, float* out, int sm_count,
                             cudaStream_t stream);
// out [n, dim] fp32 = decoded TurboQuant rows; codes [n, dim] one byte per coordinate, norm_codes [n] 8-bit log codes.
void launch_tq_decode_rows(const uint8_t* codes, const uint8_t* norm_codes, int64_t n, const TqSpec& spec, float* out,
                           int sm_count, cudaStream_t stream);

}  // namespace eosb
