// Host-side interface of the token-pool encoder kernels (token_pool.cu): the fp32 single-head encoder whose
// per-token rows are pooled over token spans into child vectors (runtime/sparse_token_pool_vector_export.go).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace eosb {

// out[i, :] = table[tokens[i], :], zeros for an id outside [0, vocab) (gatherTokenRows, :1337-1349)
void launch_tp_gather(const float* table, int vocab, int dim, const int32_t* tokens, int n, float* out, cudaStream_t s);
// out[r, o] = sum_i rows[r, i] * w[i, o], a float sum in i order (matmulRowsRight, :1620-1633); epilogue 1 = tanh GELU
void launch_tp_matmul(const float* rows, int row_count, int in_dim, const float* w, int out_dim, int epilogue, float* out,
                      cudaStream_t s);
void launch_tp_add(const float* a, const float* b, long long n, float* out, cudaStream_t s);
// non-affine LayerNorm of every row, eps 1e-5 inside the double square root (layerNormRow, embedding_trainer.go:13005-13024)
void launch_tp_layernorm(const float* rows, int row_count, int dim, float* out, cudaStream_t s);
// rows scaled to unit L2 norm, sum of squares in double (normalizeRetrievalVector, retrieval_eval.go:1040-1054)
void launch_tp_normalize(float* rows, int row_count, int dim, cudaStream_t s);
// dense single-head attention without a 1/sqrt(d) factor (denseSoftmaxAttentionRows, :1430-1465); scores is scratch
// [seq_len, seq_len]
void launch_tp_dense_attention(const float* q, const float* k, const float* v, int seq_len, int dim, float* scores,
                               float* out, int sm_count, cudaStream_t s);
// out[s, :] = unit-normalised mean of the rows r in [starts[s], ends[s]) with mask[r] != 0
// (poolSparseTokenRowsRange, :1597-1618); fallback_all != 0: a span without active rows pools all of its rows
// (maskedMeanPoolNormalized, :1534-1559), otherwise its vector is all zeros and flags[s] = 1
void launch_tp_span_pool(const float* rows, const int32_t* mask, const int* starts, const int* ends, int spans, int dim,
                         int fallback_all, float* out, int* flags, cudaStream_t s);
// codes [n][ceil(dim * bits / 8)] packed little-end first -> one byte per coordinate
void launch_tp_unpack_codes(const uint8_t* packed, long long n, int dim, int bits, uint8_t* out, cudaStream_t s);

}  // namespace eosb
