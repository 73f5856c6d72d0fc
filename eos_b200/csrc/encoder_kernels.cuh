// Launchers of the bandwidth-bound encoder kernels and of attention (encoder_kernels.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace eosb {

// Packed-row bookkeeping of one batch: only tokens whose attention_mask is non-zero get a row
// (padding is skipped, not computed and masked).  All arrays live on the device.
struct SeqLayout {
    int* key_count;   // [B]   tokens with mask != 0 (they are the keys and, pooled, the mean's rows)
    int* row_count;   // [B]   rows of the sequence (= key_count, + 1 query-only CLS row when token 0 is masked)
    int* cu_rows;     // [B+1] exclusive prefix sum of row_count
    int* cls_row;     // [B]   packed row that holds token 0
    int* row_src;     // [M]   flat index b*T + t of every packed row
    int* total_rows;  // [1]
    int* cu_qtiles;   // [B+1] exclusive prefix sum of ceil(row_count / 128): 128-query tiles per sequence
    int4* qtile_info; // [sum of q-tiles] per 128-query tile: {first row of the sequence, its rows, its keys, tile's first query}
    int4* qtile_win;  // [sum of q-tiles] key tiles of 128 the tile attends to: {first, end, first fully visible, end of those}
                      // both lists are ordered by the number of key tiles a tile visits, most first, so that a kernel
                      // that deals the tiles out round-robin gives every worker the same amount of work
    int4* qtile_info_seq;  // the same two lists in sequence order (what the fill kernel writes; scratch)
    int4* qtile_win_seq;
};

// window: local attention window of the model (<= 0: none); it only shapes qtile_win.
void launch_seq_layout(const int32_t* mask, int batch, int tokens, int cls_pooling, int window, const SeqLayout& lay,
                       cudaStream_t stream);

// hidden[r,:] = LayerNorm(tok[id] + pos[t] + typ[type]) * gamma + beta for every packed row.
void launch_embed_ln(const int32_t* ids, const int32_t* types, const SeqLayout& lay, int tokens, const __half* tok,
                     int vocab, const __half* pos, int max_pos, const __half* typ, int type_vocab, const float* gamma,
                     const float* beta, float eps, int dim, int m_alloc, __half* out, int* status, int sm_count,
                     cudaStream_t stream);

// out[r,:] = LayerNorm(in[r,:]) * gamma + beta, rows < *total_rows.
void launch_layernorm(const __half* in, const float* gamma, const float* beta, float eps, int dim, int m_alloc,
                      const int* total_rows, __half* out, int sm_count, cudaStream_t stream);

// Multi-head self-attention over the packed rows.  qkv is [M, 3*hidden] (q | k | v, heads
// interleaved as head*head_dim + d); ctx is [M, hidden].  Keys of a sequence are its first
// key_count rows; every row is a query.  window <= 0: full attention; window > 0: key j is
// visible to query i only if |pos_i - pos_j| < window/2 (local-window extension).
void launch_attention(const __half* qkv, const SeqLayout& lay, int batch, int tokens, int hidden, int heads,
                      int window, __half* ctx, cudaStream_t stream);

// pooled -> L2 -> optional head ([hidden, head_out], in-major) -> L2; writes out [B, E] fp32.
void launch_pool_head(const __half* hidden_states, const SeqLayout& lay, int batch, int dim, int cls_pooling,
                      const float* head_w, int head_out, float* pooled_scratch, float* out, cudaStream_t stream);

// Compact encoder profile (models/default_embedding.go:461-505).
// hidden[r,:] = rope(tok[id] + role[role id]) for every packed row; rope_cs is [rope_tokens, dim/2] (cos, sin).
void launch_embed_rope(const int32_t* ids, const int32_t* roles, const SeqLayout& lay, int tokens, const __half* tok,
                       int vocab, const __half* role_tab, int role_vocab, const float2* rope_cs, int rope_tokens, int dim,
                       int m_alloc, __half* out, int* status, int sm_count, cudaStream_t stream);
// out [rows, dim] fp32 = the packed f16 rows, each divided by its L2 norm (zero rows stay zero).
void launch_rows_normalize_f32(const __half* x, const SeqLayout& lay, int dim, int m_alloc, float* out, int sm_count,
                                cudaStream_t stream);
// In place per-row L2 normalisation of the packed rows (zero rows untouched).
void launch_token_normalize(__half* x, const SeqLayout& lay, int dim, int m_alloc, int sm_count, cudaStream_t stream);
// out [B, dim] fp32 = mean over each sequence's valid tokens of the (optionally L2-normalised) rows.
void launch_compact_pool(const __half* hidden_states, const SeqLayout& lay, int batch, int tokens, int dim, int normalize,
                         float* out, cudaStream_t stream);

// Compiled pipeline gather -> matmul -> per-token normalize -> masked mean_pool: one launch over groups of 8
// valid tokens (partial sums) and one that adds a sequence's groups in order.
// table [vocab, dim] f16, projection [dim, out_dim] f16 (in-major), out [B, out_dim] fp32;
// partial [B, ceil(tlen / 8), out_dim] fp32 and counts [B] are scratch.  matmul_scale multiplies the projected rows.
void launch_embed_pooled(const int32_t* tokens, const int32_t* mask, int batch, int tlen, const __half* table,
                         int vocab, int dim, const __half* projection, int out_dim, float matmul_scale, int pool_then_l2,
                         float* partial, int* counts, float* out, int* status, cudaStream_t stream);

}  // namespace eosb
