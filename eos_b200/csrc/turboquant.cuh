// Launchers of the TurboQuant kernels (turboquant.cu): Hadamard/MSE code packing, the scan
// layout, query preparation, the scoring scan with per-CTA exact top-k and the merge.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace eosb {

// Rotation + codebook of one quantiser, device resident.  Same fields the reference's
// turboquant Spec() exposes (runtime/backends/cuda/native_linux.go:9532-9545).
struct TqSpec {
    int dim;
    int bits;
    const int* perm;          // [dim]
    const float* signs1;      // [dim]
    const float* signs2;      // [dim]
    const float* centroids;   // [2^bits] ascending
    const float* boundaries;  // [2^bits - 1]
};

constexpr int kTqDocsPerTile = 16;   // documents per scan tile (one m16 MMA row block)
constexpr int kTqChunkCoords = 128;  // coordinates per 16-byte code chunk group (8 k-steps of 16)
constexpr int kTqMaxK = 128;         // largest k of the fused top-k
constexpr int kTqWideK = 256;        // largest k of the merge kernel (the wide path: all scores, then one select)
constexpr int kTqScanWarps = 16;

// bytes of one scan tile: 16 documents x padded_dim/2 bytes
inline size_t tq_tile_bytes(int dim) {
    const int padded = (dim + kTqChunkCoords - 1) / kTqChunkCoords * kTqChunkCoords;
    return (size_t)kTqDocsPerTile * padded / 2;
}
__host__ __device__ inline int tq_ksteps(int dim) { return (dim + kTqChunkCoords - 1) / kTqChunkCoords * (kTqChunkCoords / 16); }

// x [n, dim] fp32 -> packed codes [n, dim*bits/8] (low bits first) + fp32 norms [n].
void launch_tq_pack(const float* x, int64_t n, const TqSpec& spec, uint8_t* codes, float* norms,
                    cudaStream_t stream);

// reference-format codes -> scan tiles (sign-magnitude nibbles in MMA fragment order).
void launch_tq_transcode(const uint8_t* codes, int64_t n, int dim, int bits, uint8_t* tiles, cudaStream_t stream);

// queries [q, dim] fp32 -> rotated f16 B fragments [ceil(q/8)][ksteps][32 lanes] x 8 bytes;
// also the rotated fp32 queries when rotated_out != null.
// Fragments are written for q_fill >= q queries (a multiple of 8); queries past q are zeros.
// qperm, when non-null, receives the rotated queries as f16 rows [q_fill][padded dim] with the coordinates of every
// 64-block in the order of the scan layout's code words (the A operand of the tensor-core kernel); bfrag may be null.
void launch_tq_prepare(const float* queries, int q, int q_fill, const TqSpec& spec, uint2* bfrag, float* rotated_out,
                       __half* qperm, cudaStream_t stream);

// keys[p] = sortable key of (sum over `rows` of the per-row parent aggregate, parent id p):
// per row and parent the mean of the best min(top_n, 5, children) child scores minus
// penalty * log1p(children); parents without children get key 0.  child_order lists children
// grouped by parent, offsets [parents + 1]; scores is [rows][stride].
void launch_parent_keys(const float* scores, long long stride, int rows, const int* child_order, const int* offsets,
                        int parents, int top_n, double penalty, float* agg_scratch, uint64_t* keys,
                        cudaStream_t stream);

struct TqScanArgs {
    const uint8_t* tiles;
    const float* norms;
    int64_t n_docs;
    uint32_t id_base;      // document id of row 0 (ids are carried inside the candidate keys)
    int dim;
    const uint2* bfrag;    // fragments of the first query tile of this pass
    int query_tiles;       // 1, 2 or 4 tiles of 8 queries scored per corpus pass
    int k;
    uint32_t mag_hi[2];    // high / low bytes of the f16 magnitude table (8 entries)
    uint32_t mag_lo[2];
    uint64_t* cand_keys;   // [query_tiles*8][grid][kTqMaxK]
    int* cand_count;       // [query_tiles*8][grid]
    int grid;
    int* status;           // device status word (receives kStatusPipelineTimeout if a bounded wait runs out)
    unsigned long long* shared_tau;  // when non-null: [query_tiles*8] keys, zero before the pass; the CTAs publish the
                                     // k-th best key they hold, and every CTA prunes with the largest one published
    float* all_scores;     // when non-null: every score is stored at all_scores[q * all_stride + doc]
    long long all_stride;  // and the top-k bookkeeping is skipped
};
// Returns the dynamic shared memory the configuration needs (0 = unsupported).
size_t tq_scan_smem_bytes(int query_tiles, int dim);
std::string tq_check_dim(int dim);
cudaError_t tq_scan_init();
void launch_tq_scan(const TqScanArgs& a, cudaStream_t stream);

// Batched scoring on the tensor cores (turboquant_tc.cu): one launch = kTqTcQueries queries x the whole shard.
constexpr int kTqTcQueries = 128;  // queries per launch
constexpr int kTqTcDocs = 256;     // documents per tile, queries staged through shared memory
constexpr int kTqTcDocsQ = 128;    // documents per tile, queries resident in tensor memory (padded dim <= 768)
constexpr int kTqTcSegLen = 256;   // slots of one candidate list; a launch of `grid` CTAs fills 2 * grid lists per query
struct TqTcArgs {
    const uint8_t* tiles;
    const float* norms;
    int64_t n_docs;
    uint32_t id_base;
    int dim;
    int q_row0;            // first row of this launch's queries in the permuted f16 query matrix
    int q_valid;           // queries of this launch that exist (the rest are padding and collect nothing)
    int k;                 // <= kTqMaxK
    uint32_t mag_hi[2];
    uint32_t mag_lo[2];
    uint64_t* cand_keys;   // [kTqTcQueries][2 * grid][kTqTcSegLen]
    int* cand_count;       // [kTqTcQueries][2 * grid]
    unsigned long long* shared_tau;  // [kTqTcQueries] pruning thresholds: seeded by the caller (0 = none), raised by
                                     // every CTA that cuts a list
    float* seed_scores;    // seed mode when non-null: every score goes to seed_scores[query * seed_stride + row] and
    int64_t seed_stride;   // no list is kept
    const __half* qperm;   // the permuted f16 query matrix itself (variant with the queries in tensor memory)
    int* status;
    // late-interaction (MaxSim) mode when maxsim_children > 0: rows of the corpus are child vectors, every
    // maxsim_children (16, 32, 64 or 128) consecutive rows belong to one parent, every maxsim_group (a power of two
    // <= 32) consecutive query vectors to one query; the score of (query, parent) is the sum over the query's
    // vectors of the best child score.  Candidate keys carry parent ids ((id_base + row) / maxsim_children); lists,
    // counts and thresholds are indexed by query (query vector / maxsim_group), not by query vector.
    int maxsim_children;
    int maxsim_group;
    int maxsim_list_base;   // index of this launch's first query among the candidate lists (several launches share one merge)
};
cudaError_t tq_tc_init();
// Tensor map of the permuted query matrix [rows][padded_dim] f16 (rows a multiple of kTqTcQueries).
std::string tq_tc_make_query_map(CUtensorMap* tm, const __half* qperm, int padded_dim, int rows);
// True when the rotated queries of a launch fit tensor memory beside one accumulator (padded dim <= 768).
bool tq_tc_queries_fit_tmem(int dim);
// q_in_tmem selects the variant: tiles of kTqTcDocsQ documents with the queries resident in tensor memory, or tiles
// of kTqTcDocs documents with the queries staged through shared memory by TMA (tm_q).
void launch_tq_score_tc(const CUtensorMap& tm_q, const TqTcArgs& a, bool q_in_tmem, int grid, cudaStream_t stream);

// The same batch scoring with the operand roles swapped (turboquant_tc256.cu): one launch = kTqTc256Queries queries,
// tiles of kTqTc256Docs documents as the MMA's M rows; one candidate list per CTA and query
// (cand_keys [256][grid][kTqTcSegLen], cand_count [256][grid], shared_tau [256]); seed mode as above.
constexpr int kTqTc256Queries = 256;
constexpr int kTqTc256Docs = 128;
cudaError_t tq_tc256_init();
std::string tq_tc256_make_query_map(CUtensorMap* tm, const __half* qperm, int padded_dim, int rows);
void launch_tq_score_tc256(const CUtensorMap& tm_q, const TqTcArgs& a, int grid, cudaStream_t stream);

// For every query: the k best of n_segs x seg_len candidate keys (key 0 = empty), sorted by
// score descending then id ascending.  cand is [queries][n_segs][seg_len] with the given
// strides (in keys).  counts, when non-null, is [queries][n_segs] entries in use.
void launch_tq_merge(const uint64_t* cand, int64_t query_stride, int64_t seg_stride, int n_segs, int seg_len,
                     const int* counts, int queries, int k, int64_t id_base, int64_t* out_ids, float* out_scores,
                     uint64_t* out_keys, cudaStream_t stream);
cudaError_t tq_merge_init();
// The same merge for counted lists (counts != null, at most 1024 lists per query), with the keys gathered once into
// shared memory; keys carry the document ids (no id_base).  Falls back to launch_tq_merge above 1024 lists.
void launch_tq_merge_lists(const uint64_t* cand, int64_t query_stride, int64_t seg_stride, int n_segs, int seg_len,
                           const int* counts, int queries, int k, int64_t* out_ids, float* out_scores, uint64_t* out_keys,
                           cudaStream_t stream);
// tau[q] = largest key that every document scoring at least the k-th best of scores[q][0..total) still beats (0 when
// total < k; the scores are compared on their upper 16 bits, rounded down); scores is [queries][query_stride] fp32,
// NaN = no document.  At most 40960 scores per query are used.
void launch_tq_seed_tau_scores(const float* scores, int64_t query_stride, int total, int queries, int k,
                               unsigned long long* tau, cudaStream_t stream);

// keys[q * cand + j] = sortable key (score, row) of query q against document row j (cand_ids == null, cand = n_rows)
// or against row cand_ids[q * cand + j] (negative or out-of-range id: key 0 = absent).  docs is [n_rows, dim] fp32 or
// f16; metric 0 = dot product, 1 = cosine (0 when either norm is 0).  dim <= 1024.  Feed the keys to launch_tq_merge
// with one segment of cand keys per query for the exact top-k (score descending, row ascending).
void launch_dense_keys(const void* docs, bool docs_f16, int64_t n_rows, int dim, const float* queries, int nq,
                       const int64_t* cand_ids, int64_t cand, int metric, uint64_t* keys, int sm_count,
                       cudaStream_t stream);

// Wide path helpers.  keys[q * key_stride + r] = sortable key (scores[q * score_stride + r], r) for r < n, 0 (empty) for
// n <= r < key_stride: feed them to launch_tq_merge in segments for k up to kTqWideK.
void launch_tq_score_keys(const float* scores, int64_t score_stride, int queries, int64_t n, int64_t key_stride,
                          uint64_t* keys, int sm_count, cudaStream_t stream);
// Sign stage of the inner-product quantiser: scores[q, row] += norms[row] * resnorms[row] * qjl_scale *
// sum_i sketch[q, i] * (bit i of signs[row] ? +1 : -1).  signs is [n][ceil(dim / 32)] 32-bit words, bit i of a row at
// word i / 32, bit i % 32; sketch is [queries, dim] fp32.
cudaError_t tq_ip_init();
size_t tq_ip_sign_stage_smem(int dim);
void launch_tq_ip_sign_stage(const uint32_t* signs, const float* resnorms, const float* norms, int64_t n,
                             const float* sketch, int queries, int dim, float qjl_scale, float* scores,
                             int64_t score_stride, int sm_count, cudaStream_t stream);

}  // namespace eosb
