/*
 * eos_b200.h -- C ABI of libeos_b200.so: the B200 (sm_100a) implementation of Eos's query-time
 * embed-and-score path.  Every entry point states which Eos interface it stands in for
 * (path inside the Eos project : lines).
 *
 * Conventions (the ones of Eos's CGo CUDA bridge, runtime/backends/cuda/native_linux.go:1-1616
 * and eos_cuda_abi.h:22-38):
 *   - every call returns int: 0 = ok, 1 = failure, 2 = the device status word is non-zero
 *     (bad token id and the like; native_linux.go:699-705, 8119-8127);
 *   - on a non-zero return *err (when err != NULL) is a malloc'd, NUL-terminated message owned by
 *     the caller and released with eos_b200_free_cstring (eosCudaFreeCString, :1378-1382);
 *   - handles are opaque, C-allocated and explicitly destroyed; no caller pointer is retained
 *     after a call returns (bind calls copy what they need to the device);
 *   - every call makes its runtime's device current first, so calls may come from any OS thread
 *     (the Go runtime migrates goroutines); one call in flight per handle, as the reference's
 *     mutexes guarantee (runtime/backends/cuda/cuda.go:401-402);
 *   - pointers named h_* are host memory, d_* device memory of the runtime's device;
 *   - there is no CPU fallback: without a compute-capability 10.x device every call fails.
 */
#ifndef EOS_B200_H
#define EOS_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define EOS_B200_API __attribute__((visibility("default")))
#else
#define EOS_B200_API
#endif

#define EOS_B200_OK 0
#define EOS_B200_ERROR 1
#define EOS_B200_DEVICE_STATUS 2

typedef struct EosB200Runtime EosB200Runtime;
typedef struct EosB200Encoder EosB200Encoder;
typedef struct EosB200EmbedPooled EosB200EmbedPooled;
typedef struct EosB200Quantizer EosB200Quantizer;
typedef struct EosB200Corpus EosB200Corpus;
typedef struct EosB200IpCorpus EosB200IpCorpus;
typedef struct EosB200TokenPool EosB200TokenPool;

/* Accounting of one call; mirrors the fields of backend.ExecutionAccounting that the reference
 * fills per run (runtime/backend/backend.go:1364-1400): launches, bytes moved, device time. */
typedef struct {
    int32_t kernel_launches;   /* kernels of this library launched by the call */
    int32_t reserved;
    int64_t uploaded_bytes;    /* host -> device */
    int64_t downloaded_bytes;  /* device -> host */
    int64_t valid_tokens;      /* encoder: rows actually computed (mask != 0) */
    float device_ms;           /* CUDA-event time of the call's device work (0 for *_device calls) */
    float reserved2;
} EosB200Stats;

typedef struct {
    int32_t device;
    int32_t cc_major, cc_minor;
    int32_t sm_count;
    int64_t total_memory_bytes;
    char name[128];
} EosB200DeviceInfo;

/* ---------------------------------------------------------------------------------------------
 * runtime
 * ------------------------------------------------------------------------------------------- */

/* Replaces newDeviceRuntime / eosCudaRuntimeCreate (native_linux.go:150-260, 3127): binds the
 * device, creates one stream.  Fails unless the device is compute capability 10.x. */
EOS_B200_API int eos_b200_runtime_create(int device, EosB200Runtime** out, char** err);
EOS_B200_API void eos_b200_runtime_destroy(EosB200Runtime* rt);
EOS_B200_API int eos_b200_runtime_info(EosB200Runtime* rt, EosB200DeviceInfo* out, char** err);
/* No counterpart in Eos.  Every wait inside this library's pipelined kernels is bounded: when it runs out the
 * kernel leaves, sets the runtime's device status word, and the host call that reads it returns
 * EOS_B200_DEVICE_STATUS ("pipeline timeout") instead of a result.  This self-test exercises exactly that path
 * without touching any data: one warp waits, with a limit of limit_cycles SM clocks (at most 2e8, about 0.1 s),
 * on a barrier nothing ever completes.  Expected return: EOS_B200_DEVICE_STATUS; the runtime stays usable. */
EOS_B200_API int eos_b200_selftest_bounded_wait(EosB200Runtime* rt, int64_t limit_cycles, char** err);
/* eosCudaFreeCString, native_linux.go:1378-1382 */
EOS_B200_API void eos_b200_free_cstring(char* s);
EOS_B200_API const char* eos_b200_version(void);

/* ---------------------------------------------------------------------------------------------
 * weights
 * ------------------------------------------------------------------------------------------- */

/* A dense weight in HF [out, in] layout (runtime/backend/bert_encoder_layer_ops.go:452-462).
 * Either q8: int8 codes + scales with the grid of runtime/embedding_trainer.go:11413-11446 /
 * runtime/weight_file.go:305-356 (value = code * scale; n_scales = 1 for the reference's
 * per-tensor scale, = rows for per-output-channel scales), or dense fp32 values (rounded to f16
 * on upload) when q8_codes is NULL. */
typedef struct {
    int32_t rows, cols;
    const int8_t* q8_codes;
    const float* q8_scales;
    int32_t n_scales;
    int32_t reserved;
    const float* dense;
} EosB200Matrix;

/* The 16 tensors of one encoder layer in the order of
 * runtime/pretrained_bert_importer.go:936-951. */
typedef struct {
    EosB200Matrix query;      const float* query_bias;
    EosB200Matrix key;        const float* key_bias;
    EosB200Matrix value;      const float* value_bias;
    EosB200Matrix attn_out;   const float* attn_out_bias;
    const float* attn_ln_gamma; const float* attn_ln_beta;
    EosB200Matrix inter;      const float* inter_bias;
    EosB200Matrix out;        const float* out_bias;
    const float* out_ln_gamma;  const float* out_ln_beta;
} EosB200EncoderLayer;

#define EOS_B200_ACT_GELU_ERF 0   /* exactGELU, bert_encoder_layer_ops.go:742-744 */
#define EOS_B200_ACT_GELU_TANH 1  /* geluTensor, runtime/backend/tensor_ops.go:1926-1934 */
#define EOS_B200_POOL_MASKED_MEAN 0
#define EOS_B200_POOL_CLS 1
#define EOS_B200_WEIGHTS_Q8_SMEM_DEQUANT 0 /* 8-bit codes stay 8-bit in HBM; expanded in shared memory */
#define EOS_B200_WEIGHTS_F16_RESIDENT 1    /* codes expanded to f16 once at bind */

/* What StepBERTEmbedder carries (runtime/backend/tensor_ops.go:102-136; attributes
 * num_attention_heads, epsilon, pooling per runtime/pretrained_bert_importer.go:920-984).
 * Embedding tables are fp32 arrays as backend.Tensor holds them (runtime/backend/tensor.go:11-19)
 * and are stored as f16 on the device. */
typedef struct {
    int32_t layers, hidden, heads, intermediate;
    int32_t vocab, max_positions, type_vocab;
    int32_t activation;        /* EOS_B200_ACT_* */
    int32_t pooling;           /* EOS_B200_POOL_* */
    int32_t weight_mode;       /* EOS_B200_WEIGHTS_* (q8 layers only) */
    int32_t attention_window;  /* 0 = full attention; > 0: local window (extension, not in Eos) */
    int32_t head_out;          /* 0 = no projection head */
    double epsilon;            /* LayerNorm epsilon, default 1e-12 (tensor_ops.go:1434-1447) */
    const float* token_embeddings;     /* [vocab, hidden] */
    const float* position_embeddings;  /* [max_positions, hidden] */
    const float* type_embeddings;      /* [type_vocab, hidden] */
    const float* embedding_ln_gamma;
    const float* embedding_ln_beta;
    const EosB200EncoderLayer* layer;  /* [layers] */
    const float* head_weights;         /* [hidden, head_out], in-major, no bias
                                          (runtime/pretrained_bert_projection_head.go:84-100) */
} EosB200EncoderDesc;

/* ---------------------------------------------------------------------------------------------
 * q8 encoder forward
 * ------------------------------------------------------------------------------------------- */

/* Replaces the weight binding of Backend.load / bindBGEFullEncoder (runtime/backends/cuda/
 * cuda.go:70-112, 174-228): validates shapes, copies every tensor to the device once. */
EOS_B200_API int eos_b200_encoder_bind(EosB200Runtime* rt, const EosB200EncoderDesc* desc, EosB200Encoder** out, char** err);
EOS_B200_API void eos_b200_encoder_destroy(EosB200Encoder* enc);
/* Pre-allocates the activation workspace for batches up to [batch, tokens]. */
EOS_B200_API int eos_b200_encoder_reserve(EosB200Encoder* enc, int batch, int tokens, char** err);

/* Replaces dispatchStep(StepBERTEmbedder) -> runBGEFullEncoderHidden (cuda.go:394-452,
 * native_linux.go:7941-8190) and the host path BERTEmbedderReferenceWithPooling
 * (runtime/backend/bert_embedder_ops.go:101-197) [+ PretrainedBERTProjectionHead.Apply].
 * h_ids/h_mask/h_types are [batch, tokens] int32 (h_types may be NULL = all zero); h_out is
 * [batch, E] fp32, E = head_out or hidden.  Out-of-range ids return EOS_B200_DEVICE_STATUS
 * (tensor_ops.go:1479-1487); an all-masked sequence yields a zero vector.
 * The forward is captured into a CUDA graph the first time a [batch, tokens] shape is seen and replayed afterwards
 * (one launch call instead of 92 for 12 layers; EOS_B200_NO_GRAPHS=1 turns this off). */
EOS_B200_API int eos_b200_encoder_run(EosB200Encoder* enc, const int32_t* h_ids, const int32_t* h_mask, const int32_t* h_types,
                         int batch, int tokens, float* h_out, EosB200Stats* stats, char** err);
/* The same forward without waiting for it: the uploads, the kernels and the download of h_out are enqueued on the
 * runtime's stream and the call returns; eos_b200_encoder_wait blocks until every submitted batch is complete and
 * reports the first device status raised by any of them.  A host that has the next batch ready keeps the GPU busy
 * across the copies this way (EmbedBatch callers that loop over batches, runtime/embedding_model.go:664-700).
 * h_ids / h_mask / h_types must not be modified and h_out not read before the wait; buffers of different batches in
 * flight must be distinct; for the copies to overlap the host buffers have to be page-locked.  stats of the wait:
 * launches and bytes of all the batches waited for. */
EOS_B200_API int eos_b200_encoder_submit(EosB200Encoder* enc, const int32_t* h_ids, const int32_t* h_mask,
                                         const int32_t* h_types, int batch, int tokens, float* h_out, char** err);
EOS_B200_API int eos_b200_encoder_wait(EosB200Encoder* enc, EosB200Stats* stats, char** err);

/* ---- compact encoder profile ----------------------------------------------------------------
 * The native q8 encoder graph of models/default_embedding.go:461-505 (pipeline embed_pooled_batch):
 * gather(token_embedding) + gather(role_embedding) -> rope (runtime/backend/tensor_ops.go:1936-1965)
 * -> per layer { q, k, v = h @ W (no bias); multi-head attention over the unmasked keys
 * (compactMultiheadAttentionTensor, tensor_ops.go:1867-1924); @ Wo; layernorm(attended + h)
 * (non-affine, epsilon 1e-5, tensor_ops.go:1393-1421); tanh-GELU FFN (tensor_ops.go:1926-1934);
 * layernorm(projected + attn_hidden) } -> per-token L2 normalize -> optional output projection ->
 * masked mean pool (the result is not re-normalised).
 * Weights are in Eos's matmul layout [in, out] (EosB200Matrix.rows = in, .cols = out); a q8 matrix
 * has n_scales = 1 (the reference's per-tensor scale) or = cols (per output channel).  The bound
 * handle is an EosB200Encoder: run / run_device / sync / profile / destroy are the entry points
 * above, with the role ids passed where the token type ids go. */
typedef struct {
    EosB200Matrix attn_q, attn_k, attn_v, attn_o;  /* [hidden, hidden] */
    EosB200Matrix ffn_up;                          /* [hidden, intermediate] */
    EosB200Matrix ffn_down;                        /* [intermediate, hidden] */
} EosB200CompactLayer;

typedef struct {
    int32_t layers, hidden, heads, intermediate;
    int32_t vocab, role_vocab;
    int32_t output_dim;            /* 0 or hidden: no output projection */
    int32_t weight_mode;           /* EOS_B200_WEIGHTS_* */
    const float* token_embedding;  /* [vocab, hidden], dequantised values */
    const float* role_embedding;   /* [role_vocab, hidden] */
    const EosB200CompactLayer* layer;
    EosB200Matrix output_projection;  /* [hidden, output_dim]; ignored without a projection */
} EosB200CompactEncoderDesc;

EOS_B200_API int eos_b200_compact_encoder_bind(EosB200Runtime* rt, const EosB200CompactEncoderDesc* desc, EosB200Encoder** out,
                                               char** err);

/* Same forward with inputs and output resident in device memory; enqueued on `stream`
 * (a cudaStream_t; NULL = the runtime's stream) without synchronising.  The device status word
 * is read by eos_b200_encoder_sync. */
EOS_B200_API int eos_b200_encoder_run_device(EosB200Encoder* enc, const int32_t* d_ids, const int32_t* d_mask,
                                const int32_t* d_types, int batch, int tokens, float* d_out, void* stream,
                                EosB200Stats* stats, char** err);
/* Per-token output vectors (the long-context multi-vector document path; no single counterpart in Eos, whose
 * multi-vector documents come from span pooling, runtime/sparse_token_pool_vector_export.go): a projection
 * [hidden, token_dim] (in-major, no bias, as a projection head is stored) applied to every valid token's final
 * hidden row, then L2 normalisation.  set_token_head is called once after bind (the CLS-pooling row layout is
 * not supported together with it).  token_vectors_device runs the forward on `stream` and writes the vectors of
 * the valid tokens, sequence after sequence in token order, to d_vectors [rows, token_dim] fp32 (rows <=
 * batch * tokens; the count is written to d_row_count when non-null); they are the input of
 * eos_b200_quantize_device. */
EOS_B200_API int eos_b200_encoder_set_token_head(EosB200Encoder* enc, const float* h_weights, int token_dim, char** err);
EOS_B200_API int eos_b200_encoder_token_vectors_device(EosB200Encoder* enc, const int32_t* d_ids, const int32_t* d_mask,
                                                       const int32_t* d_types, int batch, int tokens, float* d_vectors,
                                                       int32_t* d_row_count, void* stream, EosB200Stats* stats, char** err);
/* Per-kernel-class device time of the forwards enqueued between profile_begin and profile_end,
 * taken with CUDA events recorded around every launch on the launching stream.  The reference
 * keeps the same kind of evidence as CUDA-event phase pairs (native_linux.go:285-498,
 * EOS_CUDA_COMPACT_PROFILE_EVENTS).  Times are totals over `steps` forwards. */
typedef struct {
    int32_t steps;
    int32_t gemm_launches, attention_launches, layernorm_launches, other_launches;
    float gemm_ms, attention_ms, layernorm_ms, embed_ms, pool_ms, layout_ms;
    float gemm_kind_ms[4];     /* fused QKV, attention output, FFN up, FFN down */
} EosB200EncoderTimes;
EOS_B200_API int eos_b200_encoder_profile_begin(EosB200Encoder* enc, int max_steps, char** err);
EOS_B200_API int eos_b200_encoder_profile_end(EosB200Encoder* enc, void* stream, EosB200EncoderTimes* out, char** err);

/* Waits for `stream` and returns EOS_B200_DEVICE_STATUS if a kernel flagged an error. */
EOS_B200_API int eos_b200_encoder_sync(EosB200Encoder* enc, void* stream, char** err);

/* Replaces MatMulAccelerator / runMatMulWithBoundRight for one dense projection
 * (runtime/backend/backend.go:785-795, native_linux.go:9286-9372) with denseHF semantics:
 * h_y[rows, w.rows] = epilogue(h_x[rows, w.cols] x W^T + bias).  epilogue: 0 = none, 1 = erf GELU,
 * 2 = + h_residual, 3 = tanh GELU.  x and residual are rounded to f16 on upload, y is f16-rounded. */
EOS_B200_API int eos_b200_linear(EosB200Runtime* rt, const float* h_x, int64_t rows, const EosB200Matrix* w, const float* h_bias,
                    int epilogue, const float* h_residual, int weight_mode, float* h_y, EosB200Stats* stats,
                    char** err);

/* ---------------------------------------------------------------------------------------------
 * compiled pipeline: gather -> matmul -> normalize -> masked mean_pool
 * (examples/embed_masked_pooled.eos:11-16; steps executed by ExecuteSymbolic,
 * runtime/backend/symbolic.go:17-172, with gatherTensor / matmulTensor / normalizeRows /
 * meanPoolMaskedTensor of runtime/backend/tensor_ops.go)
 * ------------------------------------------------------------------------------------------- */
EOS_B200_API int eos_b200_embed_pooled_bind(EosB200Runtime* rt, const float* h_table, int vocab, int dim,
                               const float* h_projection, int out_dim, EosB200EmbedPooled** out, char** err);
EOS_B200_API void eos_b200_embed_pooled_destroy(EosB200EmbedPooled* ep);
/* The matmul step's `scale` attribute (matmulScale / ApplyMatMulAttributes, runtime/backend/tensor_ops.go:1259-1315):
 * the caller resolves "rsqrt_rhs_rows" (1 / sqrt(dim)) or the literal to a number; the projected rows are multiplied by
 * it in fp32 before the normalisation.  Default 1. */
EOS_B200_API int eos_b200_embed_pooled_set_matmul_scale(EosB200EmbedPooled* ep, float scale, char** err);
/* pool_then_l2 = 0: the pipeline's order (normalize each token, then mean);
 * 1: mean of the projected rows, then one L2 normalisation. h_out [batch, out_dim] fp32. */
EOS_B200_API int eos_b200_embed_pooled_run(EosB200EmbedPooled* ep, const int32_t* h_tokens, const int32_t* h_mask, int batch,
                              int tokens, int pool_then_l2, float* h_out, EosB200Stats* stats, char** err);

/* ---------------------------------------------------------------------------------------------
 * TurboQuant (Hadamard/MSE variant): packing, scoring, top-k
 * ------------------------------------------------------------------------------------------- */

/* Holds the rotation spec {perm, signs1, signs2, centroids, boundaries} exactly as the
 * reference's turboquant Spec() exposes it (native_linux.go:9532-9545), so a Go host that owns
 * the real module can pass its own tables.  bits in {2, 4}; the centroid table must be
 * symmetric (centroids[L-1-i] == -centroids[i]). */
EOS_B200_API int eos_b200_quantizer_create(EosB200Runtime* rt, int dim, int bits, const int32_t* perm, const float* signs1,
                              const float* signs2, const float* centroids, const float* boundaries,
                              EosB200Quantizer** out, char** err);
EOS_B200_API void eos_b200_quantizer_destroy(EosB200Quantizer* qz);

/* Replaces the corpus loop `for doc: q.Quantize(doc)` (runtime/retrieval_turboquant.go:700-711):
 * h_x [n, dim] fp32 -> h_codes [n, dim*bits/8] (codes little-end first inside a byte, the nibble
 * order of runtime/mll_export.go:950-960) and h_norms [n]. */
EOS_B200_API int eos_b200_quantize(EosB200Quantizer* qz, const float* h_x, int64_t n, uint8_t* h_codes, float* h_norms,
                      EosB200Stats* stats, char** err);
EOS_B200_API int eos_b200_quantize_device(EosB200Quantizer* qz, const float* d_x, int64_t n, uint8_t* d_codes, float* d_norms,
                             void* stream, char** err);

/* Replaces the qdocs slice built at runtime/retrieval_turboquant.go:702-711: copies the packed
 * rows to the device once and converts them to the scan layout.  Row i has document id
 * id_base + i; callers assign rows in ascending id order so that "score descending, then id
 * ascending" (runtime/retrieval_eval.go:1153-1161) is the order of the results.
 * Norm rule of runtime/turboquant_quantized_vector.go:25-49: a norm <= 0 or non-finite is rejected
 * unless allow_zero_norm != 0. */
EOS_B200_API int eos_b200_corpus_bind(EosB200Quantizer* qz, const uint8_t* h_codes, const float* h_norms, int64_t n,
                         int64_t id_base, int allow_zero_norm, EosB200Corpus** out, char** err);
EOS_B200_API int eos_b200_corpus_bind_device(EosB200Quantizer* qz, const uint8_t* d_codes, const float* d_norms, int64_t n,
                                int64_t id_base, EosB200Corpus** out, char** err);
EOS_B200_API void eos_b200_corpus_destroy(EosB200Corpus* corpus);
/* runtime/turboquant_bytes.go:22-25 accounting: packed bytes per vector incl. the f32 norm. */
EOS_B200_API int64_t eos_b200_corpus_vector_bytes(const EosB200Corpus* corpus);

/* Replaces PrepareQuery + topTurboQuantRetrievalScoresWithStats per query
 * (runtime/retrieval_turboquant.go:1324-1325, 1853-1887) for the Hadamard/MSE stage of the quantiser only:
 * exact top-k of norm * <R q, centroids[codes]> over the corpus, for q_count queries [q_count, dim] fp32.
 * The reference's IPQuantizer adds a QJL sign stage (Signs, ResNorm) on top of the MSE codes; those two
 * operands are not accepted here (rows that carry them bind with eos_b200_ip_corpus_bind below).
 * queries_per_pass selects how many queries share one pass over the codes, and with it the kernel:
 *   0        automatic: 8 up to 8 queries, 128 up to 128 queries, 256 above;
 *   8        streaming scan (codes expanded in registers, mma.sync): the choice for a few queries;
 *   16, 32   the same scan with more query fragments per pass;
 *   128, 256 batch kernels on the tensor cores (codes expanded once per 128 / 256 queries into a
 *            tcgen05 operand tile): the choice for hundreds of queries (256 is the faster one once
 *            q_count exceeds 128); q_count need not be a multiple.
 * Every value gives the exact top-k of the scores its kernel computes; the kernels round differently (their scores
 * agree to about 1e-6 relative), so neighbours whose scores are closer than that may come out in either order.
 * Results [q_count, k]: ids (int64, -1 when the corpus has fewer than k rows) and scores, ordered
 * score descending then id ascending.  k <= 128 on the fused kernels; this host call also takes k in (128, 256]
 * (the over-fetch before a rerank, runtime/retrieval_turboquant.go:1610-1662: 200 candidates for a top-100): on a
 * corpus large enough for seeded thresholds one pass of the 256-query kernel answers every query whose candidate
 * lists were never cut; the others (stats->reserved counts them) and small corpora are answered by materialising the
 * scores of a chunk of queries and selecting once per query. */
EOS_B200_API int eos_b200_score_topk(EosB200Corpus* corpus, const float* h_queries, int q_count, int k, int queries_per_pass,
                        int64_t* h_ids, float* h_scores, EosB200Stats* stats, char** err);
/* Device-resident variant, enqueued on `stream`.  d_keys (nullable, [q_count, k] uint64) receives
 * the sortable (score, id) keys that eos_b200_topk_merge_device consumes after an all-gather.
 * d_ids and d_scores are given together or are both null (keys only); at least one output is required.
 * The call returns after enqueueing; eos_b200_corpus_sync waits for the stream and reports a kernel-side
 * timeout. */
EOS_B200_API int eos_b200_score_topk_device(EosB200Corpus* corpus, const float* d_queries, int q_count, int k,
                               int queries_per_pass, int64_t* d_ids, float* d_scores, uint64_t* d_keys, void* stream,
                               EosB200Stats* stats, char** err);
/* No counterpart in Eos (its scoring is per process): the two halves of the batch scoring call, for a corpus
 * sharded over several GPUs.  A threshold seeded on ANY shard (the k-th best score of a sample of that shard) is a
 * lower bound of the k-th best score of the whole corpus, so the ranks may split the work of seeding -- rank r calls
 * eos_b200_score_seed_device for its slice of the queries, the slices are all-gathered (8 bytes per query) -- and
 * every rank then scores with all thresholds.  The per-shard result is that shard's part of the global top-k (it
 * may hold fewer than k entries; the rest are empty keys), which is what eos_b200_topk_merge_device needs.
 * d_tau_out / d_tau: [q_count] uint64 keys, 0 = no threshold. */
EOS_B200_API int eos_b200_score_seed_device(EosB200Corpus* corpus, const float* d_queries, int q_count, int k,
                               uint64_t* d_tau_out, void* stream, char** err);
EOS_B200_API int eos_b200_score_topk_seeded_device(EosB200Corpus* corpus, const float* d_queries, int q_count, int k,
                                      const uint64_t* d_tau, int64_t* d_ids, float* d_scores, uint64_t* d_keys,
                                      void* stream, EosB200Stats* stats, char** err);
/* Waits for `stream` (null: the runtime's stream) and returns EOS_B200_DEVICE_STATUS if a kernel enqueued by
 * one of the *_device / _noalloc scoring calls gave up on a bounded wait; counterpart of eos_b200_encoder_sync. */
EOS_B200_API int eos_b200_corpus_sync(EosB200Corpus* corpus, void* stream, char** err);
/* (eos_b200_score_topk_noalloc below takes queries_per_pass in {8, 16, 32} only.) */
/* No counterpart in Eos: a scoring call for hosts that must not allocate device memory while they
 * serve queries -- for example a caller that holds the GPU inside a pre-sized memory arena, runs
 * with allocation forbidden after start-up, or sits on a latency path where a cudaMalloc (which can
 * synchronise the whole device) is unacceptable.  Same result as eos_b200_score_topk_device, but
 * every byte of scratch (query fragments, per-CTA candidate lists and their counts) lives in one
 * file-scope __device__ array inside the library instead of in memory the corpus handle
 * allocates on demand.  The call itself performs no cudaMalloc / cudaFree and calls no allocating
 * routine; the caller passes the device buffers for queries, ids and scores.
 * Limits: q_count <= 32, dim <= 1024, k <= 128, at most 160 SMs; larger requests are rejected
 * with an error, nothing is truncated.  The array is about 5.1 MB and is resident on every GPU
 * that loads the library until the process exits.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress); make
 * that first call before starting any stream capture.  All calls on a device share the array and
 * it keeps the previous call's contents: calls whose GPU work overlaps (two streams, two
 * threads, two corpora) race on it, so keep them ordered on one stream. */
EOS_B200_API int eos_b200_score_topk_noalloc(EosB200Corpus* corpus, const float* d_queries, int q_count, int k,
                                             int queries_per_pass, int64_t* d_ids, float* d_scores, void* stream,
                                             char** err);

/* Device time of the scan kernel alone (CUDA events around every scan launch between begin and
 * end): out_ms = total milliseconds, out_launches = scan launches covered. */
EOS_B200_API int eos_b200_corpus_profile_begin(EosB200Corpus* corpus, int max_launches, char** err);
EOS_B200_API int eos_b200_corpus_profile_end(EosB200Corpus* corpus, void* stream, float* out_ms, int* out_launches,
                                             char** err);

/* Global top-k from `shards` per-shard key lists gathered as d_keys [shards, q_count, k]
 * (one NCCL all-gather of the per-GPU results).  Keys carry global document ids. */
EOS_B200_API int eos_b200_topk_merge_device(EosB200Runtime* rt, const uint64_t* d_keys, int shards, int q_count, int k,
                               int64_t* d_ids, float* d_scores, void* stream, char** err);
/* ---- corpus sharded over several GPUs (one process per GPU) ------------------------------------
 * No counterpart in Eos (its scoring runs in one process).  The exchange steps -- thresholds, then per-shard
 * candidate lists -- are NCCL all-gathers issued by the library itself, so a host without any collective
 * library of its own (the Go host) only has to hand the 128-byte NCCL id from rank 0 to the other ranks.
 * NCCL (libnccl.so.2) is loaded when the first of these calls is made; everything else works without it. */
typedef struct { char internal[128]; } EosB200NcclId;   /* layout of ncclUniqueId */
typedef struct EosB200Comm EosB200Comm;
/* Rank 0 calls this once and distributes the id (a file, a socket, an environment of the launcher). */
EOS_B200_API int eos_b200_comm_unique_id(EosB200NcclId* out, char** err);
/* Collective over all `world` ranks (ncclCommInitRank); the runtime's device is the rank's GPU. */
EOS_B200_API int eos_b200_comm_init(EosB200Runtime* rt, int rank, int world, const EosB200NcclId* id, EosB200Comm** out,
                                    char** err);
EOS_B200_API void eos_b200_comm_destroy(EosB200Comm* comm);
/* Collective: every rank calls it with its own shard (rows in ascending global id order across ranks, id_base
 * = the shard's first id; an empty shard is allowed) and the same queries; every rank receives the exact global
 * top-k.  Sequence, all on `stream`: each rank seeds the pruning thresholds of its slice of the queries from its
 * own shard -> all-gather of the thresholds (8 bytes per query) -> batch scoring of the shard with all
 * thresholds -> all-gather of the per-shard key lists (q_count * k * 8 bytes per rank) -> merge kernel.
 * queries_per_pass as in eos_b200_score_topk (8 / 16 / 32: the streaming scan, without the threshold exchange).
 * Enqueues only; eos_b200_corpus_sync reports kernel-side timeouts.  No peer-memory loads, no multicast. */
EOS_B200_API int eos_b200_score_topk_sharded(EosB200Corpus* corpus, EosB200Comm* comm, const float* d_queries, int q_count,
                                             int k, int queries_per_pass, int64_t* d_ids, float* d_scores, void* stream,
                                             EosB200Stats* stats, char** err);
/* Late interaction (MaxSim) over a corpus of child vectors with a fixed number of children per parent
 * (the long-context multi-vector layout: a document is a run of children_per_parent consecutive rows; rows of
 * a document that do not exist are bound with a norm of NaN and score nothing).  Extension of
 * topTurboQuantMultiVectorParentScores (runtime/retrieval_multivector_turboquant.go:746-810, "max" aggregation):
 * for each query (query_group consecutive query vectors, a power of two <= 32) and each parent,
 *     score = sum over the query's vectors of max over the parent's children of norm * <R q, centroids[codes]>,
 * exact top-k over parents, score descending then parent id ascending; parent id = (id_base + row) /
 * children_per_parent.  d_queries [q_vectors, dim] fp32 on the device; results [q_vectors / query_group, k].
 * One tensor-core pass over the shard per 128 query vectors; children_per_parent in {16, 32, 64, 128}.
 * The general layout (any parent_of_child map, top-n mean, penalty) stays with eos_b200_parent_topk. */
EOS_B200_API int eos_b200_maxsim_topk_device(EosB200Corpus* corpus, const float* d_queries, int q_vectors, int query_group,
                                             int children_per_parent, int k, int64_t* d_ids, float* d_scores,
                                             uint64_t* d_keys, void* stream, EosB200Stats* stats, char** err);
/* Collective: all-gather of every rank's key lists [q_count, k] (as eos_b200_*_device calls emit them in d_keys)
 * and the merge into the global top-k, for results sharded in any other way than eos_b200_score_topk_sharded's
 * (for instance eos_b200_maxsim_topk_device over parents sharded across GPUs). */
EOS_B200_API int eos_b200_comm_merge_keys(EosB200Comm* comm, const uint64_t* d_keys, int q_count, int k, int64_t* d_ids,
                                          float* d_scores, void* stream, char** err);
/* Dense scores of a few queries against every row (no top-k), for parity checks and rerank
 * candidates: h_scores [q_count, n]. */
EOS_B200_API int eos_b200_score_all(EosB200Corpus* corpus, const float* h_queries, int q_count, float* h_scores, char** err);

/* ---- dense candidates ------------------------------------------------------------------------
 * Uncompressed document vectors on the device, for the dense scoring operators and the rerank
 * stage that follows a TurboQuant top-k.  h_vectors [n, dim] fp32 (dim <= 1024); store_f16 != 0
 * keeps them rounded to f16 (the fp16 rerank sidecar: topFP16RerankScores reads uint16 halves,
 * runtime/retrieval_turboquant.go:1637-1662), else as fp32 (topDenseRerankScores, :1610-1635). */
typedef struct EosB200DenseIndex EosB200DenseIndex;
EOS_B200_API int eos_b200_dense_bind(EosB200Runtime* rt, const float* h_vectors, int64_t n, int dim, int store_f16,
                                     EosB200DenseIndex** out, char** err);
EOS_B200_API void eos_b200_dense_destroy(EosB200DenseIndex* index);
#define EOS_B200_METRIC_DOT 0    /* dotRows, runtime/backend/tensor_ops.go:1967-1995; kernel body compiler/compiler.go:838-846 */
#define EOS_B200_METRIC_COSINE 1 /* cosineRows, tensor_ops.go:1997-2057 (0 when a norm is 0); compiler.go:847-862 */
/* Every query against every row, then topKTensor (tensor_ops.go:2124-2193: score descending,
 * ties to the lower row).  h_queries [q_count, dim] fp32; results [q_count, k], k <= 128, k <= n. */
EOS_B200_API int eos_b200_dense_score_topk(EosB200DenseIndex* index, const float* h_queries, int q_count, int metric, int k,
                                           int64_t* h_ids, float* h_scores, EosB200Stats* stats, char** err);
/* Rerank: for each query the dot product (fp32 accumulate) with its candidate rows only, then the
 * k best by score descending / row ascending, as the rerank loops of retrieval_turboquant.go:1610-1662
 * do with a heap.  h_candidates [q_count, cand] row indices; a negative or out-of-range entry is a
 * candidate without a vector (skipped, like a missing map entry).  Slots past the number of valid
 * candidates hold id -1 and score -infinity. */
EOS_B200_API int eos_b200_dense_rerank(EosB200DenseIndex* index, const float* h_queries, int q_count, const int64_t* h_candidates,
                                       int cand, int k, int64_t* h_ids, float* h_scores, EosB200Stats* stats, char** err);

/* Multi-vector parents (topTurboQuantMultiVectorParentScores,
 * runtime/retrieval_multivector_turboquant.go:746-810, 890-907): rows of the corpus are child
 * vectors, h_parent_of_child [n] maps each to its parent in [0, parents).  Per query vector the
 * parent score is the mean of its best min(top_n, 5, children) child scores (top_n <= 1: max)
 * minus penalty * log1p(children); query_group > 1 sums the parent scores of that many
 * consecutive query vectors (late-interaction MaxSim; extension, not in Eos).
 * Results [q_count / query_group, k]. */
EOS_B200_API int eos_b200_parent_topk(EosB200Corpus* corpus, const int32_t* h_parent_of_child, int parents, const float* h_queries,
                         int q_count, int query_group, int top_n, double penalty, int k, int64_t* h_ids,
                         float* h_scores, EosB200Stats* stats, char** err);

/* ---- rows quantised by the inner-product quantiser ---------------------------------------------
 * turboquant.IPQuantized{MSE, Signs, ResNorm, Norm} (runtime/turboquant_quantized_vector.go:43-49; scored by
 * IPQuantizer.InnerProductPrepared at runtime/retrieval_turboquant.go:1874): an MSE stage of bit_width - 1 bits, one
 * QJL sign bit per coordinate of the projected residual, the residual's norm and the input's norm.  The module that
 * produces them (m31labs.dev/turboquant) is not part of the reference tree, so this library takes the fields from a
 * host that has it and scores
 *     Norm * ( <R q, centroids[MSE]>  +  ResNorm * qjl_scale * sum_i sketch_q[i] * (Signs bit i ? +1 : -1) )
 * where R q is the rotation of the query by (perm, signs1, signs2), and sketch_q (the query under the module's sign
 * projection) and qjl_scale (sqrt(pi / 2) / dim in the published algorithm) come from the caller per query batch.
 * h_mse_indices [n, dim]: one level index per byte, < mse_levels (2, 4, 8 or 16; centroids ascending and symmetric);
 * h_signs [n, ceil(dim / 8)]: bit i of a row at byte i / 8, bit i % 8; h_resnorms, h_norms [n].
 * Norm rule as eos_b200_corpus_bind (validateEosQuantizedVectorNorm, :26-34).  eos_b200_ip_corpus_vector_bytes is
 * turboquantVectorBytes (runtime/turboquant_bytes.go:22-25): 392 at dim 768, bit width 4. */
EOS_B200_API int eos_b200_ip_corpus_bind(EosB200Runtime* rt, int dim, int mse_levels, const int32_t* perm, const float* signs1,
                                         const float* signs2, const float* centroids, const uint8_t* h_mse_indices,
                                         const uint8_t* h_signs, const float* h_resnorms, const float* h_norms, int64_t n,
                                         int64_t id_base, int allow_zero_norm, EosB200IpCorpus** out, char** err);
EOS_B200_API void eos_b200_ip_corpus_destroy(EosB200IpCorpus* corpus);
EOS_B200_API int64_t eos_b200_ip_corpus_vector_bytes(int dim, int bit_width);
/* The 8-bit log-scale norm side-car of the reference's device encode (manta_tq_quantize_norm /
 * manta_tq_dequantize_norm, runtime/backends/cuda/native_linux.go:1879-1904): code = round(255 (ln norm + 16) / 32)
 * clamped to [0, 255], norm = exp(-16 + 32 code / 255).  Host arithmetic; eos_b200_corpus_bind takes the decoded
 * norms, eos_b200_turbo_sparse_attention takes the codes. */
EOS_B200_API void eos_b200_norm_encode_log8(const float* norms, int64_t n, uint8_t* codes);
EOS_B200_API void eos_b200_norm_decode_log8(const uint8_t* codes, int64_t n, float* norms);
/* Exact top-k (k <= 256) of the score above for q_count queries; results as eos_b200_score_topk. */
EOS_B200_API int eos_b200_ip_score_topk(EosB200IpCorpus* corpus, const float* h_queries, const float* h_query_sketch,
                                        float qjl_scale, int q_count, int k, int64_t* h_ids, float* h_scores,
                                        EosB200Stats* stats, char** err);

/* ---- sparse attention ---------------------------------------------------------------------------
 * Replaces sparseAttentionTensor (runtime/backend/attention_ops.go:218-276; device twin
 * sparseAttentionKernelSource, runtime/backends/cuda/native_linux.go:2044-2339).  h_query [batches, q_len, dim],
 * h_key [batches, k_len, dim], h_value [batches, k_len, value_dim], h_out [batches, q_len, value_dim], fp32; a
 * rank-2 call passes batches = 1.  Per query row: scores q.k in fp32 (no 1/sqrt(d)); the best keys by score
 * descending then index ascending, as many as top_k (<= 0: ceil(sqrt(k_len))), clamped to [1, k_len];
 * route_block_size, route_top_blocks > 0 first keep the route_top_blocks key blocks whose middle key scores best
 * (block_anchor routing, :462-497); softmax over the selected scores; their values mixed in selection order.
 * k_len = 0 gives zeros.  Limits: the key budget and route_top_blocks at most 128 (EOS_SPARSE_ATTENTION_MAX_TOPK). */
EOS_B200_API int eos_b200_sparse_attention(EosB200Runtime* rt, const float* h_query, const float* h_key, const float* h_value,
                                           int batches, int q_len, int k_len, int dim, int value_dim, int top_k,
                                           int route_block_size, int route_top_blocks, float* h_out, EosB200Stats* stats,
                                           char** err);
/* Replaces turboSparseAttentionTensor (attention_ops.go:278-300): the keys and values arrive TurboQuant-compressed
 * -- codes [batches, k_len, dim] one byte per coordinate (the reference's coords tensor [B, D, T, 1] in sequence
 * order) and 8-bit log-scale norm codes [batches, k_len] (native_linux.go:1879-1904) -- and are decoded on the
 * device (manta_turboq_decode, :1959-2003) before the same attention.  key_qz / value_qz carry the rotation
 * specs of the key and value widths (the same handle when both widths are equal). */
EOS_B200_API int eos_b200_turbo_sparse_attention(EosB200Quantizer* key_qz, EosB200Quantizer* value_qz, const float* h_query,
                                                 const uint8_t* h_key_codes, const uint8_t* h_key_norm_codes,
                                                 const uint8_t* h_value_codes, const uint8_t* h_value_norm_codes,
                                                 int batches, int q_len, int k_len, int top_k, int route_block_size,
                                                 int route_top_blocks, float* h_out, EosB200Stats* stats, char** err);

/* ---- token-pool encoder and token-span child vectors --------------------------------------------
 * Replaces sparseTokenPoolEncoder.embedTextFullEncoderRows / embedTextFullEncoder and the span pooling of
 * writeSparseTokenPoolTokenSpanChildVectorCache (runtime/sparse_token_pool_vector_export.go:1290-1335, 802-890):
 * gather -> encoder_repeats x [single-head Q/K/V projections over the whole width, attention, output projection,
 * optional residual + non-affine LayerNorm, tanh-GELU FFN, optional residual + LayerNorm] with ONE set of weights
 * shared by all repeats -> per-token L2-normalised rows.  All tensors fp32, projections in [in, out] layout
 * (matmulRowsRight, :1620-1633); arithmetic is float in the reference's summation orders.
 * attention_mode: DENSE = denseSoftmaxAttentionRows (:1430-1465, no 1/sqrt(d)); TURBO_SPARSE = the key and value rows
 * are TurboQuant-encoded (key_qz / value_qz carry the rotation specs, codes + 8-bit log norms as
 * TurboQuantEncodeReference, runtime/backend/image_ops.go:212-249) and attended to with
 * eos_b200_turbo_sparse_attention's kernels (top_k, route_block_size, route_top_blocks as there).
 * Outputs, each optional (null = skip): h_rows [seq_len, dim]; h_pooled [dim] = maskedMeanPoolNormalized (:1534-1559);
 * h_children [n, dim] = one unit vector per token span (sparseTokenPoolTokenSpans :1561-1595 with span_tokens,
 * span_overlap, span_min_tokens; poolSparseTokenRowsRange :1597-1618), n returned in *n_children (<= max_children).
 * A span without an active token is an error, as in the reference. */
typedef struct {
    int32_t vocab, dim, hidden, encoder_repeats;
    int32_t attention_residual, attention_layer_norm, ffn_residual, ffn_layer_norm;   /* manifest flags */
    const float* token_embedding;    /* [vocab, dim] */
    const float* attention_query;    /* [dim, dim] */
    const float* attention_key;
    const float* attention_value;
    const float* attention_output;
    const float* hidden_projection;  /* [dim, hidden] */
    const float* projection;         /* [hidden, dim] */
} EosB200TokenPoolDesc;
#define EOS_B200_TOKEN_POOL_DENSE 0
#define EOS_B200_TOKEN_POOL_TURBO_SPARSE 1
EOS_B200_API int eos_b200_token_pool_bind(EosB200Runtime* rt, const EosB200TokenPoolDesc* desc, EosB200TokenPool** out,
                                          char** err);
EOS_B200_API void eos_b200_token_pool_destroy(EosB200TokenPool* tp);
EOS_B200_API int eos_b200_token_pool_encode(EosB200TokenPool* tp, const int32_t* h_tokens, const int32_t* h_mask, int seq_len,
                                            int attention_mode, EosB200Quantizer* key_qz, EosB200Quantizer* value_qz,
                                            int top_k, int route_block_size, int route_top_blocks, int span_tokens,
                                            int span_overlap, int span_min_tokens, float* h_rows, float* h_pooled,
                                            float* h_children, int max_children, int* n_children, EosB200Stats* stats,
                                            char** err);

/* Seeded synthetic data on the device (bench / tests): n rows of dim N(0,1) values, optionally
 * L2-normalised, row r generated from (seed, row_offset + r) only. */
EOS_B200_API int eos_b200_synth_gaussian_device(EosB200Runtime* rt, uint64_t seed, int64_t row_offset, int64_t n, int dim,
                                   int normalize, float* d_out, void* stream, char** err);

#ifdef __cplusplus
}
#endif
#endif /* EOS_B200_H */
