/*
 * eos_oracle.c -- CPU restatement of the Eos host reference for the query-time
 * embed-and-score path.  TEST INFRASTRUCTURE ONLY: this file is the checker that the
 * CUDA path is compared against (and the timed CPU baseline); nothing in the shipped
 * library links, loads or calls it.
 *
 * Every function cites the Eos source (path inside the Eos project : lines) whose loop
 * order and accumulation types it follows.  Accumulation widths (float vs double) and
 * summation order are kept exactly as the reference writes them.
 *
 * Parity status:
 *   - encoder functions: PINNED against Eos's own golden fixture
 *     runtime/testdata/pretrained_bert_golden/golden.json (max_abs <= 2e-3,
 *     min_cosine >= 0.9999, runtime/pretrained_bert_golden_parity_test.go:99-103) and
 *     against the hand-computed expectations in runtime/backend (tensor_ops_test.go, bert_encoder_layer_ops_test.go).
 *   - TurboQuant functions: the arithmetic lives in the third-party Go module
 *     m31labs.dev/turboquant v0.2.1 (go.mod:9) whose source is not part of the Eos tree; what is
 *     restated here is the Hadamard/MSE variant exactly as Eos's own CUDA restatement spells it
 *     (runtime/backends/cuda/native_linux.go:1812-2003), with the rotation spec (perm, signs,
 *     centroids, boundaries) supplied by the caller.  Encode (rotation + code assignment + 8-bit
 *     norm code) and decode are PINNED bit for bit against that reference code compiled for the
 *     host (oracle/build_ref.py -> oracle/_ref, tests/test_oracle_pins.py).  UNPINNED: the seed ->
 *     spec generator and the scoring of the module's IP variant (QJL signs, ResNorm), which the
 *     Eos tree does not contain.
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off, no -march flags, so that float
 * expressions are evaluated without fused multiply-add exactly as written).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define EOS_ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------ */
/* threading helper: contiguous chunks over `workers` threads, as the reference does     */
/* over GOMAXPROCS (runtime/backend/bert_encoder_layer_ops.go:243-270, 423-450).         */
/* ------------------------------------------------------------------------------------ */
typedef void (*range_fn)(void *ctx, int64_t start, int64_t end);
typedef struct {
    range_fn fn;
    void *ctx;
    int64_t start, end;
} range_job;

static void *range_thread(void *p) {
    range_job *j = (range_job *)p;
    j->fn(j->ctx, j->start, j->end);
    return NULL;
}

static void parallel_ranges(range_fn fn, void *ctx, int64_t n, int workers) {
    if (workers <= 1 || n < 2) {
        fn(ctx, 0, n);
        return;
    }
    if (workers > n) workers = (int)n;
    if (workers > 256) workers = 256;
    int64_t chunk = (n + workers - 1) / workers;
    pthread_t tids[256];
    range_job jobs[256];
    int used = 0;
    for (int64_t s = 0; s < n; s += chunk) {
        int64_t e = s + chunk;
        if (e > n) e = n;
        jobs[used].fn = fn;
        jobs[used].ctx = ctx;
        jobs[used].start = s;
        jobs[used].end = e;
        pthread_create(&tids[used], NULL, range_thread, &jobs[used]);
        used++;
    }
    for (int i = 0; i < used; i++) pthread_join(tids[i], NULL);
}

/* ------------------------------------------------------------------------------------ */
/* f16 <-> f32, as runtime/mll_export.go:1007-1044 (float32ToHalf: round-half-up on the  */
/* 13 dropped mantissa bits) and runtime/weight_file.go:461-483 (halfToFloat32).         */
/* ------------------------------------------------------------------------------------ */
EOS_ORACLE_API uint16_t eos_oracle_f32_to_f16_bits(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    uint16_t sign = (uint16_t)((bits >> 16) & 0x8000);
    int exp = (int)((bits >> 23) & 0xff) - 127 + 15;
    uint32_t mant = bits & 0x7fffff;
    if (exp <= 0) {
        if (exp < -10) return sign;
        mant |= 0x800000;
        uint32_t shift = (uint32_t)(14 - exp);
        uint16_t half = (uint16_t)(mant >> shift);
        if ((mant >> (shift - 1)) & 1) half++;
        return sign | half;
    }
    if (exp >= 0x1f) {
        if (mant == 0) return sign | 0x7c00;
        return sign | 0x7c00 | (uint16_t)(mant >> 13);
    }
    uint16_t half_exp = (uint16_t)(exp << 10);
    uint16_t half_mant = (uint16_t)(mant >> 13);
    if (mant & 0x00001000) {
        half_mant++;
        if (half_mant & 0x0400) {
            half_mant = 0;
            half_exp += 0x0400;
            if (half_exp >= 0x7c00) half_exp = 0x7c00;
        }
    }
    return sign | half_exp | half_mant;
}

EOS_ORACLE_API float eos_oracle_f16_bits_to_f32(uint16_t bits) {
    uint32_t sign = (uint32_t)(bits & 0x8000) << 16;
    uint32_t exp = (bits >> 10) & 0x1f;
    uint32_t mant = bits & 0x03ff;
    uint32_t out;
    if (exp == 0) {
        if (mant == 0) {
            out = sign;
        } else {
            uint32_t exp32 = 127 - 15 + 1;
            while ((mant & 0x0400) == 0) {
                mant <<= 1;
                exp32--;
            }
            mant &= 0x03ff;
            out = sign | (exp32 << 23) | (mant << 13);
        }
    } else if (exp == 0x1f) {
        out = sign | 0x7f800000u | (mant << 13);
    } else {
        out = sign | ((exp + (127 - 15)) << 23) | (mant << 13);
    }
    float f;
    memcpy(&f, &out, 4);
    return f;
}

/* ------------------------------------------------------------------------------------ */
/* q8 grid: runtime/embedding_trainer.go:11413-11446 (fakeQuantizeDataInPlace).          */
/* Symmetric abs-max, levels = 2^(bits-1)-1, scale = maxAbs/levels (float), q =           */
/* round-half-away(v/scale) clamped to +-levels.  `group` = number of consecutive         */
/* elements sharing one scale: the whole tensor for the reference's per-tensor rule, one  */
/* weight row ([out,in] layout) for per-output-channel scales.  A non-zero   */
/* `scale_round_f16` flag rounds each scale to f16 (mll_export.go rule) before use.       */
/* Writes int8 codes and one float scale per group; all-zero groups get scale 0, codes 0. */
/* ------------------------------------------------------------------------------------ */
EOS_ORACLE_API void eos_oracle_quantize_symmetric(const float *data, int64_t n, int64_t group, int bits,
                                                  int scale_round_f16, int8_t *codes, float *scales) {
    if (group <= 0) group = n;
    int levels_int = (1 << (bits - 1)) - 1;
    float levels = (float)levels_int;
    for (int64_t g0 = 0, gi = 0; g0 < n; g0 += group, gi++) {
        int64_t g1 = g0 + group;
        if (g1 > n) g1 = n;
        float max_abs = 0.0f;
        for (int64_t i = g0; i < g1; i++) {
            float a = (float)fabs((double)data[i]);
            if (a > max_abs) max_abs = a;
        }
        float scale = max_abs / levels;
        if (scale_round_f16 && scale != 0.0f) {
            scale = eos_oracle_f16_bits_to_f32(eos_oracle_f32_to_f16_bits(scale));
        }
        scales[gi] = scale;
        for (int64_t i = g0; i < g1; i++) {
            if (scale == 0.0f) {
                codes[i] = 0;
                continue;
            }
            float q = (float)round((double)(data[i] / scale));
            if (q > levels) q = levels;
            if (q < -levels) q = -levels;
            codes[i] = (int8_t)q;
        }
    }
}

/* dequant: float(int8) * scale, runtime/weight_file.go:305-356 */
EOS_ORACLE_API void eos_oracle_dequantize(const int8_t *codes, int64_t n, int64_t group, const float *scales,
                                          float *out) {
    if (group <= 0) group = n;
    for (int64_t i = 0; i < n; i++) out[i] = (float)codes[i] * scales[i / group];
}

/* ------------------------------------------------------------------------------------ */
/* Generic tensor ops of the compiled-pipeline path (config "masked mean-pooled embed").  */
/* ------------------------------------------------------------------------------------ */

/* gatherTensor, rank-2 table x rank-2 indices: runtime/backend/tensor_ops.go:1015-1064.
 * Returns 0, or 1 when an index is outside [0, rows). */
EOS_ORACLE_API int eos_oracle_gather(const float *table, int rows, int cols, const int32_t *indices, int64_t count,
                                     float *out) {
    for (int64_t i = 0; i < count; i++) {
        int32_t idx = indices[i];
        if (idx < 0 || idx >= rows) return 1;
        memcpy(out + i * cols, table + (int64_t)idx * cols, sizeof(float) * (size_t)cols);
    }
    return 0;
}

/* matmulTensor, [rows,k] x [k,n] with rhs in [in,out] layout, float accumulate in k order:
 * runtime/backend/tensor_ops.go:1168-1232; optional scale per ApplyMatMulAttributes :1256-1272. */
EOS_ORACLE_API void eos_oracle_matmul(const float *lhs, int64_t rows, int k, const float *rhs, int n, float scale,
                                      float *out) {
    for (int64_t i = 0; i < rows; i++) {
        for (int j = 0; j < n; j++) {
            float sum = 0.0f;
            for (int kk = 0; kk < k; kk++) sum += lhs[i * k + kk] * rhs[(int64_t)kk * n + j];
            out[i * n + j] = sum;
        }
    }
    if (scale != 1.0f) {
        for (int64_t i = 0; i < rows * n; i++) out[i] *= scale;
    }
}

/* normalizeRows: runtime/backend/tensor_ops.go:1367-1391 (double sum of squares, float
 * norm, zero row left untouched, float division). */
EOS_ORACLE_API void eos_oracle_normalize_rows(const float *in, int64_t rows, int cols, float *out) {
    for (int64_t r = 0; r < rows; r++) {
        double sum = 0.0;
        for (int c = 0; c < cols; c++) {
            double v = (double)in[r * cols + c];
            sum += v * v;
        }
        float norm = (float)sqrt(sum);
        for (int c = 0; c < cols; c++) out[r * cols + c] = (norm == 0.0f) ? in[r * cols + c] : in[r * cols + c] / norm;
    }
}

/* meanPoolMaskedTensor rank-3: runtime/backend/tensor_ops.go:1680-1705 (float sum in t
 * order, multiply by 1/float(count), count 0 -> zeros). */
EOS_ORACLE_API void eos_oracle_mean_pool_masked(const float *in, const int32_t *mask, int batches, int rows, int cols,
                                                float *out) {
    for (int b = 0; b < batches; b++) {
        float *o = out + (int64_t)b * cols;
        for (int c = 0; c < cols; c++) o[c] = 0.0f;
        int count = 0;
        for (int r = 0; r < rows; r++) {
            if (mask[(int64_t)b * rows + r] == 0) continue;
            count++;
            const float *src = in + ((int64_t)b * rows + r) * cols;
            for (int c = 0; c < cols; c++) o[c] += src[c];
        }
        if (count == 0) continue;
        float inv = 1.0f / (float)count;
        for (int c = 0; c < cols; c++) o[c] *= inv;
    }
}

/* clsPoolTensor: runtime/backend/bert_embedder_ops.go:199-218 */
EOS_ORACLE_API void eos_oracle_cls_pool(const float *in, int batches, int rows, int cols, float *out) {
    for (int b = 0; b < batches; b++)
        memcpy(out + (int64_t)b * cols, in + (int64_t)b * rows * cols, sizeof(float) * (size_t)cols);
}

/* The compiled pipeline examples/embed_masked_pooled.eos:11-16:
 * gather -> matmul -> normalize (per token) -> masked mean_pool.  `pool_then_l2` != 0 selects
 * the other order (mean-pool the projected rows, then normalize the pooled row).
 * Returns 1 on an out-of-range token id. */
EOS_ORACLE_API int eos_oracle_embed_pooled(const float *table, int vocab, int dim, const float *projection, int out_dim,
                                           const int32_t *tokens, const int32_t *mask, int batch, int tlen,
                                           int pool_then_l2, float matmul_scale, float *out) {
    int64_t rows = (int64_t)batch * tlen;
    float *hidden = (float *)malloc(sizeof(float) * (size_t)(rows * dim));
    float *proj = (float *)malloc(sizeof(float) * (size_t)(rows * out_dim));
    int rc = eos_oracle_gather(table, vocab, dim, tokens, rows, hidden);
    if (rc == 0) {
        eos_oracle_matmul(hidden, rows, dim, projection, out_dim, matmul_scale, proj);
        if (!pool_then_l2) {
            float *norm = (float *)malloc(sizeof(float) * (size_t)(rows * out_dim));
            eos_oracle_normalize_rows(proj, rows, out_dim, norm);
            eos_oracle_mean_pool_masked(norm, mask, batch, tlen, out_dim, out);
            free(norm);
        } else {
            float *pooled = (float *)malloc(sizeof(float) * (size_t)batch * out_dim);
            eos_oracle_mean_pool_masked(proj, mask, batch, tlen, out_dim, pooled);
            eos_oracle_normalize_rows(pooled, batch, out_dim, out);
            free(pooled);
        }
    }
    free(hidden);
    free(proj);
    return rc;
}

/* ------------------------------------------------------------------------------------ */
/* BERT-family encoder                                                                   */
/* ------------------------------------------------------------------------------------ */

/* BERTEmbeddingsReference: runtime/backend/tensor_ops.go:1451-1512.  float add of the
 * three rows, double mean/variance, out = float(normalized*gamma + beta).
 * Returns 0 ok; 1 token id, 2 position id, 3 type id out of range. */
EOS_ORACLE_API int eos_oracle_bert_embeddings(const float *tok, int vocab, const float *pos, int max_pos,
                                              const float *typ, int type_vocab, const float *gamma, const float *beta,
                                              const int32_t *input_ids, const int32_t *position_ids,
                                              const int32_t *type_ids, int64_t rows, int dim, double eps, float *out) {
    for (int64_t row = 0; row < rows; row++) {
        int t = input_ids[row], p = position_ids[row], tt = type_ids[row];
        if (t < 0 || t >= vocab) return 1;
        if (p < 0 || p >= max_pos) return 2;
        if (tt < 0 || tt >= type_vocab) return 3;
        float *o = out + row * dim;
        double mean = 0.0;
        for (int d = 0; d < dim; d++) {
            float sum = tok[(int64_t)t * dim + d] + pos[(int64_t)p * dim + d] + typ[(int64_t)tt * dim + d];
            o[d] = sum;
            mean += (double)sum;
        }
        mean /= (double)dim;
        double var = 0.0;
        for (int d = 0; d < dim; d++) {
            double c = (double)o[d] - mean;
            var += c * c;
        }
        var /= (double)dim;
        double inv = 1.0 / sqrt(var + eps);
        for (int d = 0; d < dim; d++) {
            double nrm = ((double)o[d] - mean) * inv;
            o[d] = (float)(nrm * (double)gamma[d] + (double)beta[d]);
        }
    }
    return 0;
}

/* denseHFRange: runtime/backend/bert_encoder_layer_ops.go:452-462.  y = x W^T + b with W in
 * HF [out,in] layout and a double accumulator seeded with the bias. */
typedef struct {
    const float *input, *weight, *bias;
    float *result;
    int in, out;
} dense_ctx;

static void dense_range(void *p, int64_t r0, int64_t r1) {
    dense_ctx *c = (dense_ctx *)p;
    for (int64_t r = r0; r < r1; r++) {
        for (int o = 0; o < c->out; o++) {
            double sum = (double)c->bias[o];
            const float *x = c->input + r * c->in;
            const float *w = c->weight + (int64_t)o * c->in;
            for (int k = 0; k < c->in; k++) sum += (double)x[k] * (double)w[k];
            c->result[r * c->out + o] = (float)sum;
        }
    }
}

EOS_ORACLE_API void eos_oracle_dense_hf(const float *input, int64_t rows, int in, const float *weight,
                                        const float *bias, int out, float *result, int workers) {
    dense_ctx c = {input, weight, bias, result, in, out};
    parallel_ranges(dense_range, &c, rows, workers);
}

/* bertSelfAttentionContextRange: runtime/backend/bert_encoder_layer_ops.go:326-379.
 * One job per (batch, query token, head); double logits over unmasked keys only,
 * max-subtracted softmax, context += float(prob * v); no active key -> zeros.
 * Padded query rows are computed like any other.
 * Extension (NOT in the reference, which has no local attention): with window > 0 key j is
 * visible to query i only if 2*|i - j| < window; everything else is unchanged. */
typedef struct {
    const float *q, *k, *v;
    const int32_t *mask;
    float *context;
    int tokens, hidden, heads, head_dim;
    int window; /* 0 = the reference (full attention); > 0 = local-window extension, see below */
} attn_ctx;

static void attn_range(void *p, int64_t j0, int64_t j1) {
    attn_ctx *c = (attn_ctx *)p;
    double scale = 1.0 / sqrt((double)c->head_dim);
    double *logits = (double *)malloc(sizeof(double) * (size_t)c->tokens);
    for (int64_t job = j0; job < j1; job++) {
        int head = (int)(job % c->heads);
        int64_t qi = job / c->heads;
        int64_t batch = qi / c->tokens;
        int64_t qrow = qi;
        int qt = (int)(qi % c->tokens);
        int active = 0;
        double max_logit = -INFINITY;
        for (int kt = 0; kt < c->tokens; kt++) {
            if (c->mask[batch * c->tokens + kt] == 0 || (c->window > 0 && 2 * abs(qt - kt) >= c->window)) continue;
            active++;
            int64_t krow = batch * c->tokens + kt;
            double dot = 0.0;
            for (int d = 0; d < c->head_dim; d++) {
                int idx = head * c->head_dim + d;
                dot += (double)c->q[qrow * c->hidden + idx] * (double)c->k[krow * c->hidden + idx];
            }
            double logit = dot * scale;
            logits[kt] = logit;
            if (logit > max_logit) max_logit = logit;
        }
        if (active == 0) continue;
        double sum_exp = 0.0;
        for (int kt = 0; kt < c->tokens; kt++) {
            if (c->mask[batch * c->tokens + kt] == 0 || (c->window > 0 && 2 * abs(qt - kt) >= c->window)) continue;
            double ev = exp(logits[kt] - max_logit);
            logits[kt] = ev;
            sum_exp += ev;
        }
        for (int kt = 0; kt < c->tokens; kt++) {
            if (c->mask[batch * c->tokens + kt] == 0 || (c->window > 0 && 2 * abs(qt - kt) >= c->window)) continue;
            double prob = logits[kt] / sum_exp;
            int64_t vrow = batch * c->tokens + kt;
            for (int d = 0; d < c->head_dim; d++) {
                int idx = head * c->head_dim + d;
                c->context[qrow * c->hidden + idx] += (float)(prob * (double)c->v[vrow * c->hidden + idx]);
            }
        }
    }
    free(logits);
}

EOS_ORACLE_API void eos_oracle_bert_attention_window(const float *q, const float *k, const float *v,
                                                     const int32_t *mask, int batch, int tokens, int hidden,
                                                     int heads, int window, float *context, int workers) {
    memset(context, 0, sizeof(float) * (size_t)batch * tokens * hidden);
    attn_ctx c = {q, k, v, mask, context, tokens, hidden, heads, hidden / heads, window};
    parallel_ranges(attn_range, &c, (int64_t)batch * tokens * heads, workers);
}

EOS_ORACLE_API void eos_oracle_bert_attention(const float *q, const float *k, const float *v, const int32_t *mask,
                                              int batch, int tokens, int hidden, int heads, float *context,
                                              int workers) {
    memset(context, 0, sizeof(float) * (size_t)batch * tokens * hidden);
    attn_ctx c = {q, k, v, mask, context, tokens, hidden, heads, hidden / heads, 0};
    parallel_ranges(attn_range, &c, (int64_t)batch * tokens * heads, workers);
}

/* layerNormAffine: runtime/backend/bert_encoder_layer_ops.go:718-740 */
EOS_ORACLE_API void eos_oracle_layernorm_affine(const float *in, int64_t rows, int dim, const float *gamma,
                                                const float *beta, double eps, float *out) {
    for (int64_t r = 0; r < rows; r++) {
        const float *x = in + r * dim;
        double mean = 0.0;
        for (int d = 0; d < dim; d++) mean += (double)x[d];
        mean /= (double)dim;
        double var = 0.0;
        for (int d = 0; d < dim; d++) {
            double c = (double)x[d] - mean;
            var += c * c;
        }
        var /= (double)dim;
        double inv = 1.0 / sqrt(var + eps);
        for (int d = 0; d < dim; d++) {
            double nrm = ((double)x[d] - mean) * inv;
            out[r * dim + d] = (float)(nrm * (double)gamma[d] + (double)beta[d]);
        }
    }
}

/* exactGELU: runtime/backend/bert_encoder_layer_ops.go:742-744 */
EOS_ORACLE_API float eos_oracle_exact_gelu(float x) { return 0.5f * x * (1.0f + (float)erf((double)x / M_SQRT2)); }

/* geluTensor (tanh form of the compact path): runtime/backend/tensor_ops.go:1926-1934 */
EOS_ORACLE_API float eos_oracle_tanh_gelu(float x) {
    double v = (double)x;
    return (float)(0.5 * v * (1.0 + tanh(0.7978845608028654 * (v + 0.044715 * v * v * v))));
}

/* One encoder layer, bertEncoderLayerReferenceWithProjector:
 * runtime/backend/bert_encoder_layer_ops.go:186-224.  `w` holds the 16 tensors in the fixed
 * order of runtime/pretrained_bert_importer.go:936-951:
 * qW qB kW kB vW vB aoW aoB aLNg aLNb iW iB oW oB oLNg oLNb. `hidden` is updated in place. */
static void bert_layer_impl(float *hidden_states, const int32_t *mask, int batch, int tokens, int hidden, int inter,
                            int heads, const float *const *w, double eps, int window, int workers) {
    int64_t rows = (int64_t)batch * tokens;
    size_t hsz = sizeof(float) * (size_t)(rows * hidden);
    float *q = (float *)malloc(hsz), *k = (float *)malloc(hsz), *v = (float *)malloc(hsz);
    float *ctx = (float *)malloc(hsz), *tmp = (float *)malloc(hsz), *attn_layer = (float *)malloc(hsz);
    float *mid = (float *)malloc(sizeof(float) * (size_t)(rows * inter));
    eos_oracle_dense_hf(hidden_states, rows, hidden, w[0], w[1], hidden, q, workers);
    eos_oracle_dense_hf(hidden_states, rows, hidden, w[2], w[3], hidden, k, workers);
    eos_oracle_dense_hf(hidden_states, rows, hidden, w[4], w[5], hidden, v, workers);
    eos_oracle_bert_attention_window(q, k, v, mask, batch, tokens, hidden, heads, window, ctx, workers);
    eos_oracle_dense_hf(ctx, rows, hidden, w[6], w[7], hidden, tmp, workers);
    for (int64_t i = 0; i < rows * hidden; i++) tmp[i] = tmp[i] + hidden_states[i];
    eos_oracle_layernorm_affine(tmp, rows, hidden, w[8], w[9], eps, attn_layer);
    eos_oracle_dense_hf(attn_layer, rows, hidden, w[10], w[11], inter, mid, workers);
    for (int64_t i = 0; i < rows * inter; i++) mid[i] = eos_oracle_exact_gelu(mid[i]);
    eos_oracle_dense_hf(mid, rows, inter, w[12], w[13], hidden, tmp, workers);
    for (int64_t i = 0; i < rows * hidden; i++) tmp[i] = tmp[i] + attn_layer[i];
    eos_oracle_layernorm_affine(tmp, rows, hidden, w[14], w[15], eps, hidden_states);
    free(q);
    free(k);
    free(v);
    free(ctx);
    free(tmp);
    free(attn_layer);
    free(mid);
}

EOS_ORACLE_API void eos_oracle_bert_layer(float *hidden_states, const int32_t *mask, int batch, int tokens, int hidden,
                                          int inter, int heads, const float *const *w, double eps, int workers) {
    bert_layer_impl(hidden_states, mask, batch, tokens, hidden, inter, heads, w, eps, 0, workers);
}

/* Whole embedder, BERTEmbedderReferenceWithPooling: runtime/backend/bert_embedder_ops.go:101-197
 * (position ids 0..T-1 per :220-228; pooling 0 = masked_mean, 1 = cls; then normalizeRows),
 * optionally followed by PretrainedBERTProjectionHead.Apply
 * (runtime/pretrained_bert_projection_head.go:84-100: [in,out] weights, no bias, double
 * accumulate) and normalizeRetrievalVector (runtime/retrieval_eval.go:1040-1054).
 * out is [batch, head ? head_out : hidden].  Returns the bert_embeddings error code.
 * window = 0 is the reference; window > 0 selects the local-window extension of the attention. */
EOS_ORACLE_API int eos_oracle_bert_embedder(const int32_t *input_ids, const int32_t *mask, const int32_t *type_ids,
                                            int batch, int tokens, const float *tok, int vocab, const float *pos,
                                            int max_pos, const float *typ, int type_vocab, const float *emb_gamma,
                                            const float *emb_beta, const float *const *layer_weights, int layers,
                                            int hidden, int inter, int heads, double eps, int pooling,
                                            const float *head_w, int head_out, int window, float *out, int workers) {
    int64_t rows = (int64_t)batch * tokens;
    int32_t *pos_ids = (int32_t *)malloc(sizeof(int32_t) * (size_t)rows);
    for (int b = 0; b < batch; b++)
        for (int t = 0; t < tokens; t++) pos_ids[(int64_t)b * tokens + t] = t;
    float *hs = (float *)malloc(sizeof(float) * (size_t)(rows * hidden));
    int rc = eos_oracle_bert_embeddings(tok, vocab, pos, max_pos, typ, type_vocab, emb_gamma, emb_beta, input_ids,
                                        pos_ids, type_ids, rows, hidden, eps, hs);
    free(pos_ids);
    if (rc != 0) {
        free(hs);
        return rc;
    }
    for (int l = 0; l < layers; l++)
        bert_layer_impl(hs, mask, batch, tokens, hidden, inter, heads, layer_weights + (size_t)l * 16, eps, window,
                        workers);
    float *pooled = (float *)malloc(sizeof(float) * (size_t)batch * hidden);
    float *normed = (float *)malloc(sizeof(float) * (size_t)batch * hidden);
    if (pooling == 1)
        eos_oracle_cls_pool(hs, batch, tokens, hidden, pooled);
    else
        eos_oracle_mean_pool_masked(hs, mask, batch, tokens, hidden, pooled);
    eos_oracle_normalize_rows(pooled, batch, hidden, normed);
    if (head_w == NULL) {
        memcpy(out, normed, sizeof(float) * (size_t)batch * hidden);
    } else {
        for (int b = 0; b < batch; b++) {
            const float *vec = normed + (int64_t)b * hidden;
            float *o = out + (int64_t)b * head_out;
            double sq = 0.0;
            for (int j = 0; j < head_out; j++) {
                double sum = 0.0;
                for (int i = 0; i < hidden; i++) sum += (double)vec[i] * (double)head_w[(int64_t)i * head_out + j];
                o[j] = (float)sum;
            }
            for (int j = 0; j < head_out; j++) sq += (double)o[j] * (double)o[j];
            if (sq != 0.0) {
                float sc = (float)(1.0 / sqrt(sq));
                for (int j = 0; j < head_out; j++) o[j] *= sc;
            }
        }
    }
    free(hs);
    free(pooled);
    free(normed);
    return 0;
}

/* Per-token output vectors (long-context multi-vector documents): the same embeddings and layers, then for every
 * token with mask != 0 the final hidden row times token_w [hidden, token_dim] (in-major, no bias, double accumulate
 * like the projection head of runtime/pretrained_bert_projection_head.go:84-100) and normalizeRetrievalVector
 * (runtime/retrieval_eval.go:1040-1054).  out is [batch, tokens, token_dim]; rows of masked tokens are zero. */
EOS_ORACLE_API int eos_oracle_bert_token_vectors(const int32_t *input_ids, const int32_t *mask, const int32_t *type_ids,
                                                 int batch, int tokens, const float *tok, int vocab, const float *pos,
                                                 int max_pos, const float *typ, int type_vocab, const float *emb_gamma,
                                                 const float *emb_beta, const float *const *layer_weights, int layers,
                                                 int hidden, int inter, int heads, double eps, const float *token_w,
                                                 int token_dim, int window, float *out, int workers) {
    int64_t rows = (int64_t)batch * tokens;
    int32_t *pos_ids = (int32_t *)malloc(sizeof(int32_t) * (size_t)rows);
    for (int b = 0; b < batch; b++)
        for (int t = 0; t < tokens; t++) pos_ids[(int64_t)b * tokens + t] = t;
    float *hs = (float *)malloc(sizeof(float) * (size_t)(rows * hidden));
    int rc = eos_oracle_bert_embeddings(tok, vocab, pos, max_pos, typ, type_vocab, emb_gamma, emb_beta, input_ids,
                                        pos_ids, type_ids, rows, hidden, eps, hs);
    free(pos_ids);
    if (rc != 0) {
        free(hs);
        return rc;
    }
    for (int l = 0; l < layers; l++)
        bert_layer_impl(hs, mask, batch, tokens, hidden, inter, heads, layer_weights + (size_t)l * 16, eps, window,
                        workers);
    for (int64_t r = 0; r < rows; r++) {
        float *o = out + r * token_dim;
        if (mask[r] == 0) {
            memset(o, 0, sizeof(float) * (size_t)token_dim);
            continue;
        }
        const float *vec = hs + r * hidden;
        double sq = 0.0;
        for (int j = 0; j < token_dim; j++) {
            double sum = 0.0;
            for (int i = 0; i < hidden; i++) sum += (double)vec[i] * (double)token_w[(int64_t)i * token_dim + j];
            o[j] = (float)sum;
        }
        for (int j = 0; j < token_dim; j++) sq += (double)o[j] * (double)o[j];
        if (sq != 0.0) {
            float sc = (float)(1.0 / sqrt(sq));
            for (int j = 0; j < token_dim; j++) o[j] *= sc;
        }
    }
    free(hs);
    return 0;
}

/* ------------------------------------------------------------------------------------ */
/* Sparse attention: sparseAttentionTensor, runtime/backend/attention_ops.go:218-276        */
/* (device twin: sparseAttentionKernelSource, runtime/backends/cuda/native_linux.go:2044).  */
/* Per query row: scores q.k (float accumulate in d order, no 1/sqrt(d)), top-`budget` keys */
/* by score descending then index ascending (:518-531), optionally routed through the        */
/* `route_top_blocks` blocks whose anchor key (the block's middle) scores best (:462-497);   */
/* softmax over the selected scores with exp in double (:533-560); out += float(w/denom) * v */
/* accumulated in float in selection order.                                                  */
/* ------------------------------------------------------------------------------------ */
typedef struct {
    int index;
    float score;
} sparse_cand;

static int sparse_cand_cmp(const void *a, const void *b) {
    const sparse_cand *x = (const sparse_cand *)a, *y = (const sparse_cand *)b;
    if (x->score == y->score) return (x->index > y->index) - (x->index < y->index);
    return x->score > y->score ? -1 : 1;
}

/* budget: top_k attribute, else ceil(sqrt(key_len)), clamped to [1, key_len] (:445-460) */
EOS_ORACLE_API int eos_oracle_sparse_attention_budget(int top_k, int key_len) {
    if (key_len <= 0) return 0;
    int budget = top_k;
    if (budget <= 0) budget = (int)ceil(sqrt((double)key_len));
    if (budget < 1) budget = 1;
    if (budget > key_len) budget = key_len;
    return budget;
}

/* (block size, top blocks) after normalizeSparseAttentionRoute (:503-516); 0, 0 = no routing */
EOS_ORACLE_API void eos_oracle_sparse_attention_route(int key_len, int block_size, int top_blocks, int *out_block,
                                                      int *out_top) {
    *out_block = 0;
    *out_top = 0;
    if (key_len <= 0 || block_size <= 0 || top_blocks <= 0) return;
    if (block_size > key_len) block_size = key_len;
    int block_count = (key_len + block_size - 1) / block_size;
    if (top_blocks > block_count) top_blocks = block_count;
    *out_block = block_size;
    *out_top = top_blocks;
}

static float sparse_score(const float *q, const float *k, int dim) {
    float sum = 0.0f;
    for (int d = 0; d < dim; d++) sum += q[d] * k[d];
    return sum;
}

/* query [batches, q_len, dim], key [batches, k_len, dim], value [batches, k_len, vdim] -> out [batches, q_len, vdim] */
EOS_ORACLE_API void eos_oracle_sparse_attention(const float *query, const float *key, const float *value, int batches,
                                                int q_len, int k_len, int dim, int vdim, int top_k, int route_block_size,
                                                int route_top_blocks, float *out) {
    memset(out, 0, sizeof(float) * (size_t)batches * q_len * vdim);
    if (k_len <= 0) return;
    int budget = eos_oracle_sparse_attention_budget(top_k, k_len);
    int bs, tb;
    eos_oracle_sparse_attention_route(k_len, route_block_size, route_top_blocks, &bs, &tb);
    sparse_cand *cand = (sparse_cand *)malloc(sizeof(sparse_cand) * (size_t)k_len);
    sparse_cand *blocks = (sparse_cand *)malloc(sizeof(sparse_cand) * (size_t)k_len);
    double *weights = (double *)malloc(sizeof(double) * (size_t)k_len);
    for (int b = 0; b < batches; b++) {
        const float *kb = key + (int64_t)b * k_len * dim;
        const float *vb = value + (int64_t)b * k_len * vdim;
        for (int q = 0; q < q_len; q++) {
            const float *qv = query + ((int64_t)b * q_len + q) * dim;
            int n = 0;
            if (bs <= 0 || tb <= 0) {
                for (int k = 0; k < k_len; k++) {
                    cand[n].index = k;
                    cand[n].score = sparse_score(qv, kb + (int64_t)k * dim, dim);
                    n++;
                }
            } else {
                int block_count = (k_len + bs - 1) / bs;
                for (int blk = 0; blk < block_count; blk++) {
                    int start = blk * bs, end = start + bs;
                    if (end > k_len) end = k_len;
                    int anchor = start + (end - start) / 2;
                    blocks[blk].index = blk;
                    blocks[blk].score = sparse_score(qv, kb + (int64_t)anchor * dim, dim);
                }
                qsort(blocks, (size_t)block_count, sizeof(sparse_cand), sparse_cand_cmp);
                int nb = tb < block_count ? tb : block_count;
                for (int i = 0; i < nb; i++) {
                    int start = blocks[i].index * bs, end = start + bs;
                    if (end > k_len) end = k_len;
                    for (int k = start; k < end; k++) {
                        cand[n].index = k;
                        cand[n].score = sparse_score(qv, kb + (int64_t)k * dim, dim);
                        n++;
                    }
                }
            }
            /* (score desc, index asc) is a total order, so qsort gives the stable sort's result */
            qsort(cand, (size_t)n, sizeof(sparse_cand), sparse_cand_cmp);
            if (budget < n) n = budget;
            if (n == 0) continue;
            float max_score = cand[0].score;
            for (int i = 1; i < n; i++)
                if (cand[i].score > max_score) max_score = cand[i].score;
            double denom = 0.0;
            for (int i = 0; i < n; i++) {
                weights[i] = exp((double)(cand[i].score - max_score));
                denom += weights[i];
            }
            if (denom == 0.0 || isnan(denom)) continue;
            float *row = out + ((int64_t)b * q_len + q) * vdim;
            for (int i = 0; i < n; i++) {
                float scale = (float)(weights[i] / denom);
                const float *vv = vb + (int64_t)cand[i].index * vdim;
                for (int d = 0; d < vdim; d++) row[d] += scale * vv[d];
            }
        }
    }
    free(cand);
    free(blocks);
    free(weights);
}

/* ------------------------------------------------------------------------------------ */
/* TurboQuant, Hadamard/MSE variant (encode / decode pinned to the reference's device     */
/* source compiled for the host, see header).                                             */
/* Structure follows Eos's device restatement runtime/backends/cuda/native_linux.go:      */
/*   blocked normalised FWHT over greedy power-of-two blocks  :1822-1851                  */
/*   nearest centroid = first boundary greater than the value :1865-1877                  */
/*   encode: unit-normalise, permute*signs1, FWHT, signs2*inverse-permute :1906-1957      */
/* Deviations, stated: the norm side-car is the float L2 norm (not the 8-bit log code of  */
/* :1879-1904) because the retrieval configuration stores an f32 norm per vector; the     */
/* block scale is 1.0f/sqrtf(size) (correctly rounded) where the device string uses       */
/* rsqrtf (approximate on a GPU).                                                         */
/* ------------------------------------------------------------------------------------ */
static int highest_pow2_le(int value) {
    int p = 1;
    while ((p << 1) <= value) p <<= 1;
    return p;
}

static void fwht_normalized(float *values, int size) {
    if (size <= 1) return;
    for (int step = 1; step < size; step <<= 1) {
        int jump = step << 1;
        for (int i = 0; i < size; i += jump) {
            for (int j = i; j < i + step; j++) {
                float a = values[j], b = values[j + step];
                values[j] = a + b;
                values[j + step] = a - b;
            }
        }
    }
    float scale = 1.0f / sqrtf((float)size);
    for (int i = 0; i < size; i++) values[i] *= scale;
}

static void apply_blocks(float *values, int channels) {
    int offset = 0, remaining = channels;
    while (remaining > 0) {
        int size = highest_pow2_le(remaining);
        fwht_normalized(values + offset, size);
        offset += size;
        remaining -= size;
    }
}

/* rotated = R(x * prescale): work[i] = x[perm[i]]*prescale*signs1[i]; FWHT blocks;
 * rotated[perm[i]] = work[i]*signs2[i].  native_linux.go:1940-1950 */
EOS_ORACLE_API void eos_oracle_tq_rotate(const float *x, int dim, const int32_t *perm, const float *signs1,
                                         const float *signs2, float prescale, float *rotated) {
    float *work = (float *)malloc(sizeof(float) * (size_t)dim);
    for (int i = 0; i < dim; i++) work[i] = x[perm[i]] * prescale * signs1[i];
    apply_blocks(work, dim);
    for (int i = 0; i < dim; i++) rotated[perm[i]] = work[i] * signs2[i];
    free(work);
}

static int nearest_centroid(float value, const float *boundaries, int levels) {
    int lo = 0, hi = levels - 1;
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (boundaries[mid] > value)
            hi = mid;
        else
            lo = mid + 1;
    }
    return lo;
}

/* Packed code bytes per vector: codes are `bits` wide, little-end first inside each byte
 * (the nibble order of runtime/mll_export.go:950-960); bits in {2,4,8}. */
EOS_ORACLE_API int64_t eos_oracle_tq_code_bytes(int dim, int bits) { return ((int64_t)dim * bits + 7) / 8; }

/* Encode n vectors [n,dim] -> packed codes [n, code_bytes] + float norms [n].
 * Sequential float sum of squares, norm = sqrtf, scale = 1/norm if norm > 1e-12 else 1
 * (native_linux.go:1930-1939). */
EOS_ORACLE_API void eos_oracle_tq_encode(const float *x, int64_t n, int dim, int bits, const int32_t *perm,
                                         const float *signs1, const float *signs2, const float *boundaries,
                                         uint8_t *codes, float *norms) {
    int levels = 1 << bits;
    int64_t cb = eos_oracle_tq_code_bytes(dim, bits);
    int per_byte = 8 / bits;
    float *rot = (float *)malloc(sizeof(float) * (size_t)dim);
    for (int64_t v = 0; v < n; v++) {
        const float *xv = x + v * dim;
        float norm_sq = 0.0f;
        for (int c = 0; c < dim; c++) norm_sq += xv[c] * xv[c];
        float norm = sqrtf(norm_sq);
        float scale = 1.0f;
        if (norm > 1.0e-12f) scale = 1.0f / norm;
        eos_oracle_tq_rotate(xv, dim, perm, signs1, signs2, scale, rot);
        uint8_t *cv = codes + v * cb;
        memset(cv, 0, (size_t)cb);
        for (int c = 0; c < dim; c++) {
            int idx = nearest_centroid(rot[c], boundaries, levels);
            cv[c / per_byte] |= (uint8_t)(idx << ((c % per_byte) * bits));
        }
        norms[v] = norm;
    }
    free(rot);
}

/* The reference's encode stores the norm as an 8-bit code on a log scale:
 * code = round(255 * (ln(norm) + 16) / 32) clamped to [0, 255]; 0 for norm <= 0 or NaN, 255 for +inf;
 * value = exp(-16 + 32 * code / 255).  native_linux.go:1879-1904. */
EOS_ORACLE_API void eos_oracle_tq_norm_code(const float *norms, int64_t n, uint8_t *codes) {
    for (int64_t i = 0; i < n; i++) {
        float norm = norms[i];
        int code;
        if (norm <= 0.0f || isnan(norm)) {
            code = 0;
        } else if (isinf(norm)) {
            code = 255;
        } else {
            float t = (logf(norm) + 16.0f) / 32.0f;
            if (t <= 0.0f) code = 0;
            else if (t >= 1.0f) code = 255;
            else code = (int)roundf(t * 255.0f);
        }
        codes[i] = (uint8_t)code;
    }
}
EOS_ORACLE_API void eos_oracle_tq_norm_value(const uint8_t *codes, int64_t n, float *norms) {
    for (int64_t i = 0; i < n; i++) norms[i] = expf(-16.0f + ((float)codes[i] / 255.0f) * 32.0f);
}

EOS_ORACLE_API void eos_oracle_tq_unpack(const uint8_t *codes, int dim, int bits, int32_t *idx) {
    int per_byte = 8 / bits;
    int maskv = (1 << bits) - 1;
    for (int c = 0; c < dim; c++) idx[c] = (codes[c / per_byte] >> ((c % per_byte) * bits)) & maskv;
}

/* Decode (the exact inverse: centroids -> signs2 -> FWHT -> signs1 * norm),
 * native_linux.go:1959-2003 with the float norm. */
EOS_ORACLE_API void eos_oracle_tq_decode(const uint8_t *codes, const float *norms, int64_t n, int dim, int bits,
                                         const int32_t *perm, const float *signs1, const float *signs2,
                                         const float *centroids, float *out) {
    int64_t cb = eos_oracle_tq_code_bytes(dim, bits);
    float *rot = (float *)malloc(sizeof(float) * (size_t)dim);
    float *work = (float *)malloc(sizeof(float) * (size_t)dim);
    int32_t *idx = (int32_t *)malloc(sizeof(int32_t) * (size_t)dim);
    for (int64_t v = 0; v < n; v++) {
        eos_oracle_tq_unpack(codes + v * cb, dim, bits, idx);
        for (int c = 0; c < dim; c++) rot[c] = centroids[idx[c]];
        for (int i = 0; i < dim; i++) work[i] = rot[perm[i]] * signs2[i];
        apply_blocks(work, dim);
        for (int i = 0; i < dim; i++) out[v * dim + perm[i]] = work[i] * signs1[i] * norms[v];
    }
    free(rot);
    free(work);
    free(idx);
}

/* Prepared query = the same rotation applied to the raw query (no normalisation): the
 * rotation is orthogonal, so <q, doc> ~= norm * <R q, centroids[codes]>.  Call sites of the
 * prepared-query scoring: runtime/retrieval_turboquant.go:1324-1325, 1861-1874; the norm
 * multiplies the whole estimate (runtime/turboquant_quantized_vector.go:9-13). */
EOS_ORACLE_API void eos_oracle_tq_prepare_query(const float *q, int dim, const int32_t *perm, const float *signs1,
                                                const float *signs2, float *prepared) {
    eos_oracle_tq_rotate(q, dim, perm, signs1, signs2, 1.0f, prepared);
}

/* Score of rows quantised by the inner-product quantiser, turboquant.IPQuantized{MSE, Signs, ResNorm, Norm}
 * (runtime/turboquant_quantized_vector.go:43-49; call site of IPQuantizer.InnerProductPrepared:
 * runtime/retrieval_turboquant.go:1874).  The module (m31labs.dev/turboquant v0.2.0, go.mod:9) is not in the
 * reference tree, so this restates the published two-stage estimator -- MSE stage plus the QJL sign stage on the
 * residual, the whole estimate multiplied by Norm (turboquant_quantized_vector.go:9-13) -- with the sign projection
 * of the query (sketch) and its scale supplied by the caller.  PARITY UNPINNED for this function.
 * mse_idx [n, dim] one level index per byte; signs [n, ceil(dim/8)], bit i at byte i/8, bit i%8. */
EOS_ORACLE_API void eos_oracle_tq_ip_score(const uint8_t *mse_idx, const uint8_t *signs, const float *resnorms,
                                           const float *norms, int64_t n, int dim, const float *centroids,
                                           const float *prepared, const float *sketch, float qjl_scale, float *scores) {
    int sb = (dim + 7) / 8;
    for (int64_t v = 0; v < n; v++) {
        float a = 0.0f, b = 0.0f;
        for (int c = 0; c < dim; c++) a += prepared[c] * centroids[mse_idx[v * dim + c]];
        for (int i = 0; i < dim; i++) {
            int on = (signs[v * sb + i / 8] >> (i % 8)) & 1;
            b += on ? sketch[i] : -sketch[i];
        }
        scores[v] = norms[v] * (a + resnorms[v] * qjl_scale * b);
    }
}

/* scores[v] = norm[v] * sum_c prepared[c]*centroids[code[v,c]], float accumulate in
 * coordinate order. */
EOS_ORACLE_API void eos_oracle_tq_score(const uint8_t *codes, const float *norms, int64_t n, int dim, int bits,
                                        const float *centroids, const float *prepared, float *scores) {
    int64_t cb = eos_oracle_tq_code_bytes(dim, bits);
    int per_byte = 8 / bits;
    int maskv = (1 << bits) - 1;
    for (int64_t v = 0; v < n; v++) {
        const uint8_t *cv = codes + v * cb;
        float sum = 0.0f;
        for (int c = 0; c < dim; c++) {
            int idx = (cv[c / per_byte] >> ((c % per_byte) * bits)) & maskv;
            sum += prepared[c] * centroids[idx];
        }
        scores[v] = sum * norms[v];
    }
}

/* ------------------------------------------------------------------------------------ */
/* Exact top-k with the reference's order: score descending, then id ascending            */
/* (retrievalScoreBetter runtime/retrieval_eval.go:1153-1161; heap + insertion sort        */
/* runtime/retrieval_turboquant.go:1853-1916).  ids are row indices offset by id_base.     */
/* ------------------------------------------------------------------------------------ */
typedef struct {
    float score;
    int64_t id;
} scored;

static int better(scored a, scored b) {
    if (a.score > b.score) return 1;
    if (a.score < b.score) return 0;
    return a.id < b.id;
}

static int cmp_better(const void *pa, const void *pb) {
    scored a = *(const scored *)pa, b = *(const scored *)pb;
    if (better(a, b)) return -1;
    if (better(b, a)) return 1;
    return 0;
}

/* min-heap on "better": root is the worst kept element */
static void heap_sift_down(scored *h, int n, int i) {
    for (;;) {
        int l = 2 * i + 1, r = l + 1, m = i;
        if (l < n && better(h[m], h[l])) m = l;
        if (r < n && better(h[m], h[r])) m = r;
        if (m == i) return;
        scored t = h[i];
        h[i] = h[m];
        h[m] = t;
        i = m;
    }
}

static void heap_sift_up(scored *h, int i) {
    while (i > 0) {
        int p = (i - 1) / 2;
        if (!better(h[p], h[i])) return;
        scored t = h[i];
        h[i] = h[p];
        h[p] = t;
        i = p;
    }
}

/* Returns the number of results written (min(k, n)). */
EOS_ORACLE_API int eos_oracle_topk(const float *scores, int64_t n, int64_t id_base, int k, int64_t *out_ids,
                                   float *out_scores) {
    if (k <= 0 || k > n) k = (int)n;
    if (k == 0) return 0;
    scored *h = (scored *)malloc(sizeof(scored) * (size_t)k);
    int len = 0;
    for (int64_t i = 0; i < n; i++) {
        scored s = {scores[i], id_base + i};
        if (len < k) {
            h[len] = s;
            heap_sift_up(h, len);
            len++;
            continue;
        }
        if (better(s, h[0])) {
            h[0] = s;
            heap_sift_down(h, len, 0);
        }
    }
    for (int i = 1; i < len; i++)
        for (int j = i; j > 0 && better(h[j], h[j - 1]); j--) {
            scored t = h[j];
            h[j] = h[j - 1];
            h[j - 1] = t;
        }
    for (int i = 0; i < len; i++) {
        out_ids[i] = h[i].id;
        out_scores[i] = h[i].score;
    }
    free(h);
    return len;
}

/* Score one prepared query against a packed corpus and keep the top-k: the per-query body
 * of topTurboQuantRetrievalScoresWithStats (runtime/retrieval_turboquant.go:1853-1887)
 * without pruning (4-bit has no pruning bound, turboquant_retrieval_pruning_test.go:38-54). */
EOS_ORACLE_API int eos_oracle_tq_score_topk(const uint8_t *codes, const float *norms, int64_t n, int dim, int bits,
                                            const float *centroids, const float *prepared, int64_t id_base, int k,
                                            int64_t *out_ids, float *out_scores) {
    float *scores = (float *)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1));
    eos_oracle_tq_score(codes, norms, n, dim, bits, centroids, prepared, scores);
    int r = eos_oracle_topk(scores, n, id_base, k, out_ids, out_scores);
    free(scores);
    return r;
}

/* Merge several per-shard top-k lists into the global top-k with the same order. */
EOS_ORACLE_API int eos_oracle_topk_merge(const int64_t *ids, const float *scores, int64_t total, int k,
                                         int64_t *out_ids, float *out_scores) {
    if (k <= 0 || k > total) k = (int)total;
    scored *all = (scored *)malloc(sizeof(scored) * (size_t)(total > 0 ? total : 1));
    for (int64_t i = 0; i < total; i++) {
        all[i].score = scores[i];
        all[i].id = ids[i];
    }
    qsort(all, (size_t)total, sizeof(scored), cmp_better);
    for (int i = 0; i < k; i++) {
        out_ids[i] = all[i].id;
        out_scores[i] = all[i].score;
    }
    free(all);
    return k;
}

/* Multi-vector parents: topTurboQuantMultiVectorParentScores + accumulator + aggregation,
 * runtime/retrieval_multivector_turboquant.go:746-810, 890-907.  child_scores[c] is the
 * score of child c, parent_of_child[c] in [0, parents).  top_n <= 0 or 1 = "max"
 * aggregation (top_n = 1), otherwise mean of the best min(top_n, 5, count) child scores in
 * double; penalty * log1p(count) subtracted when penalty != 0; parents with no children
 * do not appear.  Result: top-k parents, score desc then parent id asc. */
EOS_ORACLE_API int eos_oracle_parent_topk(const float *child_scores, const int32_t *parent_of_child, int64_t children,
                                          int parents, int top_n, double penalty, int k, int64_t *out_ids,
                                          float *out_scores) {
    float *top = (float *)malloc(sizeof(float) * (size_t)parents * 5);
    int *kept = (int *)calloc((size_t)parents, sizeof(int));
    int *count = (int *)calloc((size_t)parents, sizeof(int));
    for (int64_t c = 0; c < children; c++) {
        int p = parent_of_child[c];
        float *t = top + (size_t)p * 5;
        count[p]++;
        int len = kept[p];
        float s = child_scores[c];
        if (len < 5) {
            t[len] = s;
            len++;
        } else if (s > t[4]) {
            t[4] = s;
        } else {
            continue;
        }
        for (int i = len - 1; i > 0 && t[i] > t[i - 1]; i--) {
            float x = t[i];
            t[i] = t[i - 1];
            t[i - 1] = x;
        }
        kept[p] = len;
    }
    int present = 0;
    float *agg = (float *)malloc(sizeof(float) * (size_t)parents);
    int64_t *pid = (int64_t *)malloc(sizeof(int64_t) * (size_t)parents);
    for (int p = 0; p < parents; p++) {
        if (count[p] == 0) continue;
        int avail = top_n <= 0 ? 1 : top_n; /* "max" and unknown labels aggregate the best child */
        if (avail > kept[p]) avail = kept[p];
        double sum = 0.0;
        for (int i = 0; i < avail; i++) sum += (double)top[(size_t)p * 5 + i];
        double score = sum / (double)avail;
        if (penalty != 0.0) score -= penalty * log1p((double)count[p]);
        agg[present] = (float)score;
        pid[present] = p;
        present++;
    }
    /* top-k over (agg, pid) with ids taken from pid */
    if (k <= 0 || k > present) k = present;
    scored *all = (scored *)malloc(sizeof(scored) * (size_t)(present > 0 ? present : 1));
    for (int i = 0; i < present; i++) {
        all[i].score = agg[i];
        all[i].id = pid[i];
    }
    qsort(all, (size_t)present, sizeof(scored), cmp_better);
    for (int i = 0; i < k; i++) {
        out_ids[i] = all[i].id;
        out_scores[i] = all[i].score;
    }
    free(top);
    free(kept);
    free(count);
    free(agg);
    free(pid);
    free(all);
    return k;
}

/* dotRetrievalVectors: runtime/retrieval_eval.go:1189-1199 (float accumulate) */
EOS_ORACLE_API float eos_oracle_dot(const float *a, const float *b, int n) {
    float sum = 0.0f;
    for (int i = 0; i < n; i++) sum += a[i] * b[i];
    return sum;
}

/* dotRows: runtime/backend/tensor_ops.go:1967-1995 (one query against every row, float accumulate in
 * column order).  out[r] for r in [0, rows). */
EOS_ORACLE_API void eos_oracle_dot_rows(const float *query, const float *docs, int64_t rows, int cols, float *out) {
    for (int64_t r = 0; r < rows; r++) {
        float sum = 0.0f;
        const float *d = docs + r * (int64_t)cols;
        for (int c = 0; c < cols; c++) sum += query[c] * d[c];
        out[r] = sum;
    }
}

/* cosineRows: runtime/backend/tensor_ops.go:1997-2057 (double accumulation of the dot product and of
 * both squared norms; a zero denominator gives 0). */
EOS_ORACLE_API void eos_oracle_cosine_rows(const float *query, const float *docs, int64_t rows, int cols, float *out) {
    double qn = 0.0;
    for (int c = 0; c < cols; c++) qn += (double)query[c] * (double)query[c];
    for (int64_t r = 0; r < rows; r++) {
        double dot = 0.0, dn = 0.0;
        const float *d = docs + r * (int64_t)cols;
        for (int c = 0; c < cols; c++) {
            dot += (double)query[c] * (double)d[c];
            dn += (double)d[c] * (double)d[c];
        }
        const double denom = sqrt(qn) * sqrt(dn);
        out[r] = denom == 0.0 ? 0.0f : (float)(dot / denom);
    }
}

/* ropeRows: runtime/backend/tensor_ops.go:1936-1965.  `in` is [rows, cols]; the position of row r is
 * r % seq_rows (seq_rows = rows for a rank-2 input, = T for a [B, T, cols] input); the angle is computed
 * in double and its cosine / sine rounded to float before the rotation of each (even, odd) pair. */
EOS_ORACLE_API void eos_oracle_rope_rows(const float *in, int64_t rows, int seq_rows, int cols, float *out) {
    memcpy(out, in, sizeof(float) * (size_t)rows * (size_t)cols);
    for (int64_t r = 0; r < rows; r++) {
        const int64_t pos = r % seq_rows;
        for (int c = 0; c + 1 < cols; c += 2) {
            const double theta = (double)pos / pow(10000.0, (double)c / (double)cols);
            const float cos_t = (float)cos(theta), sin_t = (float)sin(theta);
            const float x0 = in[r * cols + c], x1 = in[r * cols + c + 1];
            out[r * cols + c] = x0 * cos_t - x1 * sin_t;
            out[r * cols + c + 1] = x0 * sin_t + x1 * cos_t;
        }
    }
}

/* layerNormRows (non-affine, epsilon 1e-5, float statistics): runtime/backend/tensor_ops.go:1393-1421. */
EOS_ORACLE_API void eos_oracle_layernorm_rows(const float *in, int64_t rows, int cols, float *out) {
    for (int64_t r = 0; r < rows; r++) {
        const float *x = in + r * (int64_t)cols;
        float mean = 0.0f;
        for (int c = 0; c < cols; c++) mean += x[c];
        mean /= (float)cols;
        float variance = 0.0f;
        for (int c = 0; c < cols; c++) {
            const float centered = x[c] - mean;
            variance += centered * centered;
        }
        variance /= (float)cols;
        const float inv_std = (float)(1.0 / sqrt((double)variance + 1e-5));
        for (int c = 0; c < cols; c++) out[r * (int64_t)cols + c] = (x[c] - mean) * inv_std;
    }
}

/* geluTensor with its float intermediates: runtime/backend/tensor_ops.go:1926-1934. */
EOS_ORACLE_API void eos_oracle_gelu_tanh_rows(const float *in, int64_t n, float *out) {
    for (int64_t i = 0; i < n; i++) {
        const float x = in[i];
        const float cubic = x * x * x;
        const float inner = 0.7978845608f * (x + 0.044715f * cubic);
        out[i] = 0.5f * x * (1.0f + (float)tanh((double)inner));
    }
}

/* ------------------------------------------------------------------------------------ */
/* Token-pool encoder and token-span child vectors                                       */
/* ------------------------------------------------------------------------------------ */

/* geluForward: runtime/embedding_trainer.go:13471-13475 (float arithmetic, tanh in double) */
static float tp_gelu(float x) {
    float cubic = x * x * x;
    float inner = 0.7978845608f * (x + 0.044715f * cubic);
    return 0.5f * x * (1.0f + (float)tanh((double)inner));
}

/* matmulRowsRight: runtime/sparse_token_pool_vector_export.go:1620-1633 (weight [in, out], float sum in i order) */
static void tp_matmul(const float *rows, int row_count, int in_dim, const float *w, int out_dim, float *out) {
    for (int r = 0; r < row_count; r++)
        for (int o = 0; o < out_dim; o++) {
            float sum = 0.0f;
            for (int i = 0; i < in_dim; i++) sum += rows[(int64_t)r * in_dim + i] * w[(int64_t)i * out_dim + o];
            out[(int64_t)r * out_dim + o] = sum;
        }
}

/* layerNormRow: runtime/embedding_trainer.go:13005-13024 */
static void tp_layernorm_rows(const float *rows, int row_count, int dim, float *out) {
    for (int r = 0; r < row_count; r++) {
        const float *src = rows + (int64_t)r * dim;
        float *dst = out + (int64_t)r * dim;
        float mean = 0.0f;
        for (int i = 0; i < dim; i++) mean += src[i];
        mean /= (float)dim;
        float variance = 0.0f;
        for (int i = 0; i < dim; i++) {
            float centered = src[i] - mean;
            variance += centered * centered;
        }
        variance /= (float)dim;
        float inv_std = (float)(1.0 / sqrt((double)variance + 1e-5));
        for (int i = 0; i < dim; i++) dst[i] = (src[i] - mean) * inv_std;
    }
}

/* normalizeRetrievalVector: runtime/retrieval_eval.go:1040-1054 */
static void tp_normalize(float *v, int dim) {
    double sum = 0.0;
    for (int i = 0; i < dim; i++) sum += (double)v[i] * (double)v[i];
    if (sum == 0.0) return;
    float scale = (float)(1.0 / sqrt(sum));
    for (int i = 0; i < dim; i++) v[i] *= scale;
}

/* denseSoftmaxAttentionRows: runtime/sparse_token_pool_vector_export.go:1430-1465 */
static void tp_dense_attention(const float *q, const float *k, const float *v, int seq_len, int dim, float *out) {
    float *scores = (float *)malloc(sizeof(float) * (size_t)seq_len);
    memset(out, 0, sizeof(float) * (size_t)seq_len * dim);
    for (int row = 0; row < seq_len; row++) {
        float max_score = -INFINITY;
        for (int col = 0; col < seq_len; col++) {
            float score = 0.0f;
            for (int d = 0; d < dim; d++) score += q[(int64_t)row * dim + d] * k[(int64_t)col * dim + d];
            scores[col] = score;
            if (score > max_score) max_score = score;
        }
        float sum = 0.0f;
        for (int col = 0; col < seq_len; col++) {
            float prob = (float)exp((double)(scores[col] - max_score));
            scores[col] = prob;
            sum += prob;
        }
        if (sum == 0.0f) continue;
        for (int col = 0; col < seq_len; col++) {
            float prob = scores[col] / sum;
            for (int d = 0; d < dim; d++) out[(int64_t)row * dim + d] += prob * v[(int64_t)col * dim + d];
        }
    }
    free(scores);
}

/* sparseTokenPoolEncoder.embedTextFullEncoderRows: runtime/sparse_token_pool_vector_export.go:1301-1335.
 * weights: token_embedding [vocab, dim], attention q / k / v / output [dim, dim], hidden_projection [dim, hidden],
 * projection [hidden, dim]; flags = {attention_residual, attention_layer_norm, ffn_residual, ffn_layer_norm}.
 * mode 0: dense attention; mode 1: key / value rows TurboQuant-encoded (codes + 8-bit log norm, :1369-1401 with
 * runtime/backend/image_ops.go:212-249), decoded, sparse attention with top_k / route knobs.  kspec / vspec =
 * {perm, signs1, signs2, centroids, boundaries} of the key / value quantisers (the module that derives them from a
 * seed is not in the reference tree; the caller supplies them). */
EOS_ORACLE_API void eos_oracle_token_pool_rows(const float *token_embedding, int vocab, int dim, int hidden,
                                               const float *wq, const float *wk, const float *wv, const float *wo,
                                               const float *w1, const float *w2, int repeats, const int32_t *flags,
                                               const int32_t *tokens, int seq_len, int mode, int key_bits,
                                               const int32_t *kperm, const float *ks1, const float *ks2,
                                               const float *kcent, const float *kbound, int value_bits,
                                               const int32_t *vperm, const float *vs1, const float *vs2,
                                               const float *vcent, const float *vbound, int top_k,
                                               int route_block_size, int route_top_blocks, float *rows_out) {
    size_t td = (size_t)seq_len * dim;
    float *cur = (float *)calloc(td, sizeof(float));
    float *q = (float *)malloc(sizeof(float) * td), *k = (float *)malloc(sizeof(float) * td);
    float *v = (float *)malloc(sizeof(float) * td), *att = (float *)malloc(sizeof(float) * td);
    float *hid = (float *)malloc(sizeof(float) * td), *tmp = (float *)malloc(sizeof(float) * td);
    float *ffn = (float *)malloc(sizeof(float) * (size_t)seq_len * hidden);
    for (int i = 0; i < seq_len; i++) {   /* gatherTokenRows :1337-1349: rows of unknown ids stay zero */
        int tok = tokens[i];
        if (tok >= 0 && tok < vocab) memcpy(cur + (size_t)i * dim, token_embedding + (size_t)tok * dim, sizeof(float) * dim);
    }
    for (int layer = 0; layer < repeats; layer++) {
        tp_matmul(cur, seq_len, dim, wq, dim, q);
        tp_matmul(cur, seq_len, dim, wk, dim, k);
        tp_matmul(cur, seq_len, dim, wv, dim, v);
        if (mode == 0) {
            tp_dense_attention(q, k, v, seq_len, dim, att);
        } else {
            for (int side = 0; side < 2; side++) {
                int bits = side == 0 ? key_bits : value_bits;
                float *rowsf = side == 0 ? k : v;
                int64_t cb = eos_oracle_tq_code_bytes(dim, bits);
                uint8_t *codes = (uint8_t *)malloc((size_t)seq_len * cb);
                float *norms = (float *)malloc(sizeof(float) * (size_t)seq_len);
                uint8_t *ncodes = (uint8_t *)malloc((size_t)seq_len);
                eos_oracle_tq_encode(rowsf, seq_len, dim, bits, side == 0 ? kperm : vperm, side == 0 ? ks1 : vs1,
                                     side == 0 ? ks2 : vs2, side == 0 ? kbound : vbound, codes, norms);
                eos_oracle_tq_norm_code(norms, seq_len, ncodes);
                eos_oracle_tq_norm_value(ncodes, seq_len, norms);
                eos_oracle_tq_decode(codes, norms, seq_len, dim, bits, side == 0 ? kperm : vperm, side == 0 ? ks1 : vs1,
                                     side == 0 ? ks2 : vs2, side == 0 ? kcent : vcent, rowsf);
                free(codes);
                free(norms);
                free(ncodes);
            }
            eos_oracle_sparse_attention(q, k, v, 1, seq_len, seq_len, dim, dim, top_k, route_block_size, route_top_blocks,
                                        att);
        }
        tp_matmul(att, seq_len, dim, wo, dim, hid);
        if (flags[0])
            for (size_t i = 0; i < td; i++) hid[i] = hid[i] + cur[i];
        if (flags[1]) {
            tp_layernorm_rows(hid, seq_len, dim, tmp);
            float *t = hid;
            hid = tmp;
            tmp = t;
        }
        tp_matmul(hid, seq_len, dim, w1, hidden, ffn);
        for (size_t i = 0; i < (size_t)seq_len * hidden; i++) ffn[i] = tp_gelu(ffn[i]);
        tp_matmul(ffn, seq_len, hidden, w2, dim, tmp);
        if (flags[2])
            for (size_t i = 0; i < td; i++) tmp[i] = tmp[i] + hid[i];
        if (flags[3]) {
            tp_layernorm_rows(tmp, seq_len, dim, cur);
        } else {
            float *t = cur;
            cur = tmp;
            tmp = t;
        }
    }
    for (int r = 0; r < seq_len; r++) tp_normalize(cur + (size_t)r * dim, dim);
    memcpy(rows_out, cur, sizeof(float) * td);
    free(cur);
    free(q);
    free(k);
    free(v);
    free(att);
    free(hid);
    free(tmp);
    free(ffn);
}

/* poolSparseTokenRowsRange (:1597-1618) when fallback_all == 0, maskedMeanPoolNormalized (:1534-1559) otherwise.
 * Returns the number of active rows (0 with fallback_all == 0: no vector is produced). */
EOS_ORACLE_API int eos_oracle_token_span_pool(const float *rows, const int32_t *mask, int start, int end, int dim,
                                              int fallback_all, float *out) {
    int active = 0;
    for (int d = 0; d < dim; d++) out[d] = 0.0f;
    for (int r = start; r < end; r++) {
        if (mask[r] == 0) continue;
        active++;
        for (int d = 0; d < dim; d++) out[d] += rows[(int64_t)r * dim + d];
    }
    if (active == 0) {
        if (!fallback_all) return 0;
        active = end - start;
        for (int r = start; r < end; r++)
            for (int d = 0; d < dim; d++) out[d] += rows[(int64_t)r * dim + d];
    }
    float scale = (float)(1.0 / (double)active);
    for (int d = 0; d < dim; d++) out[d] *= scale;
    tp_normalize(out, dim);
    return active;
}

/* sparseTokenPoolTokenSpans: runtime/sparse_token_pool_vector_export.go:1561-1595.  Returns the span count;
 * starts / ends hold at most cap entries. */
EOS_ORACLE_API int eos_oracle_token_spans(int token_count, int span_tokens, int overlap, int min_tokens, int32_t *starts,
                                          int32_t *ends, int cap) {
    int n = 0;
    if (token_count <= 0 || span_tokens <= 0) return 0;
    if (min_tokens <= 0) min_tokens = 1;
    if (token_count <= span_tokens) {
        if (token_count < min_tokens) return 0;
        if (cap > 0) {
            starts[0] = 0;
            ends[0] = token_count;
        }
        return 1;
    }
    int step = span_tokens - overlap;
    if (step <= 0) return 0;
    for (int start = 0; start < token_count; start += step) {
        int end = start + span_tokens;
        if (end > token_count) end = token_count;
        if (end - start < min_tokens) break;
        if (n < cap) {
            starts[n] = start;
            ends[n] = end;
        }
        n++;
        if (end >= token_count) break;
    }
    return n;
}
