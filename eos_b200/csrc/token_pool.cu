// Token-pool encoder: the reference's fp32 host model behind its token-span child vectors
// (sparseTokenPoolEncoder.embedTextFullEncoderRows, runtime/sparse_token_pool_vector_export.go:1301-1335) as device
// kernels.  The model is small and the reference's arithmetic is float with fixed summation orders, so every
// kernel keeps those orders (separate multiply and add, sums in index order) and the rows come out as the host
// computes them up to the last bit of the two double-precision library calls (tanh, exp); speed is not the point.
#include "token_pool.cuh"

#include <cmath>

namespace eosb {

namespace {

__global__ void tp_gather_kernel(const float* __restrict__ table, int vocab, int dim, const int32_t* __restrict__ tokens,
                                 int n, float* __restrict__ out) {
    const long long total = (long long)n * dim;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / dim), d = (int)(i - (long long)r * dim);
        const int tok = tokens[r];
        out[i] = (tok >= 0 && tok < vocab) ? table[(size_t)tok * dim + d] : 0.f;
    }
}

// geluForward (runtime/embedding_trainer.go:13471-13475): float arithmetic, tanh in double
__device__ __forceinline__ float tp_gelu(float x) {
    const float cubic = __fmul_rn(__fmul_rn(x, x), x);
    const float inner = __fmul_rn(0.7978845608f, __fadd_rn(x, __fmul_rn(0.044715f, cubic)));
    return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, (float)tanh((double)inner)));
}

// thread = one output element; the weight row i is read by consecutive threads
__global__ void __launch_bounds__(128)
tp_matmul_kernel(const float* __restrict__ rows, int row_count, int in_dim, const float* __restrict__ w, int out_dim,
                 int epilogue, float* __restrict__ out) {
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (o >= out_dim || r >= row_count) return;
    const float* x = rows + (size_t)r * in_dim;
    float sum = 0.f;
    for (int i = 0; i < in_dim; ++i) sum = __fadd_rn(sum, __fmul_rn(x[i], __ldg(w + (size_t)i * out_dim + o)));
    out[(size_t)r * out_dim + o] = epilogue == 1 ? tp_gelu(sum) : sum;
}

__global__ void tp_add_kernel(const float* a, const float* b, long long n, float* out) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = __fadd_rn(a[i], b[i]);
}

// thread = one row: the three passes of layerNormRow are sequential float sums
__global__ void tp_layernorm_kernel(const float* __restrict__ rows, int row_count, int dim, float* __restrict__ out) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= row_count) return;
    const float* x = rows + (size_t)r * dim;
    float mean = 0.f;
    for (int i = 0; i < dim; ++i) mean = __fadd_rn(mean, x[i]);
    mean = __fdiv_rn(mean, (float)dim);
    float var = 0.f;
    for (int i = 0; i < dim; ++i) {
        const float c = __fsub_rn(x[i], mean);
        var = __fadd_rn(var, __fmul_rn(c, c));
    }
    var = __fdiv_rn(var, (float)dim);
    const float inv = (float)(1.0 / sqrt((double)var + 1e-5));
    for (int i = 0; i < dim; ++i) out[(size_t)r * dim + i] = __fmul_rn(__fsub_rn(x[i], mean), inv);
}

__device__ __forceinline__ void tp_normalize_row(float* x, int dim) {
    double sum = 0.0;
    for (int i = 0; i < dim; ++i) sum += (double)x[i] * (double)x[i];
    if (sum == 0.0) return;
    const float scale = (float)(1.0 / sqrt(sum));
    for (int i = 0; i < dim; ++i) x[i] = __fmul_rn(x[i], scale);
}

__global__ void tp_normalize_kernel(float* __restrict__ rows, int row_count, int dim) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < row_count) tp_normalize_row(rows + (size_t)r * dim, dim);
}

// One warp per query row.  Scores: a lane per key, the dot product in d order.  The maximum is order-free; the sum of
// the probabilities is the reference's sequential float sum (lane 0); the value mix runs one output column per lane
// over the keys in order.
__global__ void __launch_bounds__(128)
tp_dense_attention_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, int seq_len,
                          int dim, float* __restrict__ scores, float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < seq_len; row += warps) {
        const float* qr = q + (size_t)row * dim;
        float* sc = scores + (size_t)row * seq_len;
        float mx = -INFINITY;
        for (int col = lane; col < seq_len; col += 32) {
            const float* kr = k + (size_t)col * dim;
            float s = 0.f;
            for (int d = 0; d < dim; ++d) s = __fadd_rn(s, __fmul_rn(qr[d], kr[d]));
            sc[col] = s;
            mx = fmaxf(mx, s);
        }
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        __syncwarp();
        for (int col = lane; col < seq_len; col += 32) sc[col] = (float)exp((double)__fsub_rn(sc[col], mx));
        __syncwarp();
        float sum = 0.f;
        if (lane == 0)
            for (int col = 0; col < seq_len; ++col) sum = __fadd_rn(sum, sc[col]);
        sum = __shfl_sync(0xffffffffu, sum, 0);
        float* o_row = out + (size_t)row * dim;
        if (sum == 0.f) {
            for (int d = lane; d < dim; d += 32) o_row[d] = 0.f;
        } else {
            for (int d = lane; d < dim; d += 32) {
                float acc = 0.f;
                for (int col = 0; col < seq_len; ++col)
                    acc = __fadd_rn(acc, __fmul_rn(__fdiv_rn(sc[col], sum), __ldg(v + (size_t)col * dim + d)));
                o_row[d] = acc;
            }
        }
        __syncwarp();
    }
}

// One block per span: a thread per column sums the active rows in order, thread 0 normalises.
__global__ void __launch_bounds__(256)
tp_span_pool_kernel(const float* __restrict__ rows, const int32_t* __restrict__ mask, const int* __restrict__ starts,
                    const int* __restrict__ ends, int dim, int fallback_all, float* __restrict__ out, int* __restrict__ flags) {
    const int s = blockIdx.x;
    const int start = starts[s], end = ends[s];
    __shared__ int s_active;
    if (threadIdx.x == 0) {
        int active = 0;
        for (int r = start; r < end; ++r) active += mask[r] != 0;
        s_active = active;
    }
    __syncthreads();
    int active = s_active;
    const bool all = active == 0 && fallback_all != 0;
    float* o = out + (size_t)s * dim;
    if (active == 0 && !all) {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) o[d] = 0.f;
        if (threadIdx.x == 0 && flags != nullptr) flags[s] = 1;
        return;
    }
    if (all) active = end - start;
    const float scale = (float)(1.0 / (double)active);
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float acc = 0.f;
        for (int r = start; r < end; ++r)
            if (all || mask[r] != 0) acc = __fadd_rn(acc, rows[(size_t)r * dim + d]);
        o[d] = __fmul_rn(acc, scale);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        tp_normalize_row(o, dim);
        if (flags != nullptr) flags[s] = 0;
    }
}

__global__ void tp_unpack_codes_kernel(const uint8_t* __restrict__ packed, long long n, int dim, int bits,
                                       uint8_t* __restrict__ out) {
    const int per_byte = 8 / bits;
    const unsigned maskv = (1u << bits) - 1u;
    const long long cb = ((long long)dim * bits + 7) / 8;
    const long long total = n * dim;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long v = i / dim;
        const int c = (int)(i - v * dim);
        out[i] = (uint8_t)((packed[v * cb + c / per_byte] >> ((c % per_byte) * bits)) & maskv);
    }
}

inline int grid_for(long long total, int block) {
    long long g = (total + block - 1) / block;
    return (int)(g < 1 ? 1 : (g > 65535 ? 65535 : g));
}

}  // namespace

void launch_tp_gather(const float* table, int vocab, int dim, const int32_t* tokens, int n, float* out, cudaStream_t s) {
    if (n <= 0) return;
    tp_gather_kernel<<<grid_for((long long)n * dim, 256), 256, 0, s>>>(table, vocab, dim, tokens, n, out);
}

void launch_tp_matmul(const float* rows, int row_count, int in_dim, const float* w, int out_dim, int epilogue, float* out,
                      cudaStream_t s) {
    if (row_count <= 0 || out_dim <= 0) return;
    tp_matmul_kernel<<<dim3((out_dim + 127) / 128, row_count), 128, 0, s>>>(rows, row_count, in_dim, w, out_dim, epilogue, out);
}

void launch_tp_add(const float* a, const float* b, long long n, float* out, cudaStream_t s) {
    if (n <= 0) return;
    tp_add_kernel<<<grid_for(n, 256), 256, 0, s>>>(a, b, n, out);
}

void launch_tp_layernorm(const float* rows, int row_count, int dim, float* out, cudaStream_t s) {
    if (row_count <= 0) return;
    tp_layernorm_kernel<<<(row_count + 63) / 64, 64, 0, s>>>(rows, row_count, dim, out);
}

void launch_tp_normalize(float* rows, int row_count, int dim, cudaStream_t s) {
    if (row_count <= 0) return;
    tp_normalize_kernel<<<(row_count + 63) / 64, 64, 0, s>>>(rows, row_count, dim);
}

void launch_tp_dense_attention(const float* q, const float* k, const float* v, int seq_len, int dim, float* scores,
                               float* out, int sm_count, cudaStream_t s) {
    if (seq_len <= 0) return;
    int blocks = (seq_len + 3) / 4;
    if (blocks > sm_count * 8) blocks = sm_count * 8;
    tp_dense_attention_kernel<<<blocks, 128, 0, s>>>(q, k, v, seq_len, dim, scores, out);
}

void launch_tp_span_pool(const float* rows, const int32_t* mask, const int* starts, const int* ends, int spans, int dim,
                         int fallback_all, float* out, int* flags, cudaStream_t s) {
    if (spans <= 0) return;
    tp_span_pool_kernel<<<spans, 256, 0, s>>>(rows, mask, starts, ends, dim, fallback_all, out, flags);
}

void launch_tp_unpack_codes(const uint8_t* packed, long long n, int dim, int bits, uint8_t* out, cudaStream_t s) {
    if (n <= 0) return;
    tp_unpack_codes_kernel<<<grid_for(n * dim, 256), 256, 0, s>>>(packed, n, dim, bits, out);
}

}  // namespace eosb
