// Top-k sparse attention and its TurboQuant-compressed K/V variant.
//
// Reference semantics: sparseAttentionTensor / turboSparseAttentionTensor, runtime/backend/attention_ops.go:218-300
// (device twins: sparseAttentionKernelSource, runtime/backends/cuda/native_linux.go:2044-2339).  Per query row:
// scores q.k (fp32, accumulated in d order, no 1/sqrt(d)); the `budget` best keys by score descending then index
// ascending, optionally routed through the `top_blocks` key blocks whose anchor (the block's middle key) scores
// best; softmax over the selected scores (exp in double); out = sum of float(w / denom) * v in selection order.
//
// One warp per query row.  Scores are computed without fused multiply-add, in the reference's order, so the
// selection is the reference's selection bit for bit; the best `budget` candidates of a stream are kept with a
// 256-slot list in shared memory that one warp sorts (bitonic) whenever it is full.  The value mix runs one output
// column per lane, keys in selection order, so every output element is the reference's sequence of fp32 adds.
#include "sparse_attention.cuh"

#include <cmath>

#include "common.cuh"
#include "turboquant.cuh"
#include "turboquant_dev.cuh"

namespace eosb {

namespace {

constexpr int kSaWarps = 4;

// norm of an 8-bit log code, exp(-16 + 32 code / 255) (native_linux.go:1895-1904), tabulated on the host so that the
// values are the host library's expf
__constant__ float c_norm_of_code[256];

// q . k with separate multiply and add, d ascending (the reference's float loop)
__device__ __forceinline__ float dot_in_order(const float* __restrict__ q, const float* __restrict__ k, int dim) {
    float sum = 0.f;
    if ((dim & 3) == 0 && ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(q)) & 15u) == 0) {
        // 16-byte loads, the same adds in the same order
        const float4* k4 = reinterpret_cast<const float4*>(k);
        const float4* q4 = reinterpret_cast<const float4*>(q);
#pragma unroll 4
        for (int d = 0; d < (dim >> 2); ++d) {
            const float4 kv = __ldg(k4 + d);
            const float4 qv = q4[d];
            sum = __fadd_rn(sum, __fmul_rn(qv.x, kv.x));
            sum = __fadd_rn(sum, __fmul_rn(qv.y, kv.y));
            sum = __fadd_rn(sum, __fmul_rn(qv.z, kv.z));
            sum = __fadd_rn(sum, __fmul_rn(qv.w, kv.w));
        }
        return sum;
    }
    for (int d = 0; d < dim; ++d) sum = __fadd_rn(sum, __fmul_rn(q[d], __ldg(k + d)));
    return sum;
}

// Keeps the best `keep` (<= kSaMaxBudget) keys of a stream of `count` items in list[0 .. keep); item(i) returns the
// sortable key of item i (0 = skip).  Returns the number of keys kept.
template <typename F>
__device__ int warp_top_keys(u64* list, int keep, int count, int lane, F&& item) {
    int fill = 0;   // multiple of 32, <= 224 before an append
    int seen = 0;
    for (int base = 0; base < count; base += 32) {
        const int i = base + lane;
        list[fill + lane] = i < count ? item(i) : 0ull;
        fill += 32;
        __syncwarp();
        if (fill == kSortCap) {
            warp_sort_desc(list, kSortCap, lane);
            fill = (keep + 31) & ~31;
            for (int j = keep + lane; j < fill; j += 32) list[j] = 0ull;   // only the best `keep` survive a cut
            __syncwarp();
        }
        seen += 32;
    }
    warp_sort_desc(list, fill, lane);
    int n = count < keep ? count : keep;
    // items that returned 0 (skipped) sort to the end: count the real ones
    int real = 0;
    for (int j = lane; j < n; j += 32) real += list[j] != 0ull;
    for (int o = 16; o > 0; o >>= 1) real += __shfl_xor_sync(0xffffffffu, real, o);
    (void)seen;
    return real;
}

__global__ void __launch_bounds__(kSaWarps * 32)
sparse_attention_kernel(const float* __restrict__ query, const float* __restrict__ key, const float* __restrict__ value,
                        int batches, int q_len, int k_len, int dim, int vdim, int budget, int block_size, int top_blocks,
                        float* __restrict__ out) {
    extern __shared__ __align__(16) uint8_t sa_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    u64* list = reinterpret_cast<u64*>(sa_smem) + (size_t)warp * (kSortCap + kSaMaxBudget);
    u64* blocks = list + kSortCap;                                                   // selected route blocks
    float* qs = reinterpret_cast<float*>(sa_smem + (size_t)kSaWarps * (kSortCap + kSaMaxBudget) * 8) + (size_t)warp * dim;
    float* scale = reinterpret_cast<float*>(sa_smem + (size_t)kSaWarps * (kSortCap + kSaMaxBudget) * 8 +
                                            (size_t)kSaWarps * dim * 4) + (size_t)warp * kSaMaxBudget;
    const long long rows = (long long)batches * q_len;
    for (long long row = (long long)blockIdx.x * kSaWarps + warp; row < rows; row += (long long)gridDim.x * kSaWarps) {
        const int b = (int)(row / q_len);
        const float* kb = key + (size_t)b * k_len * dim;
        const float* vb = value + (size_t)b * k_len * vdim;
        for (int d = lane; d < dim; d += 32) qs[d] = query[row * dim + d];
        __syncwarp();
        int n;
        if (block_size <= 0 || top_blocks <= 0) {
            n = warp_top_keys(list, budget, k_len, lane,
                              [&](int k) { return make_key(dot_in_order(qs, kb + (size_t)k * dim, dim), (uint32_t)k); });
        } else {
            const int block_count = (k_len + block_size - 1) / block_size;
            const int nb = warp_top_keys(list, top_blocks, block_count, lane, [&](int blk) {
                const int start = blk * block_size;
                const int end = min(start + block_size, k_len);
                const int anchor = start + (end - start) / 2;
                return make_key(dot_in_order(qs, kb + (size_t)anchor * dim, dim), (uint32_t)blk);
            });
            for (int j = lane; j < nb; j += 32) blocks[j] = list[j];
            __syncwarp();
            n = warp_top_keys(list, budget, nb * block_size, lane, [&](int i) -> u64 {
                const int blk = (int)(0xffffffffu - (uint32_t)(blocks[i / block_size] & 0xffffffffu));
                const int k = blk * block_size + i % block_size;
                if (k >= k_len) return 0ull;
                return make_key(dot_in_order(qs, kb + (size_t)k * dim, dim), (uint32_t)k);
            });
        }
        float* o = out + row * vdim;
        if (n == 0) {
            for (int d = lane; d < vdim; d += 32) o[d] = 0.f;
            __syncwarp();
            continue;
        }
        // softmax over the selected scores: the list is sorted, so its first score is the maximum; the sum runs in
        // selection order in double, like the reference's loop
        if (lane == 0) {
            const float max_score = ordered_to_float((uint32_t)(list[0] >> 32));
            double denom = 0.0;
            for (int i = 0; i < n; ++i) denom += exp((double)(ordered_to_float((uint32_t)(list[i] >> 32)) - max_score));
            const bool bad = denom == 0.0 || denom != denom;
            for (int i = 0; i < n; ++i) {
                const double w = exp((double)(ordered_to_float((uint32_t)(list[i] >> 32)) - max_score));
                scale[i] = bad ? 0.f : (float)(w / denom);
            }
        }
        __syncwarp();
        for (int d = lane; d < vdim; d += 32) {
            float acc = 0.f;
            for (int i = 0; i < n; ++i) {
                const uint32_t k = 0xffffffffu - (uint32_t)(list[i] & 0xffffffffu);
                acc = __fadd_rn(acc, __fmul_rn(scale[i], __ldg(vb + (size_t)k * vdim + d)));
            }
            o[d] = acc;
        }
        __syncwarp();
    }
}

// Decode of TurboQuant-compressed rows (manta_turboq_decode, native_linux.go:1959-2003): out[v, perm[i]] =
// FWHT(centroids[code[v, perm[.]]] * signs2)[i] * signs1[i] * norm(v), norm from the 8-bit log code.
// One warp per vector; codes are one byte per coordinate, [n, dim].
__global__ void __launch_bounds__(128)
tq_decode_rows_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ norm_codes, long long n, TqSpec s,
                      float* __restrict__ out) {
    extern __shared__ float dec_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* work = dec_smem + (size_t)warp * s.dim;
    const int levels = 1 << s.bits;
    for (long long v = (long long)blockIdx.x * 4 + warp; v < n; v += (long long)gridDim.x * 4) {
        const uint8_t* cv = codes + v * s.dim;
        for (int i = lane; i < s.dim; i += 32) {
            int idx = cv[s.perm[i]];
            idx = idx >= levels ? levels - 1 : idx;
            work[i] = __fmul_rn(s.centroids[idx], s.signs2[i]);
        }
        __syncwarp();
        warp_fwht_blocks(work, s.dim, lane);
        const float norm = c_norm_of_code[norm_codes[v]];
        for (int i = lane; i < s.dim; i += 32)
            out[v * s.dim + s.perm[i]] = __fmul_rn(__fmul_rn(work[i], s.signs1[i]), norm);
        __syncwarp();
    }
}

}  // namespace

size_t sparse_attention_smem_bytes(int dim) {
    return (size_t)kSaWarps * (kSortCap + kSaMaxBudget) * 8 + (size_t)kSaWarps * dim * 4 + (size_t)kSaWarps * kSaMaxBudget * 4;
}

cudaError_t sparse_attention_init() {
    float table[256];
    for (int c = 0; c < 256; ++c) table[c] = expf(-16.0f + ((float)c / 255.0f) * 32.0f);
    cudaError_t e = cudaMemcpyToSymbol(c_norm_of_code, table, sizeof(table));
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(sparse_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
}

void launch_sparse_attention(const float* q, const float* k, const float* v, int batches, int q_len, int k_len, int dim,
                             int vdim, int budget, int block_size, int top_blocks, float* out, int sm_count,
                             cudaStream_t stream) {
    const long long rows = (long long)batches * q_len;
    if (rows <= 0) return;
    long long blocks = (rows + kSaWarps - 1) / kSaWarps;
    if (blocks > (long long)sm_count * 8) blocks = (long long)sm_count * 8;
    sparse_attention_kernel<<<(int)blocks, kSaWarps * 32, sparse_attention_smem_bytes(dim), stream>>>(
        q, k, v, batches, q_len, k_len, dim, vdim, budget, block_size, top_blocks, out);
}

void launch_tq_decode_rows(const uint8_t* codes, const uint8_t* norm_codes, int64_t n, const TqSpec& spec, float* out,
                           int sm_count, cudaStream_t stream) {
    if (n <= 0) return;
    long long blocks = (n + 3) / 4;
    if (blocks > (long long)sm_count * 8) blocks = (long long)sm_count * 8;
    tq_decode_rows_kernel<<<(int)blocks, 128, (size_t)4 * spec.dim * sizeof(float), stream>>>(codes, norm_codes, (long long)n,
                                                                                            spec, out);
}

}  // namespace eosb
