// Bandwidth-bound pieces of the q8 encoder forward and its attention, for sm_100a.
//
// Reference semantics restated here (file:line inside the Eos project):
//   embeddings + LayerNorm   runtime/backend/tensor_ops.go:1451-1512
//                            (device twin: manta_bert_embedding_affine_layernorm,
//                             runtime/backends/cuda/native_linux.go:2700-2753)
//   LayerNorm(x + residual)  runtime/backend/bert_encoder_layer_ops.go:718-740
//   self-attention           runtime/backend/bert_encoder_layer_ops.go:326-379
//                            (device twin: manta_bert_attention_context, native_linux.go:2857-2969)
//   masked mean / CLS + L2   runtime/backend/tensor_ops.go:1680-1705, 1367-1391;
//                            runtime/backend/bert_embedder_ops.go:174-218
//   projection head + L2     runtime/pretrained_bert_projection_head.go:84-100
//   compiled pipeline        examples/embed_masked_pooled.eos:11-16
//
// Unlike the reference, rows whose attention_mask is zero are never materialised: they cannot
// influence a kept row (keys are masked, pooling skips them), so the batch is packed to its
// valid tokens first and every later kernel works on packed rows.
#include "encoder_kernels.cuh"

#include <type_traits>

#include "common.cuh"

namespace eosb {

namespace {

// ------------------------------------------------------------------------------------------
// sequence layout
// ------------------------------------------------------------------------------------------
__global__ void seq_count_kernel(const int32_t* __restrict__ mask, int tokens, int cls_pooling, int* key_count,
                                 int* row_count) {
    const int b = blockIdx.x;
    const int32_t* m = mask + (size_t)b * tokens;
    int local = 0;
    for (int t = threadIdx.x; t < tokens; t += blockDim.x) local += (m[t] != 0);
    __shared__ int warp_tot[32];
    int w = local;
    for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
    if ((threadIdx.x & 31) == 0) warp_tot[threadIdx.x >> 5] = w;
    __syncthreads();
    if (threadIdx.x == 0) {
        int total = 0;
        for (int i = 0; i < (blockDim.x + 31) / 32; ++i) total += warp_tot[i];
        key_count[b] = total;
        row_count[b] = total + ((cls_pooling && m[0] == 0) ? 1 : 0);
    }
}

__global__ void seq_scan_kernel(const int* row_count, int batch, int unit, int* cu_rows, int* total_rows) {
    // single block; sequential chunks of blockDim.x with a running carry; scans ceil(row_count / unit)
    __shared__ int buf[1024];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < batch; base += blockDim.x) {
        const int i = base + threadIdx.x;
        const int v = i < batch ? (row_count[i] + unit - 1) / unit : 0;
        buf[threadIdx.x] = v;
        __syncthreads();
        for (int o = 1; o < blockDim.x; o <<= 1) {
            int add = threadIdx.x >= o ? buf[threadIdx.x - o] : 0;
            __syncthreads();
            buf[threadIdx.x] += add;
            __syncthreads();
        }
        if (i < batch) cu_rows[i] = carry + buf[threadIdx.x] - v;
        __syncthreads();
        if (threadIdx.x == 0) carry += buf[blockDim.x - 1];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        cu_rows[batch] = carry;
        if (total_rows != nullptr) *total_rows = carry;
    }
}

__global__ void seq_fill_kernel(const int32_t* __restrict__ mask, int tokens, int cls_pooling, const int* cu_rows,
                                const int* key_count, const int* cu_qtiles, int window, int* row_src, int* cls_row,
                                int4* qtile_info, int4* qtile_win) {
    const int b = blockIdx.x;
    const int32_t* m = mask + (size_t)b * tokens;
    const int row0 = cu_rows[b];
    __shared__ int warp_off[33];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int base = 0; base < tokens; base += blockDim.x) {
        const int t = base + threadIdx.x;
        const int valid = (t < tokens) && (m[t] != 0);
        const unsigned bal = __ballot_sync(0xffffffffu, valid);
        if (lane == 0) warp_off[warp] = __popc(bal);
        __syncthreads();
        if (threadIdx.x == 0) {
            int run = carry;
            for (int i = 0; i < nwarps; ++i) {
                int c = warp_off[i];
                warp_off[i] = run;
                run += c;
            }
            warp_off[32] = run;
        }
        __syncthreads();
        if (valid) row_src[row0 + warp_off[warp] + __popc(bal & ((1u << lane) - 1u))] = b * tokens + t;
        __syncthreads();
        if (threadIdx.x == 0) carry = warp_off[32];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        if (cls_pooling && m[0] == 0) {
            // token 0 is masked: it is still a query (the reference computes every row and CLS
            // pooling reads row 0), so it gets a query-only row after the sequence's keys.
            row_src[row0 + key_count[b]] = b * tokens;
            cls_row[b] = row0 + key_count[b];
        } else {
            cls_row[b] = row0;
        }
    }
    __syncthreads();  // row_src of this sequence is complete (written by this block only)
    {
        const int nrows = cu_rows[b + 1] - row0;
        const int nkeys = key_count[b];
        const int ntiles = (nkeys + 127) >> 7;
        const int qt0 = cu_qtiles[b];
        for (int q = threadIdx.x; q < cu_qtiles[b + 1] - qt0; q += blockDim.x) {
            qtile_info[qt0 + q] = make_int4(row0, nrows, nkeys, q * 128);
            // key tiles (of 128 keys) the tile's queries can see, and among them the ones every query sees in
            // full; positions grow along the packed keys, so both are contiguous ranges
            int kb = 0, ke = ntiles, fb = 0, fe = ntiles;
            if (window > 0 && nkeys > 0) {
                const int q0 = q * 128;
                const int qlast = min(q0 + 127, nrows - 1);
                int qlo = row_src[row0 + q0], qhi = row_src[row0 + qlast];
                const bool has_cls_row = nrows > nkeys && qlast == nrows - 1;  // query-only row at position 0
                if (has_cls_row) {
                    qlo = b * tokens;
                    qhi = q0 < nkeys ? row_src[row0 + nkeys - 1] : b * tokens;
                }
                auto first_pos = [&](int t) { return row_src[row0 + t * 128]; };
                auto last_pos = [&](int t) { return row_src[row0 + min(t * 128 + 127, nkeys - 1)]; };
                while (kb < ke && 2 * (qlo - last_pos(kb)) >= window) ++kb;
                while (ke > kb && 2 * (first_pos(ke - 1) - qhi) >= window) --ke;
                auto full = [&](int t) {
                    return !has_cls_row && 2 * (qhi - first_pos(t)) < window && 2 * (last_pos(t) - qlo) < window;
                };
                fb = kb;
                while (fb < ke && !full(fb)) ++fb;
                fe = fb;
                while (fe < ke && full(fe)) ++fe;
            }
            qtile_win[qt0 + q] = make_int4(kb, ke, fb, fe);
        }
    }
}

// Orders the 128-query tiles by the number of key tiles each visits, most first (a counting sort in one block).
// The attention kernel deals tiles out round-robin over its workers; in sequence order the workers' sums differ by
// several percent (the slowest one sets the kernel's time), in this order by at most a tile or two.  Tiles of equal
// cost land in no particular order: every tile's result is independent of where it runs.
constexpr int kQtileCostBins = 66;   // costs 0 .. 64 key tiles, anything above shares the top bin
__global__ void qtile_sort_kernel(const int* __restrict__ cu_qtiles, int batch, const int4* __restrict__ info_seq,
                                  const int4* __restrict__ win_seq, int4* __restrict__ info, int4* __restrict__ win) {
    __shared__ int count[kQtileCostBins];
    __shared__ int start[kQtileCostBins];
    const int total = cu_qtiles[batch];
    for (int i = threadIdx.x; i < kQtileCostBins; i += blockDim.x) count[i] = 0;
    __syncthreads();
    auto bin_of = [](const int4& w) { return max(0, min(w.y - w.x, kQtileCostBins - 1)); };
    for (int i = threadIdx.x; i < total; i += blockDim.x) atomicAdd(&count[bin_of(win_seq[i])], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int b = kQtileCostBins - 1; b >= 0; --b) {
            start[b] = run;
            run += count[b];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int4 w = win_seq[i];
        const int at = atomicAdd(&start[bin_of(w)], 1);
        win[at] = w;
        info[at] = info_seq[i];
    }
}

// ------------------------------------------------------------------------------------------
// row-wise kernels: one warp per row, 8 f16 per 16-byte access, kChunks accesses per lane
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 u;
    __half2 h0 = __floats2half2_rn(f[0], f[1]), h1 = __floats2half2_rn(f[2], f[3]);
    __half2 h2 = __floats2half2_rn(f[4], f[5]), h3 = __floats2half2_rn(f[6], f[7]);
    u.x = *reinterpret_cast<uint32_t*>(&h0);
    u.y = *reinterpret_cast<uint32_t*>(&h1);
    u.z = *reinterpret_cast<uint32_t*>(&h2);
    u.w = *reinterpret_cast<uint32_t*>(&h3);
    return u;
}

// LayerNorm of one row held as kChunks x 8 values per lane; two-pass (mean, then centred
// variance) in fp32 like the reference's double-precision two-pass form.
template <int kChunks>
__device__ __forceinline__ void row_mean_inv(const float (&v)[kChunks][8], int dim, int lane, float eps, float* mean_out,
                                             float* inv_out) {
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const int col = (c * 32 + lane) * 8;
        if (col < dim) {
#pragma unroll
            for (int i = 0; i < 8; ++i) sum += v[c][i];
        }
    }
    const float mean = warp_sum(sum) / (float)dim;
    float var = 0.f;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const int col = (c * 32 + lane) * 8;
        if (col < dim) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float d = v[c][i] - mean;
                var += d * d;
            }
        }
    }
    var = warp_sum(var) / (float)dim;
    *mean_out = mean;
    *inv_out = 1.0f / sqrtf(var + eps);
}

// gb: optional shared-memory copy of the scale and shift, [chunk][gamma lo, gamma hi, beta lo, beta hi][lane] (the
// layout of layernorm_kernel); nullptr reads them from global memory.
template <int kChunks>
__device__ __forceinline__ void row_layernorm_store(float (&v)[kChunks][8], int dim, int lane, const float* gamma,
                                                    const float* beta, float eps, __half* out_row,
                                                    const float4 (*gb)[4][32] = nullptr) {
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const int col = (c * 32 + lane) * 8;
        if (col < dim) {
#pragma unroll
            for (int i = 0; i < 8; ++i) sum += v[c][i];
        }
    }
    const float mean = warp_sum(sum) / (float)dim;
    float var = 0.f;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const int col = (c * 32 + lane) * 8;
        if (col < dim) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float d = v[c][i] - mean;
                var += d * d;
            }
        }
    }
    var = warp_sum(var) / (float)dim;
    const float inv = 1.0f / sqrtf(var + eps);
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const int col = (c * 32 + lane) * 8;
        if (col < dim) {
            float o[8];
            const float4 g0 = gb != nullptr ? gb[c][0][lane] : *reinterpret_cast<const float4*>(gamma + col);
            const float4 g1 = gb != nullptr ? gb[c][1][lane] : *reinterpret_cast<const float4*>(gamma + col + 4);
            const float4 b0 = gb != nullptr ? gb[c][2][lane] : *reinterpret_cast<const float4*>(beta + col);
            const float4 b1 = gb != nullptr ? gb[c][3][lane] : *reinterpret_cast<const float4*>(beta + col + 4);
            const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = (v[c][i] - mean) * inv * g[i] + bb[i];
            *reinterpret_cast<uint4*>(out_row + col) = pack8(o);
        }
    }
}

template <int kChunks>
__global__ void __launch_bounds__(256)
embed_ln_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ types, const int* __restrict__ row_src,
                const int* __restrict__ total_rows, int tokens, const __half* __restrict__ tok, int vocab,
                const __half* __restrict__ pos, int max_pos, const __half* __restrict__ typ, int type_vocab,
                const float* __restrict__ gamma, const float* __restrict__ beta, float eps, int dim, int m_alloc,
                __half* __restrict__ out, int* status) {
    __shared__ float4 gb_s[kChunks][4][32];
    const int lane = threadIdx.x & 31;
    const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    int rows = *total_rows;
    if (rows > m_alloc) rows = m_alloc;
    for (int i = threadIdx.x; i < kChunks * 32; i += blockDim.x) {
        const int c = i >> 5, l = i & 31;
        const int col = (c * 32 + l) * 8;
        float g[8], b[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            g[j] = col < dim ? gamma[col + j] : 0.f;
            b[j] = col < dim ? beta[col + j] : 0.f;
        }
        gb_s[c][0][l] = make_float4(g[0], g[1], g[2], g[3]);
        gb_s[c][1][l] = make_float4(g[4], g[5], g[6], g[7]);
        gb_s[c][2][l] = make_float4(b[0], b[1], b[2], b[3]);
        gb_s[c][3][l] = make_float4(b[4], b[5], b[6], b[7]);
    }
    __syncthreads();
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps_per_grid) {
        const int src = row_src[r];
        const int t = src % tokens;
        const int id = ids[src];
        const int ty = types != nullptr ? types[src] : 0;
        int bad = 0;
        if (id < 0 || id >= vocab) bad = kStatusBadTokenId;
        else if (ty < 0 || ty >= type_vocab) bad = kStatusBadTypeId;
        else if (t >= max_pos) bad = kStatusBadPosition;
        if (bad) {
            if (lane == 0) atomicCAS(status, 0, bad);
            continue;  // row left as is; the host reports the status word and discards the result
        }
        const __half* a = tok + (size_t)id * dim;
        const __half* p = pos + (size_t)t * dim;
        const __half* q = typ + (size_t)ty * dim;
        float v[kChunks][8];
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
            const int col = (c * 32 + lane) * 8;
            if (col < dim) {
                float fa[8], fp[8], fq[8];
                unpack8(*reinterpret_cast<const uint4*>(a + col), fa);
                unpack8(*reinterpret_cast<const uint4*>(p + col), fp);
                unpack8(*reinterpret_cast<const uint4*>(q + col), fq);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[c][i] = (fa[i] + fp[i]) + fq[i];
            }
        }
        row_layernorm_store<kChunks>(v, dim, lane, gamma, beta, eps, out + (size_t)r * dim, gb_s);
    }
}

// One warp per row; the next row of a warp is requested before the current one is reduced.  The scale and shift sit
// in shared memory, laid out so that a lane's four 16-byte reads per chunk are conflict-free: held in registers they
// cost 48 registers per lane at 768 columns and halve the warps per SM (4.27 ms per 24 launches at 289,879 x 768
// against 3.85 ms this way); read per row from global memory they are four times the bytes of the row itself.
template <int kChunks>
__global__ void __launch_bounds__(256, kChunks <= 3 ? 4 : 2)
layernorm_kernel(const __half* __restrict__ in, const float* __restrict__ gamma, const float* __restrict__ beta,
                 float eps, int dim, int m_alloc, const int* __restrict__ total_rows, __half* __restrict__ out) {
    __shared__ float4 gb_s[kChunks][4][32];   // [chunk][gamma lo, gamma hi, beta lo, beta hi][lane]
    const int lane = threadIdx.x & 31;
    const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    int rows = total_rows != nullptr ? *total_rows : m_alloc;
    if (rows > m_alloc) rows = m_alloc;
    for (int i = threadIdx.x; i < kChunks * 32; i += blockDim.x) {
        const int c = i >> 5, l = i & 31;
        const int col = (c * 32 + l) * 8;
        float g[8], b[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            g[j] = col < dim ? gamma[col + j] : 0.f;
            b[j] = col < dim ? beta[col + j] : 0.f;
        }
        gb_s[c][0][l] = make_float4(g[0], g[1], g[2], g[3]);
        gb_s[c][1][l] = make_float4(g[4], g[5], g[6], g[7]);
        gb_s[c][2][l] = make_float4(b[0], b[1], b[2], b[3]);
        gb_s[c][3][l] = make_float4(b[4], b[5], b[6], b[7]);
    }
    __syncthreads();
    uint4 raw[kChunks];
    auto fetch = [&](int r, uint4 (&dst)[kChunks]) {
        const __half* x = in + (size_t)r * dim;
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
            const int col = (c * 32 + lane) * 8;
            dst[c] = make_uint4(0, 0, 0, 0);
            if (col < dim) dst[c] = *reinterpret_cast<const uint4*>(x + col);
        }
    };
    int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (r < rows) fetch(r, raw);
    while (r < rows) {
        const int rn = r + warps_per_grid;
        uint4 nxt[kChunks];
        if (rn < rows) fetch(rn, nxt);
        float v[kChunks][8];
#pragma unroll
        for (int c = 0; c < kChunks; ++c) unpack8(raw[c], v[c]);
        float mean, inv;
        row_mean_inv<kChunks>(v, dim, lane, eps, &mean, &inv);
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
            const int col = (c * 32 + lane) * 8;
            if (col < dim) {
                const float4 g0 = gb_s[c][0][lane], g1 = gb_s[c][1][lane], b0 = gb_s[c][2][lane], b1 = gb_s[c][3][lane];
                const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
                const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = (v[c][i] - mean) * inv * g[i] + bb[i];
                *reinterpret_cast<uint4*>(out + (size_t)r * dim + col) = pack8(o);
            }
        }
#pragma unroll
        for (int c = 0; c < kChunks; ++c) raw[c] = nxt[c];
        r = rn;
    }
}

// ------------------------------------------------------------------------------------------
// attention, generic head_dim (<= 64, multiple of 2): one warp per (row, head); lanes split the
// keys, each keeps an online-softmax partial, partials are merged with shuffles.  fp32 throughout.
// Used for head dims the tensor-core kernel does not cover and as its cross-check.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
attn_generic_kernel(const __half* __restrict__ qkv, const int* __restrict__ cu_rows, const int* __restrict__ key_count,
                    const int* __restrict__ row_src, int batch, int tokens, int hidden, int heads, int window,
                    __half* __restrict__ ctx) {
    const int hd = hidden / heads;
    const int lane = threadIdx.x & 31;
    const int b = blockIdx.z;
    const int head = blockIdx.y;
    const int row0 = cu_rows[b];
    const int nrows = cu_rows[b + 1] - row0;
    const int nkeys = key_count[b];
    const int qi = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (qi >= nrows) return;
    const int ld = 3 * hidden;
    const __half* qp = qkv + (size_t)(row0 + qi) * ld + head * hd;
    const float scale = rsqrtf((float)hd);
    float q[64];
#pragma unroll
    for (int d = 0; d < 64; ++d) q[d] = d < hd ? __half2float(qp[d]) * scale : 0.f;
    const int qpos = row_src[row0 + qi] % tokens;
    float m = -INFINITY, l = 0.f;
    float o[64];
#pragma unroll
    for (int d = 0; d < 64; ++d) o[d] = 0.f;
    for (int j = lane; j < nkeys; j += 32) {
        if (window > 0) {
            const int kpos = row_src[row0 + j] % tokens;
            const int dist = qpos > kpos ? qpos - kpos : kpos - qpos;
            if (2 * dist >= window) continue;
        }
        const __half* kp = qkv + (size_t)(row0 + j) * ld + hidden + head * hd;
        const __half* vp = kp + hidden;
        float s = 0.f;
#pragma unroll
        for (int d = 0; d < 64; d += 2) {
            if (d < hd) {
                const float2 kk = __half22float2(*reinterpret_cast<const __half2*>(kp + d));
                s = fmaf(q[d], kk.x, s);
                s = fmaf(q[d + 1], kk.y, s);
            }
        }
        const float mn = fmaxf(m, s);
        const float corr = __expf(m - mn);  // exp(-inf) = 0 on the first key
        const float pr = __expf(s - mn);
        l = l * corr + pr;
#pragma unroll
        for (int d = 0; d < 64; d += 2) {
            if (d < hd) {
                const float2 vv = __half22float2(*reinterpret_cast<const __half2*>(vp + d));
                o[d] = fmaf(pr, vv.x, o[d] * corr);
                o[d + 1] = fmaf(pr, vv.y, o[d + 1] * corr);
            }
        }
        m = mn;
    }
    const float mall = warp_max(m);
    const float f = (m == -INFINITY) ? 0.f : __expf(m - mall);
    const float lall = warp_sum(l * f);
    __half* op = ctx + (size_t)(row0 + qi) * hidden + head * hd;
    const float inv = lall > 0.f ? 1.0f / lall : 0.f;  // no visible key: zeros, as the reference
#pragma unroll
    for (int d = 0; d < 64; ++d) {
        if (d < hd) {
            const float tot = warp_sum(o[d] * f);
            if (lane == 0) op[d] = __float2half_rn(tot * inv);
        }
    }
}

// ------------------------------------------------------------------------------------------
// attention, head_dim 64, tensor cores (mma.sync m16n8k16 f16 -> f32), flash-style:
// one CTA = 64 queries of one (sequence, head); 4 warps x 16 query rows; K/V tiles of 64 keys
// double-buffered in shared memory with cp.async; online softmax in fp32 registers.
// ------------------------------------------------------------------------------------------
constexpr int kAttnLd = 72;  // shared row stride in halfs (64 + 8 pad: conflict-free ldmatrix)

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
    const uint32_t d = smem_u32(smem_dst);
    const int sz = valid ? 16 : 0;  // src-size 0: destination is zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = smem_u32(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
    const uint32_t a = smem_u32(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

__global__ void __launch_bounds__(128)
attn_hd64_kernel(const __half* __restrict__ qkv, const int* __restrict__ cu_rows, const int* __restrict__ key_count,
                 const int* __restrict__ row_src, int tokens, int hidden, int window, __half* __restrict__ ctx) {
    __shared__ __align__(16) __half sq[64 * kAttnLd];
    __shared__ __align__(16) __half sk[2][64 * kAttnLd];
    __shared__ __align__(16) __half sv[2][64 * kAttnLd];

    const int b = blockIdx.z;
    const int head = blockIdx.y;
    const int row0 = cu_rows[b];
    const int nrows = cu_rows[b + 1] - row0;
    const int q0 = blockIdx.x * 64;
    if (q0 >= nrows) return;
    const int nkeys = key_count[b];
    const int ld = 3 * hidden;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;

    const __half* qbase = qkv + (size_t)row0 * ld + head * 64;
    const __half* kbase = qbase + hidden;
    const __half* vbase = kbase + hidden;

    // key-tile range; with a local window only tiles that can intersect the band are visited
    int kt_begin = 0, kt_end = (nkeys + 63) / 64;
    int qpos_lo = 0, qpos_hi = 0;
    if (window > 0) {
        const int qlast = min(q0 + 63, nrows - 1);
        qpos_lo = row_src[row0 + q0] % tokens;
        qpos_hi = row_src[row0 + qlast] % tokens;
        if (qpos_hi < qpos_lo) {  // a trailing query-only CLS row (position 0) is in this block
            qpos_lo = 0;
        }
        // positions are increasing along the packed keys, so tiles far outside the band can be
        // skipped by position of their first / last key
        while (kt_begin < kt_end) {
            const int last = min(kt_begin * 64 + 63, nkeys - 1);
            const int kp = row_src[row0 + last] % tokens;
            if (2 * (qpos_lo - kp) >= window) ++kt_begin; else break;
        }
        while (kt_end > kt_begin) {
            const int kp = row_src[row0 + (kt_end - 1) * 64] % tokens;
            if (2 * (kp - qpos_hi) >= window) --kt_end; else break;
        }
    }

    auto load_tile = [&](const __half* gbase, int first_row, int limit, __half* dst) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = i * 128 + tid;
            const int r = c >> 3, ch = c & 7;
            const bool ok = (first_row + r) < limit;
            const __half* src = gbase + (size_t)(ok ? first_row + r : 0) * ld + ch * 8;
            cp_async16(dst + r * kAttnLd + ch * 8, src, ok);
        }
    };

    load_tile(qbase, q0, nrows, sq);
    if (kt_begin < kt_end) {
        load_tile(kbase, kt_begin * 64, nkeys, sk[0]);
        load_tile(vbase, kt_begin * 64, nkeys, sv[0]);
    }
    cp_async_commit();

    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};
    uint32_t qf[4][4];
    const float sl2 = 0.125f * 1.4426950408889634f;  // 1/sqrt(64) * log2(e)

    int my_pos[2] = {0, 0};
    if (window > 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int qi = q0 + warp * 16 + g + h * 8;
            my_pos[h] = qi < nrows ? row_src[row0 + qi] % tokens : 0;
        }
    }

    for (int kt = kt_begin; kt < kt_end; ++kt) {
        const int buf = (kt - kt_begin) & 1;
        if (kt + 1 < kt_end) {
            load_tile(kbase, (kt + 1) * 64, nkeys, sk[buf ^ 1]);
            load_tile(vbase, (kt + 1) * 64, nkeys, sv[buf ^ 1]);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (kt == kt_begin) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                ldsm_x4(qf[kk], sq + (warp * 16 + (lane & 15)) * kAttnLd + kk * 16 + (lane >> 4) * 8);
        }
        // S = Q K^T
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {
                uint32_t kf[4];
                ldsm_x4(kf, sk[buf] + (jp * 16 + (lane & 7) + ((lane >> 4) << 3)) * kAttnLd + kk * 16 +
                                ((lane >> 3) & 1) * 8);
                mma16816(s[2 * jp], qf[kk], kf[0], kf[1]);
                mma16816(s[2 * jp + 1], qf[kk], kf[2], kf[3]);
            }
        }
        // mask + online softmax (rows g and g+8 of this warp's 16)
        const int key0 = kt * 64;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + j * 8 + t4 * 2 + (e & 1);
                bool vis = key < nkeys;
                if (window > 0 && vis) {
                    const int kp = row_src[row0 + key] % tokens;
                    const int qp = my_pos[e >> 1];
                    const int dist = qp > kp ? qp - kp : kp - qp;
                    vis = 2 * dist < window;
                }
                const float x = vis ? s[j][e] * sl2 : -INFINITY;
                s[j][e] = x;
                mx[e >> 1] = fmaxf(mx[e >> 1], x);
            }
        }
        float corr[2], mnew[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            mnew[h] = fmaxf(m_run[h], mx[h]);
            corr[h] = (mnew[h] == -INFINITY) ? 1.f : exp2f(m_run[h] - mnew[h]);
            m_run[h] = mnew[h];
        }
        float ls[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                const float pz = (mnew[h] == -INFINITY) ? 0.f : exp2f(s[j][e] - mnew[h]);
                s[j][e] = pz;
                ls[h] += pz;
            }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * corr[h] + ls[h];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            o[i][0] *= corr[0];
            o[i][1] *= corr[0];
            o[i][2] *= corr[1];
            o[i][3] *= corr[1];
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t pf[4];
            pf[0] = pack_half2(s[2 * kk][0], s[2 * kk][1]);
            pf[1] = pack_half2(s[2 * kk][2], s[2 * kk][3]);
            pf[2] = pack_half2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pf[3] = pack_half2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < 4; ++dp) {
                uint32_t vf[4];
                ldsm_x4_t(vf, sv[buf] + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kAttnLd + dp * 16 +
                                  (lane >> 4) * 8);
                mma16816(o[2 * dp], pf, vf[0], vf[1]);
                mma16816(o[2 * dp + 1], pf, vf[2], vf[3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int qi = q0 + warp * 16 + g + h * 8;
        if (qi >= nrows) continue;
        const float inv = l_run[h] > 0.f ? 1.0f / l_run[h] : 0.f;
        __half* op = ctx + (size_t)(row0 + qi) * hidden + head * 64 + t4 * 2;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            *reinterpret_cast<__half2*>(op + i * 8) =
                __floats2half2_rn(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
        }
    }
}

// ------------------------------------------------------------------------------------------
// pooling (+ head) + L2
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < (blockDim.x + 31) / 32; ++i) tot += red[i];
    return tot;
}

__global__ void __launch_bounds__(256)
pool_l2_kernel(const __half* __restrict__ hs, const int* __restrict__ cu_rows, const int* __restrict__ key_count,
               const int* __restrict__ cls_row, int dim, int cls_pooling, float* __restrict__ out) {
    __shared__ float red[32];
    const int b = blockIdx.x;
    const int row0 = cu_rows[b];
    const int n = key_count[b];
    float sq = 0.f;
    // each thread owns columns c, c + blockDim, ...; float sum over rows in token order, then
    // * (1/count): the order of runtime/backend/tensor_ops.go:1680-1705
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        float acc = 0.f;
        if (cls_pooling) {
            acc = __half2float(hs[(size_t)cls_row[b] * dim + c]);
        } else if (n > 0) {
            for (int r = 0; r < n; ++r) acc += __half2float(hs[(size_t)(row0 + r) * dim + c]);
            acc *= 1.0f / (float)n;
        }
        out[(size_t)b * dim + c] = acc;
        sq += acc * acc;
    }
    const float tot = block_sum(sq, red);
    const float norm = sqrtf(tot);
    if (norm != 0.f) {
        for (int c = threadIdx.x; c < dim; c += blockDim.x) out[(size_t)b * dim + c] /= norm;
    }
}

// Projection head: out[b,:] = l2norm(pooled[b,:] x W), W [dim, out_dim] in-major, fp32 accumulate in input order
// (PretrainedBERTProjectionHead.Apply, runtime/pretrained_bert_projection_head.go:84-100).  A CTA serves kHeadRows
// batch rows and a thread kHeadCols output columns at a time, so that every weight it reads is used kHeadRows times
// and every 16-byte read of the rows' values in shared memory kHeadCols x 4 times.
constexpr int kHeadRows = 8;
constexpr int kHeadCols = 3;
__global__ void __launch_bounds__(256)
head_l2_kernel(const float* __restrict__ pooled, int batch, int dim, const float* __restrict__ w, int out_dim,
               float* __restrict__ out) {
    extern __shared__ __align__(16) float vec[];  // [kHeadRows][dim]
    __shared__ float red[32];
    const int b0 = blockIdx.x * kHeadRows;
    const int nb = batch - b0 < kHeadRows ? batch - b0 : kHeadRows;
    for (int i = threadIdx.x; i < kHeadRows * dim; i += blockDim.x) {
        const int r = i / dim;
        vec[i] = r < nb ? pooled[(size_t)(b0 + r) * dim + (i - r * dim)] : 0.f;
    }
    __syncthreads();
    float sq[kHeadRows];
#pragma unroll
    for (int r = 0; r < kHeadRows; ++r) sq[r] = 0.f;
    const int dim4 = (dim & 3) == 0 ? dim : 0;   // the 16-byte reads need rows that start on 16 bytes
    for (int j0 = threadIdx.x; j0 < out_dim; j0 += blockDim.x * kHeadCols) {
        float acc[kHeadCols][kHeadRows];
        int jc[kHeadCols];
#pragma unroll
        for (int c = 0; c < kHeadCols; ++c) {
            jc[c] = j0 + c * blockDim.x < out_dim ? j0 + c * blockDim.x : j0;   // a column past the end recomputes j0
#pragma unroll
            for (int r = 0; r < kHeadRows; ++r) acc[c][r] = 0.f;
        }
        int i = 0;
        for (; i + 4 <= dim4; i += 4) {
            float wv[kHeadCols][4];
#pragma unroll
            for (int c = 0; c < kHeadCols; ++c)
#pragma unroll
                for (int u = 0; u < 4; ++u) wv[c][u] = __ldg(w + (size_t)(i + u) * out_dim + jc[c]);
#pragma unroll
            for (int r = 0; r < kHeadRows; ++r) {
                const float4 v = *reinterpret_cast<const float4*>(vec + r * dim + i);
#pragma unroll
                for (int c = 0; c < kHeadCols; ++c) {   // every accumulator takes its terms in input order
                    acc[c][r] = fmaf(v.x, wv[c][0], acc[c][r]);
                    acc[c][r] = fmaf(v.y, wv[c][1], acc[c][r]);
                    acc[c][r] = fmaf(v.z, wv[c][2], acc[c][r]);
                    acc[c][r] = fmaf(v.w, wv[c][3], acc[c][r]);
                }
            }
        }
        for (; i < dim; ++i) {
#pragma unroll
            for (int c = 0; c < kHeadCols; ++c) {
                const float wv = __ldg(w + (size_t)i * out_dim + jc[c]);
#pragma unroll
                for (int r = 0; r < kHeadRows; ++r) acc[c][r] = fmaf(vec[r * dim + i], wv, acc[c][r]);
            }
        }
#pragma unroll
        for (int c = 0; c < kHeadCols; ++c) {
            if (j0 + c * blockDim.x >= out_dim) continue;
#pragma unroll
            for (int r = 0; r < kHeadRows; ++r) {
                if (r < nb) out[(size_t)(b0 + r) * out_dim + jc[c]] = acc[c][r];
                sq[r] += acc[c][r] * acc[c][r];
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kHeadRows; ++r) {
        const float tot = block_sum(sq[r], red);
        __syncthreads();
        if (r < nb && tot != 0.f) {
            const float sc = 1.0f / sqrtf(tot);
            for (int j = threadIdx.x; j < out_dim; j += blockDim.x) out[(size_t)(b0 + r) * out_dim + j] *= sc;
        }
    }
}

// ------------------------------------------------------------------------------------------
// compact encoder profile (models/default_embedding.go:461-505)
// ------------------------------------------------------------------------------------------
// hidden[r,:] = rope(tok[id] + role[rid]) for every packed row: ropeRows,
// runtime/backend/tensor_ops.go:1936-1965, with the position t of the row inside its sequence.
// rope_cs[t * dim/2 + c/2] = (cos, sin) of t / 10000^(c/dim), computed in double on the host.
template <int kChunks>
__global__ void __launch_bounds__(256)
embed_rope_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ roles, const int* __restrict__ row_src,
                  const int* __restrict__ total_rows, int tokens, const __half* __restrict__ tok, int vocab,
                  const __half* __restrict__ role_tab, int role_vocab, const float2* __restrict__ rope_cs, int rope_tokens,
                  int dim, int m_alloc, __half* __restrict__ out, int* status) {
    const int lane = threadIdx.x & 31;
    const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    int rows = *total_rows;
    if (rows > m_alloc) rows = m_alloc;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps_per_grid) {
        const int src = row_src[r];
        const int t = src % tokens;
        const int id = ids[src];
        const int ro = roles != nullptr ? roles[src] : 0;
        int bad = 0;
        if (id < 0 || id >= vocab) bad = kStatusBadTokenId;
        else if (ro < 0 || ro >= role_vocab) bad = kStatusBadTypeId;
        else if (t >= rope_tokens) bad = kStatusBadPosition;
        if (bad) {
            if (lane == 0) atomicCAS(status, 0, bad);
            continue;
        }
        const __half* a = tok + (size_t)id * dim;
        const __half* b = role_tab + (size_t)ro * dim;
        const float2* cs = rope_cs + (size_t)t * (dim / 2);
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
            const int col = (c * 32 + lane) * 8;
            if (col < dim) {
                float fa[8], fb[8], o[8];
                unpack8(*reinterpret_cast<const uint4*>(a + col), fa);
                unpack8(*reinterpret_cast<const uint4*>(b + col), fb);
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    const float x0 = fa[i] + fb[i], x1 = fa[i + 1] + fb[i + 1];
                    const float2 k = cs[(col + i) >> 1];
                    o[i] = x0 * k.x - x1 * k.y;
                    o[i + 1] = x0 * k.y + x1 * k.x;
                }
                *reinterpret_cast<uint4*>(out + (size_t)r * dim + col) = pack8(o);
            }
        }
    }
}

// In place: every packed row divided by its L2 norm (normalizeRows, tensor_ops.go:1367-1391; a zero
// row stays as it is).
template <int kChunks>
__global__ void __launch_bounds__(256)
token_normalize_kernel(__half* __restrict__ x, int dim, int m_alloc, const int* __restrict__ total_rows) {
    const int lane = threadIdx.x & 31;
    const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    int rows = *total_rows;
    if (rows > m_alloc) rows = m_alloc;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps_per_grid) {
        float v[kChunks][8];
        float sq = 0.f;
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
            const int col = (c * 32 + lane) * 8;
            if (col < dim) {
                unpack8(*reinterpret_cast<const uint4*>(x + (size_t)r * dim + col), v[c]);
#pragma unroll
                for (int i = 0; i < 8; ++i) sq = fmaf(v[c][i], v[c][i], sq);
            }
        }
        sq = warp_sum(sq);
        if (sq == 0.f) continue;
        const float inv = 1.0f / sqrtf(sq);
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
            const int col = (c * 32 + lane) * 8;
            if (col < dim) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[c][i] *= inv;
                *reinterpret_cast<uint4*>(x + (size_t)r * dim + col) = pack8(v[c]);
            }
        }
    }
}

// out[b,:] = mean over the valid tokens of sequence b of (normalize ? row / |row| : row); no valid token
// -> zeros (meanPoolMaskedTensor, tensor_ops.go:1644-1709, after the per-token normalize of the graph).
// One CTA per sequence; a thread owns columns c, c + blockDim, ...; rows are visited in token order.
__global__ void __launch_bounds__(256)
compact_pool_kernel(const __half* __restrict__ hs, const int* __restrict__ cu_rows, const int* __restrict__ key_count,
                    int dim, int normalize, float* __restrict__ out) {
    extern __shared__ float inv_norm[];  // [rows of the sequence] when normalising
    const int b = blockIdx.x;
    const int row0 = cu_rows[b];
    const int n = key_count[b];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    if (normalize) {
        for (int r = warp; r < n; r += warps) {
            float sq = 0.f;
            for (int c = lane; c < dim; c += 32) {
                const float v = __half2float(hs[(size_t)(row0 + r) * dim + c]);
                sq = fmaf(v, v, sq);
            }
            sq = warp_sum(sq);
            if (lane == 0) inv_norm[r] = sq == 0.f ? 1.0f : 1.0f / sqrtf(sq);
        }
        __syncthreads();
    }
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        float acc = 0.f;
        for (int r = 0; r < n; ++r) {
            float v = __half2float(hs[(size_t)(row0 + r) * dim + c]);
            if (normalize) v *= inv_norm[r];
            acc += v;
        }
        out[(size_t)b * dim + c] = n > 0 ? acc * (1.0f / (float)n) : 0.f;
    }
}

// ------------------------------------------------------------------------------------------
// compiled pipeline: gather -> matmul -> normalize (per token) -> masked mean_pool, one launch.
// One CTA per sequence; masked tokens are skipped (they are excluded from the mean).  Tokens are
// processed 8 at a time: rows gathered to shared memory, every thread owns output columns.
// ------------------------------------------------------------------------------------------
constexpr int kEpTok = 8;
constexpr int kEpMaxColsPerThread = 4;

// One CTA per (sequence, group of kEpTok valid tokens): gathers the group's table rows, projects them
// (fp32 accumulate in k order), L2-normalises each token's row (unless the pooling comes first) and writes
// the group's sum to partial[b][g][:].  Groups are cut over the VALID tokens, so padding costs nothing.
__global__ void __launch_bounds__(256)
embed_pooled_group_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ mask, int tlen, int groups,
                          const __half* __restrict__ table, int vocab, int dim, const __half* __restrict__ proj,
                          int out_dim, float matmul_scale, int pool_then_l2, float* __restrict__ partial,
                          int* __restrict__ counts, int* status) {
    extern __shared__ float xs[];  // [kEpTok][dim]
    __shared__ float red[32];
    __shared__ int tok_ids[kEpTok];
    __shared__ int n_tok;
    const int b = blockIdx.y, g = blockIdx.x;
    const int32_t* tk = tokens + (size_t)b * tlen;
    const int32_t* mk = mask + (size_t)b * tlen;
    // warp 0 finds the valid tokens number [g * kEpTok, (g + 1) * kEpTok) of the sequence
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        const int first = g * kEpTok;
        int seen = 0, n = 0;
        for (int t0 = 0; t0 < tlen; t0 += 32) {
            const int t = t0 + lane;
            const bool valid = t < tlen && mk[t] != 0;
            const unsigned bal = __ballot_sync(0xffffffffu, valid);
            const int rank = seen + __popc(bal & ((1u << lane) - 1u));
            if (valid && rank >= first && rank < first + kEpTok) tok_ids[rank - first] = tk[t];
            seen += __popc(bal);
        }
        n = seen - first;
        n = n < 0 ? 0 : (n > kEpTok ? kEpTok : n);
        if (lane == 0) {
            n_tok = n;
            if (g == 0) counts[b] = seen;
        }
    }
    __syncthreads();
    const int n = n_tok;
    if (n == 0) return;
    for (int i = 0; i < n; ++i) {
        const int id = tok_ids[i];
        const bool ok = id >= 0 && id < vocab;
        if (!ok && threadIdx.x == 0) atomicCAS(status, 0, kStatusBadTokenId);
        for (int k = threadIdx.x; k < dim; k += blockDim.x)
            xs[i * dim + k] = ok ? __half2float(table[(size_t)id * dim + k]) : 0.f;
    }
    for (int i = n; i < kEpTok; ++i)
        for (int k = threadIdx.x; k < dim; k += blockDim.x) xs[i * dim + k] = 0.f;
    __syncthreads();
    float acc[kEpMaxColsPerThread][kEpTok];
#pragma unroll
    for (int c = 0; c < kEpMaxColsPerThread; ++c)
#pragma unroll
        for (int i = 0; i < kEpTok; ++i) acc[c][i] = 0.f;
#pragma unroll
    for (int c = 0; c < kEpMaxColsPerThread; ++c) {
        const int j = threadIdx.x + c * blockDim.x;
        if (j < out_dim) {
            for (int k = 0; k < dim; ++k) {
                const float w = __half2float(proj[(size_t)k * out_dim + j]);
#pragma unroll
                for (int i = 0; i < kEpTok; ++i) acc[c][i] = fmaf(xs[i * dim + k], w, acc[c][i]);
            }
            // the matmul step's `scale` attribute multiplies the finished products (ApplyMatMulAttributes,
            // runtime/backend/tensor_ops.go:1261-1274)
            if (matmul_scale != 1.0f) {
#pragma unroll
                for (int i = 0; i < kEpTok; ++i) acc[c][i] *= matmul_scale;
            }
        }
    }
    float pooled[kEpMaxColsPerThread];
#pragma unroll
    for (int c = 0; c < kEpMaxColsPerThread; ++c) pooled[c] = 0.f;
    for (int i = 0; i < n; ++i) {
        float inv = 1.0f;
        if (!pool_then_l2) {
            float sq = 0.f;
#pragma unroll
            for (int c = 0; c < kEpMaxColsPerThread; ++c) sq += acc[c][i] * acc[c][i];
            const float norm = sqrtf(block_sum(sq, red));
            inv = norm != 0.f ? 1.0f / norm : 1.0f;
        }
#pragma unroll
        for (int c = 0; c < kEpMaxColsPerThread; ++c) pooled[c] += acc[c][i] * inv;
    }
#pragma unroll
    for (int c = 0; c < kEpMaxColsPerThread; ++c) {
        const int j = threadIdx.x + c * blockDim.x;
        if (j < out_dim) partial[((size_t)b * groups + g) * out_dim + j] = pooled[c];
    }
}

// out[b,:] = (sum of the sequence's group sums, in group order) / valid tokens, then optionally L2.
__global__ void __launch_bounds__(256)
embed_pooled_finish_kernel(const float* __restrict__ partial, const int* __restrict__ counts, int groups, int out_dim,
                           int pool_then_l2, float* __restrict__ out) {
    __shared__ float red[32];
    const int b = blockIdx.x;
    const int count = counts[b];
    const int used = (count + kEpTok - 1) / kEpTok;
    float pooled[kEpMaxColsPerThread];
#pragma unroll
    for (int c = 0; c < kEpMaxColsPerThread; ++c) {
        const int j = threadIdx.x + c * blockDim.x;
        float v = 0.f;
        if (j < out_dim)
            for (int g = 0; g < used; ++g) v += partial[((size_t)b * groups + g) * out_dim + j];
        pooled[c] = count > 0 ? v * (1.0f / (float)count) : 0.f;
    }
    if (pool_then_l2) {
        float sq = 0.f;
#pragma unroll
        for (int c = 0; c < kEpMaxColsPerThread; ++c) sq += pooled[c] * pooled[c];
        const float norm = sqrtf(block_sum(sq, red));
        if (norm != 0.f) {
#pragma unroll
            for (int c = 0; c < kEpMaxColsPerThread; ++c) pooled[c] /= norm;
        }
    }
#pragma unroll
    for (int c = 0; c < kEpMaxColsPerThread; ++c) {
        const int j = threadIdx.x + c * blockDim.x;
        if (j < out_dim) out[(size_t)b * out_dim + j] = pooled[c];
    }
}

template <typename F>
void dispatch_chunks(int dim, F&& f) {
    const int chunks = (dim + 255) / 256;
    if (chunks <= 1) f(std::integral_constant<int, 1>());
    else if (chunks == 2) f(std::integral_constant<int, 2>());
    else if (chunks == 3) f(std::integral_constant<int, 3>());
    else if (chunks == 4) f(std::integral_constant<int, 4>());
    else f(std::integral_constant<int, 8>());
}

// out[r,:] (fp32) = x[r,:] (f16) / ||x[r,:]|| for the packed rows r < *total_rows (a zero row stays zero);
// one warp per row, norm accumulated in fp32.
__global__ void __launch_bounds__(256)
rows_normalize_f32_kernel(const __half* __restrict__ x, int dim, int m_alloc, const int* __restrict__ total_rows,
                          float* __restrict__ out) {
    int rows = *total_rows;
    rows = rows < m_alloc ? rows : m_alloc;
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const __half* xr = x + (size_t)r * dim;
        float sq = 0.f;
        for (int c = lane; c < dim; c += 32) {
            const float v = __half2float(xr[c]);
            sq = fmaf(v, v, sq);
        }
        sq = warp_sum(sq);
        const float inv = sq > 0.f ? rsqrtf(sq) : 0.f;
        float* o = out + (size_t)r * dim;
        for (int c = lane; c < dim; c += 32) o[c] = __half2float(xr[c]) * inv;
    }
}

}  // namespace

void launch_seq_layout(const int32_t* mask, int batch, int tokens, int cls_pooling, int window, const SeqLayout& lay,
                       cudaStream_t stream) {
    seq_count_kernel<<<batch, 256, 0, stream>>>(mask, tokens, cls_pooling, lay.key_count, lay.row_count);
    seq_scan_kernel<<<1, 1024, 0, stream>>>(lay.row_count, batch, 1, lay.cu_rows, lay.total_rows);
    seq_scan_kernel<<<1, 1024, 0, stream>>>(lay.row_count, batch, 128, lay.cu_qtiles, nullptr);
    seq_fill_kernel<<<batch, 256, 0, stream>>>(mask, tokens, cls_pooling, lay.cu_rows, lay.key_count, lay.cu_qtiles,
                                               window, lay.row_src, lay.cls_row, lay.qtile_info_seq, lay.qtile_win_seq);
    qtile_sort_kernel<<<1, 1024, 0, stream>>>(lay.cu_qtiles, batch, lay.qtile_info_seq, lay.qtile_win_seq, lay.qtile_info,
                                              lay.qtile_win);
}

void launch_embed_ln(const int32_t* ids, const int32_t* types, const SeqLayout& lay, int tokens, const __half* tok,
                     int vocab, const __half* pos, int max_pos, const __half* typ, int type_vocab, const float* gamma,
                     const float* beta, float eps, int dim, int m_alloc, __half* out, int* status, int sm_count,
                     cudaStream_t stream) {
    dispatch_chunks(dim, [&](auto c) {
        constexpr int kChunks = decltype(c)::value;
        embed_ln_kernel<kChunks><<<sm_count * 8, 256, 0, stream>>>(ids, types, lay.row_src, lay.total_rows, tokens,
                                                                   tok, vocab, pos, max_pos, typ, type_vocab, gamma,
                                                                   beta, eps, dim, m_alloc, out, status);
    });
}

void launch_layernorm(const __half* in, const float* gamma, const float* beta, float eps, int dim, int m_alloc,
                      const int* total_rows, __half* out, int sm_count, cudaStream_t stream) {
    dispatch_chunks(dim, [&](auto c) {
        constexpr int kChunks = decltype(c)::value;
        // 64 registers at 768 columns: four CTAs per SM, every warp keeps its rows to the end
        layernorm_kernel<kChunks><<<sm_count * (kChunks <= 3 ? 4 : 2), 256, 0, stream>>>(in, gamma, beta, eps, dim, m_alloc,
                                                                                 total_rows, out);
    });
}

void launch_attention(const __half* qkv, const SeqLayout& lay, int batch, int tokens, int hidden, int heads,
                      int window, __half* ctx, cudaStream_t stream) {
    const int hd = hidden / heads;
    const int max_rows = tokens + 1;
    if (hd == 64) {
        dim3 grid((max_rows + 63) / 64, heads, batch);
        attn_hd64_kernel<<<grid, 128, 0, stream>>>(qkv, lay.cu_rows, lay.key_count, lay.row_src, tokens, hidden,
                                                   window, ctx);
    } else {
        dim3 grid((max_rows + 3) / 4, heads, batch);
        attn_generic_kernel<<<grid, 128, 0, stream>>>(qkv, lay.cu_rows, lay.key_count, lay.row_src, batch, tokens,
                                                      hidden, heads, window, ctx);
    }
}

void launch_pool_head(const __half* hidden_states, const SeqLayout& lay, int batch, int dim, int cls_pooling,
                      const float* head_w, int head_out, float* pooled_scratch, float* out, cudaStream_t stream) {
    float* pooled = head_w != nullptr ? pooled_scratch : out;
    pool_l2_kernel<<<batch, 256, 0, stream>>>(hidden_states, lay.cu_rows, lay.key_count, lay.cls_row, dim,
                                              cls_pooling, pooled);
    if (head_w != nullptr)
        head_l2_kernel<<<(batch + kHeadRows - 1) / kHeadRows, 256, (size_t)kHeadRows * dim * sizeof(float), stream>>>(
            pooled, batch, dim, head_w, head_out, out);
}

void launch_embed_rope(const int32_t* ids, const int32_t* roles, const SeqLayout& lay, int tokens, const __half* tok,
                       int vocab, const __half* role_tab, int role_vocab, const float2* rope_cs, int rope_tokens, int dim,
                       int m_alloc, __half* out, int* status, int sm_count, cudaStream_t stream) {
    dispatch_chunks(dim, [&](auto c) {
        constexpr int kChunks = decltype(c)::value;
        embed_rope_kernel<kChunks><<<sm_count * 8, 256, 0, stream>>>(ids, roles, lay.row_src, lay.total_rows, tokens, tok,
                                                                     vocab, role_tab, role_vocab, rope_cs, rope_tokens,
                                                                     dim, m_alloc, out, status);
    });
}

void launch_rows_normalize_f32(const __half* x, const SeqLayout& lay, int dim, int m_alloc, float* out, int sm_count,
                                cudaStream_t stream) {
    rows_normalize_f32_kernel<<<sm_count * 8, 256, 0, stream>>>(x, dim, m_alloc, lay.total_rows, out);
}

void launch_token_normalize(__half* x, const SeqLayout& lay, int dim, int m_alloc, int sm_count, cudaStream_t stream) {
    dispatch_chunks(dim, [&](auto c) {
        constexpr int kChunks = decltype(c)::value;
        token_normalize_kernel<kChunks><<<sm_count * 8, 256, 0, stream>>>(x, dim, m_alloc, lay.total_rows);
    });
}

void launch_compact_pool(const __half* hidden_states, const SeqLayout& lay, int batch, int tokens, int dim, int normalize,
                         float* out, cudaStream_t stream) {
    compact_pool_kernel<<<batch, 256, (size_t)(tokens + 1) * sizeof(float), stream>>>(
        hidden_states, lay.cu_rows, lay.key_count, dim, normalize, out);
}

void launch_embed_pooled(const int32_t* tokens, const int32_t* mask, int batch, int tlen, const __half* table,
                         int vocab, int dim, const __half* projection, int out_dim, float matmul_scale, int pool_then_l2,
                         float* partial, int* counts, float* out, int* status, cudaStream_t stream) {
    const int groups = (tlen + kEpTok - 1) / kEpTok;
    embed_pooled_group_kernel<<<dim3(groups, batch), 256, kEpTok * dim * sizeof(float), stream>>>(
        tokens, mask, tlen, groups, table, vocab, dim, projection, out_dim, matmul_scale, pool_then_l2, partial, counts,
        status);
    embed_pooled_finish_kernel<<<batch, 256, 0, stream>>>(partial, counts, groups, out_dim, pool_then_l2, out);
}

}  // namespace eosb
