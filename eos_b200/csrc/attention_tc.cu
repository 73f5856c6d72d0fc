// Multi-head self-attention, head_dim 64, any sequence length, optional local window, on the 5th-generation
// tensor cores (tcgen05) with S, P and O in tensor memory.
//
// Reference semantics: bertSelfAttentionContextRange, runtime/backend/bert_encoder_layer_ops.go:326-379
// (device twin manta_bert_attention_context, runtime/backends/cuda/native_linux.go:2857-2969):
// per (query, head): logits q.k/sqrt(hd) over unmasked keys, max-subtracted softmax, sum p.v;
// no visible key -> zeros.  Masked rows never exist here (packed layout), so "unmasked keys" are the
// first key_count rows of the sequence.  With a local window key j is visible to query i only if
// 2 |pos_i - pos_j| < window (positions are the tokens' original positions).
//
// One CTA per SM holds two independent pipelines ("streams"), each with 256 columns of tensor memory (S 128, O 64,
// P 64), its own
// shared-memory rings and its own warps, walking work items (sequence, 128-query tile, head); while one stream's
// softmax threads work the other stream's MMAs run, so neither pipe waits for the other.  Per stream:
//   4 warps      softmax, one thread per query row (thread = TMEM lane, so a row's maximum needs no exchange
//                between threads; the whole row of a tile is held in registers, which the other warps make room
//                for with setmaxnreg): per key tile read the row of S (fp32) and release S at once, update the row
//                maximum, write P = exp2(s - m) as packed f16 into P's own columns and add the row sum of exactly
//                those f16 values; after the item's last key tile O / l -> f16 -> global (one 128-byte row segment
//                per thread).  The running maximum only moves when a tile's maximum exceeds it by more than
//                kRescaleThreshold (then O and l are rescaled in place); otherwise the stale maximum is kept, which
//                cancels in O / l.  Three exponentials of four run on the MUFU unit (ex2.approx.f16x2), the fourth
//                on the FMA pipe.
//   1 warp       TMA producer: Q tile (ring of 2), then K_j and V_j tiles (128 rows x 64, 128B swizzle) into a ring
//                of 2 each.
//   1 warp       MMA issuer: S = Q K_j^T (M128 x N<=128 x K64) and O += P V_j (N = 64) with P read from tensor memory
//                as the A operand.  S(j+1) is issued as soon as the softmax threads hold S(j) in registers, ahead of
//                P V(j), which has to wait for the probabilities: the softmax of tile j + 1 never waits for a
//                tensor-pipe round trip.
// The last key tile of a sequence only pays for its visible keys: N of the first MMA, the K extent of the second
// and the softmax's column chunks are cut to the keys that exist (rounded to 16 / 32).
// All mbarrier waits are bounded (abort flag + status word); there are no named barriers, so a role that gives
// up never leaves another one waiting.
#include "attention_tc.cuh"

#include "common.cuh"
#include "tma_util.cuh"

namespace eosb {

#ifdef EOSB_ATTN_TIMING
// Cycle counts per role phase of CTA 0 (debug builds only): [0..7] softmax thread 0, [8..15] MMA thread,
// [16..19] producer thread.
__device__ long long g_attn_timing[24];
#define TDECL long long tlast__ = clock64(); long long tacc__[8] = {0, 0, 0, 0, 0, 0, 0, 0}
#define TMARK(i) do { long long now__ = clock64(); tacc__[i] += now__ - tlast__; tlast__ = now__; } while (0)
#define TFLUSH(base, cond) do { if (blockIdx.x == 0 && (cond)) for (int i__ = 0; i__ < 8; ++i__) if ((base) + i__ < 24) atomicAdd((unsigned long long*)&g_attn_timing[(base) + i__], (unsigned long long)tacc__[i__]); } while (0)
#else
#define TDECL do { } while (0)
#define TMARK(i) do { } while (0)
#define TFLUSH(base, cond) do { } while (0)
#endif

namespace {

constexpr int kStreams = 2;                    // independent pipelines per CTA, each with its own roles, rings and TMEM half
constexpr int kSoftmaxWarps = 4;               // per stream: warps 4s .. 4s+3 (one warpgroup)
constexpr int kFirstOtherWarp = kStreams * kSoftmaxWarps;   // then per stream: producer warp, MMA warp
constexpr int kAtThreads = (kStreams * kSoftmaxWarps + 2 * kStreams) * 32;   // 384
constexpr int kRegsSoftmax = 224, kRegsOther = 56;  // 8 x 224 + 4 x 56 = 12 x 168: the launch's allocation, redistributed
constexpr int kQStages = 2;
constexpr int kKStages = 2;    // the K and the V tiles ride separate rings: the first MMA of tile j + 1 is issued
constexpr int kVStages = 2;    // before the second MMA of tile j, so the two are consumed out of step
constexpr uint32_t kTileBytes = 128 * 64 * 2;   // 16 KB: Q, K_j or V_j
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffK = kOffQ + kQStages * kTileBytes;
constexpr uint32_t kOffV = kOffK + kKStages * kTileBytes;
constexpr uint32_t kOffBars = kOffV + kVStages * kTileBytes;
constexpr uint32_t kNumBars = 2 * kQStages + 2 * kKStages + 2 * kVStages + 5;
constexpr uint32_t kStreamBytes = (kOffBars + kNumBars * 8 + 1023u) & ~1023u;   // shared memory of one stream
constexpr uint32_t kOffMisc = kStreams * kStreamBytes;
constexpr uint32_t kAtSmemBytes = kOffMisc + 16 + 1024;
constexpr uint32_t kTmemCols = 256;   // per stream
constexpr uint32_t kColS = 0;         // S: 128 fp32 columns
constexpr uint32_t kColO = 128;       // O: 64 fp32 columns
constexpr uint32_t kColP = 192;       // P: 128 probabilities as packed f16 pairs in 64 columns
constexpr float kRescaleThreshold = 1.0f;  // in log2 units: probabilities stay below 2

struct Item {
    int row0;        // first packed row of the sequence
    int nrows;       // query rows of the sequence
    int nkeys;       // key rows of the sequence
    int q0;          // first query of this tile (relative to row0)
    int head;
    int kt_begin, kt_end;      // key tiles (of 128) to visit
    int full_begin, full_end;  // key tiles whose keys are all inside the window of all the tile's queries
};

// Walks the items of this CTA (item w = first + i * stride; w = q-tile * heads + head) with the next item's
// descriptors requested one item ahead, so that stepping never waits for global memory.
struct ItemWalker {
    int w, stride, total, heads;
    const int4* info;
    const int4* win;
    int4 pre_i, pre_w;
    Item it;
    __device__ __forceinline__ void fetch(int ww) {
        if (ww < total) {
            const int qi = ww / heads;
            pre_i = __ldg(info + qi);
            pre_w = __ldg(win + qi);
        }
    }
    __device__ __forceinline__ void decode() {
        it.row0 = pre_i.x;
        it.nrows = pre_i.y;
        it.nkeys = pre_i.z;
        it.q0 = pre_i.w;
        it.head = w % heads;
        it.kt_begin = pre_w.x;
        it.kt_end = pre_w.y;
        it.full_begin = pre_w.z;
        it.full_end = pre_w.w;
    }
    __device__ __forceinline__ void init(int first, int str, int tot, int h, const int4* p, const int4* pw) {
        w = first; stride = str; total = tot; heads = h; info = p; win = pw;
        pre_i = make_int4(0, 0, 0, 0);
        pre_w = make_int4(0, 0, 0, 0);
        fetch(w);
        if (w < total) {
            decode();
            fetch(w + stride);
        }
    }
    __device__ __forceinline__ bool valid() const { return w < total; }
    __device__ __forceinline__ void next() {
        w += stride;
        if (w < total) {
            decode();
            fetch(w + stride);
        }
    }
};

__device__ __forceinline__ int visible_in_tile(const Item& it, int kt) {
    const int v = it.nkeys - kt * 128;
    return v > 128 ? 128 : v;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// (a0, a1) * b + c on the packed fp32 pipe.
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b, float c) {
    uint64_t a, bb, cc, d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %1};" : "=l"(bb) : "f"(b));
    asm("mov.b64 %0, {%1, %1};" : "=l"(cc) : "f"(c));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(bb), "l"(cc));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(d));
}
// 2^x0, 2^x1 as packed f16 (x rounded to f16 first; -inf gives 0).
__device__ __forceinline__ uint32_t ex2_f16x2(float x0, float x1) {
    __half2 h = __floats2half2_rn(x0, x1);
    uint32_t hx = *reinterpret_cast<uint32_t*>(&h), px;
    asm("ex2.approx.f16x2 %0, %1;" : "=r"(px) : "r"(hx));
    return px;
}

// The same on the FMA pipe (the MUFU unit serves one ex2.approx.f16x2 per 16 cycles and scheduler, which two softmax
// warps per scheduler saturate): x = n + f with n the nearest integer (magic-number rounding), 2^f by a cubic on
// [-0.5, 0.5] (relative error 7.7e-5, a third of an f16 half-ulp), n added to the exponent field.  x <= 1 here; values
// below -125 (masked scores are -inf) give a number that rounds to 0 in f16.
#ifndef EOSB_ATTN_POLY_EVERY
#define EOSB_ATTN_POLY_EVERY 4   // every n-th pair of a row takes this path (0 = none); measured per step at 12 layers,
                                 // 1024 x 64..512 tokens: none 15.5 ms, every 4th 14.75, every 3rd 14.8, every 2nd 15.9
#endif
__device__ __forceinline__ uint32_t ex2_poly_f16x2(float x0, float x1) {
    const float magic = 12582912.0f;   // 1.5 * 2^23
    x0 = fmaxf(x0, -125.0f);
    x1 = fmaxf(x1, -125.0f);
    const float t0 = x0 + magic, t1 = x1 + magic;
    const float f0 = x0 - (t0 - magic), f1 = x1 - (t1 - magic);
    float p0 = fmaf(0.05508868f, f0, 0.24260405f), p1 = fmaf(0.05508868f, f1, 0.24260405f);
    p0 = fmaf(p0, f0, 0.69327624f);
    p1 = fmaf(p1, f1, 0.69327624f);
    p0 = fmaf(p0, f0, 0.99992894f);
    p1 = fmaf(p1, f1, 0.99992894f);
    const uint32_t r0 = __float_as_uint(p0) + (__float_as_uint(t0) << 23);
    const uint32_t r1 = __float_as_uint(p1) + (__float_as_uint(t1) << 23);
    __half2 h = __floats2half2_rn(__uint_as_float(r0), __uint_as_float(r1));
    return *reinterpret_cast<uint32_t*>(&h);
}

__global__ void __launch_bounds__(kAtThreads, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tm_qkv, const int* __restrict__ cu_qtiles,
               const int4* __restrict__ qtile_info, const int4* __restrict__ qtile_win,
               const int* __restrict__ row_src, int batch, int tokens, int hidden, int heads, int window,
               __half* __restrict__ ctx, int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base_cta = (raw + 1023u) & ~1023u;
    uint8_t* sm_cta = smem_raw + (base_cta - raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the CTA is kStreams independent pipelines: stream s = softmax warps 4s .. 4s+3, producer warp, MMA warp, its own
    // slice of shared memory (rings, barriers) and its own kTmemCols columns of tensor memory; it walks the items
    // of virtual CTA blockIdx.x * kStreams + s
    const int stream = warp < kFirstOtherWarp ? warp >> 2 : (warp - kFirstOtherWarp) >> 1;
    const bool is_producer = warp >= kFirstOtherWarp && ((warp - kFirstOtherWarp) & 1) == 0;
    const bool is_mma = warp >= kFirstOtherWarp && ((warp - kFirstOtherWarp) & 1) == 1;
    const int quarter = warp & 3;                     // softmax warps: the TMEM lane quarter they may access
    const uint32_t base = base_cta + stream * kStreamBytes;
    const int vcta = blockIdx.x * kStreams + stream, vgrid = gridDim.x * kStreams;

    const uint32_t bar0 = base + kOffBars;
    auto q_full = [&](int s) { return bar0 + 8u * s; };
    auto q_empty = [&](int s) { return bar0 + 8u * (kQStages + s); };
    auto k_full = [&](int s) { return bar0 + 8u * (2 * kQStages + s); };
    auto k_empty = [&](int s) { return bar0 + 8u * (2 * kQStages + kKStages + s); };
    auto v_full = [&](int s) { return bar0 + 8u * (2 * kQStages + 2 * kKStages + s); };
    auto v_empty = [&](int s) { return bar0 + 8u * (2 * kQStages + 2 * kKStages + kVStages + s); };
    const uint32_t s_full = bar0 + 8u * (2 * kQStages + 2 * kKStages + 2 * kVStages);  // S of a key tile is in tensor memory
    const uint32_t s_free = s_full + 8u;    // its rows are in the softmax threads' registers (4 warps arrive): S may be overwritten
    const uint32_t p_full = s_full + 16u;   // its probabilities are in tensor memory (4 warps arrive)
    const uint32_t pv_done = s_full + 24u;  // its P V product is complete: P may be overwritten, O touched
    const uint32_t o_full = s_full + 32u;   // the item's O is complete

    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm_cta + kOffMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm_cta + kOffMisc + 4);

    const int total_items = cu_qtiles[batch] * heads;

    if (threadIdx.x == 0) *abort_flag = 0;
    if (is_producer && lane == 0) {   // each stream's producer sets up the stream's barriers
        for (int s = 0; s < kQStages; ++s) {
            mbar_init(q_full(s), 1);
            mbar_init(q_empty(s), 1);
        }
        for (int s = 0; s < kKStages; ++s) {
            mbar_init(k_full(s), 1);
            mbar_init(k_empty(s), 1);
        }
        for (int s = 0; s < kVStages; ++s) {
            mbar_init(v_full(s), 1);
            mbar_init(v_empty(s), 1);
        }
        mbar_init(s_full, 1);
        mbar_init(s_free, kSoftmaxWarps);
        mbar_init(p_full, kSoftmaxWarps);
        mbar_init(pv_done, 1);
        mbar_init(o_full, 1);
        mbar_fence_init();
        tma_prefetch_desc(&tm_qkv);
    }
    if (warp == kFirstOtherWarp + 1) {   // one warp allocates (and frees) the whole CTA's tensor memory
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kStreams * kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot + stream * kTmemCols;

    if (is_producer) {
        // ------------------------------------------------------------ TMA producer
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
        if (lane == 0) {
            ItemWalker wk;
            wk.init(vcta, vgrid, total_items, heads, qtile_info, qtile_win);
            uint32_t qn = 0, kc = 0, vc = 0;
            bool ok = true;
            TDECL;
            for (; ok && wk.valid(); wk.next()) {
                const Item& it = wk.it;
                if (it.kt_end <= it.kt_begin) continue;
                const int qs = qn % kQStages;
                TMARK(0);
                if (!mbar_wait(q_empty(qs), ((qn / kQStages) & 1u) ^ 1u, abort_flag)) break;
                TMARK(1);
                mbar_arrive_expect_tx(q_full(qs), kTileBytes);
                tma_load_2d(base + kOffQ + qs * kTileBytes, &tm_qkv, it.head * 64, it.row0 + it.q0, q_full(qs));
                ++qn;
                for (int kt = it.kt_begin; ok && kt < it.kt_end; ++kt) {
                    {
                        const int s = kc % kKStages;
                        TMARK(0);
                        if (!mbar_wait(k_empty(s), ((kc / kKStages) & 1u) ^ 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                        TMARK(2);
                        mbar_arrive_expect_tx(k_full(s), kTileBytes);
                        tma_load_2d(base + kOffK + s * kTileBytes, &tm_qkv, hidden + it.head * 64, it.row0 + kt * 128,
                                    k_full(s));
                        ++kc;
                    }
                    {
                        const int s = vc % kVStages;
                        TMARK(0);
                        if (!mbar_wait(v_empty(s), ((vc / kVStages) & 1u) ^ 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                        TMARK(2);
                        mbar_arrive_expect_tx(v_full(s), kTileBytes);
                        tma_load_2d(base + kOffV + s * kTileBytes, &tm_qkv, 2 * hidden + it.head * 64,
                                    it.row0 + kt * 128, v_full(s));
                        ++vc;
                    }
                }
            }
            TFLUSH(16, stream == 0);
        }
        __syncwarp();
    } else if (is_mma) {
        // ------------------------------------------------------------ MMA issuer
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
        if (lane == 0) {
            // O += P V: P (f16) from tensor memory as the A operand, V (MN-major, as TMA delivered it) as B, N = 64
            constexpr uint32_t idesc_o = umma_idesc_f16(128, 64) | (1u << 16);
            // Two cursors over the same sequence of key tiles: the first MMA (S = Q K^T) of tile n + 1 is issued as
            // soon as the softmax threads hold S(n) in registers, i.e. before the second MMA (O += P V) of tile n,
            // which has to wait for the probabilities; the softmax of tile n + 1 then starts without waiting for a
            // tensor-pipe round trip.
            ItemWalker wq, wp;
            wq.init(vcta, vgrid, total_items, heads, qtile_info, qtile_win);
            wp.init(vcta, vgrid, total_items, heads, qtile_info, qtile_win);
            while (wq.valid() && wq.it.kt_end <= wq.it.kt_begin) wq.next();
            while (wp.valid() && wp.it.kt_end <= wp.it.kt_begin) wp.next();
            int kt_q = wq.valid() ? wq.it.kt_begin : 0, kt_p = wp.valid() ? wp.it.kt_begin : 0;
            uint32_t qn_q = 0, qn_p = 0, kc = 0, vc = 0, nqk = 0, npv = 0;
            bool ok = true;
            TDECL;
            const uint32_t tmem_s = tmem_base + kColS, tmem_o = tmem_base + kColO, tmem_p = tmem_base + kColP;
            auto issue_qk = [&]() -> bool {
                const Item& it = wq.it;
                const int qs = qn_q % kQStages;
                if (kt_q == it.kt_begin) {
                    TMARK(0);
                    if (!mbar_wait(q_full(qs), (qn_q / kQStages) & 1u, abort_flag)) return false;
                    TMARK(3);
                }
                if (nqk > 0) {   // S still holds the previous tile until its rows are in registers
                    TMARK(0);
                    if (!mbar_wait(s_free, (nqk - 1) & 1u, abort_flag)) return false;
                    TMARK(7);
                }
                const int s = kc % kKStages;
                TMARK(0);
                if (!mbar_wait(k_full(s), (kc / kKStages) & 1u, abort_flag)) return false;
                TMARK(1);
                ++kc;
                tc_fence_after();
                const int n16 = (visible_in_tile(it, kt_q) + 15) & ~15;
                const uint32_t idesc_s = umma_idesc_f16(128, n16);
                const uint32_t q_lo = umma_desc_sw128_lo(base + kOffQ + qs * kTileBytes);
                const uint32_t k_lo = umma_desc_sw128_lo(base + kOffK + s * kTileBytes);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)  // 32 bytes along K per step = 2 in descriptor units
                    umma_f16_split(tmem_s, q_lo + kk * 2, kDescSw128Hi, k_lo + kk * 2, kDescSw128Hi, idesc_s,
                                   kk > 0 ? 1u : 0u);
                umma_commit(k_empty(s));
                umma_commit(s_full);
                TMARK(2);
                ++nqk;
                if (++kt_q >= it.kt_end) {
                    ++qn_q;
                    do wq.next(); while (wq.valid() && wq.it.kt_end <= wq.it.kt_begin);
                    if (wq.valid()) kt_q = wq.it.kt_begin;
                }
                return true;
            };
            if (wq.valid()) ok = issue_qk();
            while (ok && wp.valid()) {
                if (wq.valid()) {
                    ok = issue_qk();
                    if (!ok) break;
                }
                const Item& it = wp.it;
                TMARK(0);
                if (!mbar_wait(p_full, npv & 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                TMARK(4);
                const int s = vc % kVStages;
                if (!mbar_wait(v_full(s), (vc / kVStages) & 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                TMARK(5);
                ++vc;
                tc_fence_after();
                const int ksteps = (visible_in_tile(it, kt_p) + 15) >> 4;
                const uint32_t v_addr = base + kOffV + s * kTileBytes;
                // MN-major V: the start address moves by one 16-key slab (2048 bytes = 128 units) per step
                const uint32_t v_lo = (v_addr >> 4) & 0x3fffu;
                for (int kk = 0; kk < ksteps; ++kk)
                    umma_f16_tmem_a(tmem_o, tmem_p + kk * 8, v_lo + kk * 128u, kDescSw128Hi, idesc_o,
                                    (kt_p > it.kt_begin || kk > 0) ? 1u : 0u);
                umma_commit(v_empty(s));
                umma_commit(pv_done);
                TMARK(6);
                ++npv;
                if (++kt_p >= it.kt_end) {
                    umma_commit(q_empty(qn_p % kQStages));
                    umma_commit(o_full);
                    ++qn_p;
                    do wp.next(); while (wp.valid() && wp.it.kt_end <= wp.it.kt_begin);
                    if (wp.valid()) kt_p = wp.it.kt_begin;
                }
            }
            TFLUSH(8, stream == 0);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ softmax + epilogue (warps 0-3)
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
        const int r = quarter * 32 + lane;                      // query row inside the tile = TMEM lane
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const uint32_t t_s = tmem_base + lane_addr + kColS;
        const uint32_t t_o = tmem_base + lane_addr + kColO;
        const uint32_t t_p = tmem_base + lane_addr + kColP;
        const float sl2 = 0.125f * 1.4426950408889634f;        // 1/sqrt(64) * log2(e)
        ItemWalker wk;
        wk.init(vcta, vgrid, total_items, heads, qtile_info, qtile_win);
        uint32_t sn = 0, on = 0;
        bool ok = true;
        TDECL;
        for (; ok && wk.valid(); wk.next()) {
            const Item& it = wk.it;
            const int qrow = it.q0 + r;
            const bool row_valid = qrow < it.nrows;
            __half* out = ctx + (size_t)(it.row0 + qrow) * hidden + it.head * 64;
            if (it.kt_end <= it.kt_begin) {   // no visible key at all: zeros
                if (row_valid) {
                    const uint32_t z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
                    for (int q = 0; q < 4; ++q) st_global_v8(out + q * 16, z);
                }
                continue;
            }
            // a warp whose 32 query rows are all padding of the sequence's last query tile keeps the barrier
            // protocol but computes nothing (its P and O rows are never used)
            const bool live = it.q0 + quarter * 32 < it.nrows;
            // positions enter only as differences inside one sequence, so the flat index b * tokens + t serves
            const int qpos = (window > 0 && row_valid) ? __ldg(row_src + it.row0 + qrow) : 0;
            float m_used = -INFINITY;   // the maximum the probabilities of this row are currently scaled by
            float l_run = 0.f;          // the row sum of the f16 probabilities written so far, in that scaling
            for (int kt = it.kt_begin; kt < it.kt_end; ++kt, ++sn) {
                TMARK(0);
                ok = __all_sync(0xffffffffu, mbar_wait(s_full, sn & 1u, abort_flag));
                if (!ok) break;
                TMARK(1);
                tc_fence_after();
                const int nvis = visible_in_tile(it, kt);
                const int nch = (nvis + 31) >> 5;          // 32-column chunks that hold visible keys
                const bool masked = nvis < nch * 32;
                const bool edge = kt < it.full_begin || kt >= it.full_end;   // window mask needed
                // the row's scores of this tile, all in registers (one wait for up to four loads)
                uint32_t v[4][32];
                if (live) {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (c < nch) tmem_ld_32x32(t_s + c * 32, v[c]);
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (c < nch) tmem_ld_wait32(v[c]);
                }
                // the row is in registers: the first MMA of the next tile may overwrite S
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(s_free);
                if (live) {
                    if (masked) {
                        // the sequence's last, partial tile: scores of keys that do not exist become -inf
                        // (probability 0); only the last chunk can hold any
                        const int c_last = nch - 1;
                        const int lim = nvis - c_last * 32;
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            if (c == c_last) {
#pragma unroll
                                for (int e = 0; e < 32; ++e)
                                    if (e >= lim) v[c][e] = 0xff800000u;
                            }
                    }
                    if (edge) {
                        // a tile that straddles the window's edge: keys outside this row's window become -inf
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            if (c < nch) {
#pragma unroll
                                for (int e = 0; e < 32; ++e) {
                                    const int col = c * 32 + e;
                                    if (col < nvis) {
                                        const int d = qpos - __ldg(row_src + it.row0 + kt * 128 + col);
                                        if (2 * (d < 0 ? -d : d) >= window) v[c][e] = 0xff800000u;
                                    }
                                }
                            }
                    }
                    TMARK(2);
                    float mx = -INFINITY;
                    {
                        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            if (c < nch) {
#pragma unroll
                                for (int e = 0; e < 32; e += 8) {
                                    m0 = max3(m0, __uint_as_float(v[c][e]), __uint_as_float(v[c][e + 1]));
                                    m1 = max3(m1, __uint_as_float(v[c][e + 2]), __uint_as_float(v[c][e + 3]));
                                    m2 = max3(m2, __uint_as_float(v[c][e + 4]), __uint_as_float(v[c][e + 5]));
                                    m3 = max3(m3, __uint_as_float(v[c][e + 6]), __uint_as_float(v[c][e + 7]));
                                }
                            }
                        mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
                    }
                    const float mxs = mx * sl2;
                    // P and O belong to the second MMA of the previous tile until it is complete
                    if (sn > 0 && !mbar_wait(pv_done, (sn - 1) & 1u, abort_flag)) ok = false;
                    tc_fence_after();
                    if (kt == it.kt_begin) {
                        m_used = mxs;
                    } else {
                        const bool need = mxs > m_used + kRescaleThreshold;
                        if (__any_sync(0xffffffffu, need)) {
                            // O and the row sum of the rows whose maximum moved are rescaled in place
                            float f = 1.0f;
                            if (need && m_used != -INFINITY) asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(f) : "f"(m_used - mxs));
                            uint32_t o[16];
#pragma unroll
                            for (int h = 0; h < 4; ++h) {
                                tmem_ld_32x16(t_o + h * 16, o);
                                tmem_ld_wait16(o);
#pragma unroll
                                for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
                                tmem_st_32x16(t_o + h * 16, o);
                            }
                            l_run *= f;
                            if (need) m_used = mxs;
                        }
                    }
                    TMARK(3);
                    const float neg_m = m_used == -INFINITY ? 0.0f : -m_used;
                    // probabilities as packed f16 pairs into the P columns; the row sum adds exactly the values that
                    // multiply V (two pairs are added in f16 first: sums below 4, then in fp32)
                    float l0 = 0.f, l1 = 0.f;
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (c < nch) {
                            uint32_t p[16];
#pragma unroll
                            for (int e = 0; e < 32; e += 2) {
                                float x0, x1;
                                ffma2(x0, x1, __uint_as_float(v[c][e]), __uint_as_float(v[c][e + 1]), sl2, neg_m);
                                if (EOSB_ATTN_POLY_EVERY > 0 && ((e >> 1) % (EOSB_ATTN_POLY_EVERY > 0 ? EOSB_ATTN_POLY_EVERY : 1)) ==
                                                                    (EOSB_ATTN_POLY_EVERY > 0 ? EOSB_ATTN_POLY_EVERY : 1) - 1)
                                    p[e >> 1] = ex2_poly_f16x2(x0, x1);
                                else
                                    p[e >> 1] = ex2_f16x2(x0, x1);
                            }
#pragma unroll
                            for (int e = 0; e < 16; e += 2) {
                                const __half2 hs = __hadd2(*reinterpret_cast<const __half2*>(&p[e]),
                                                           *reinterpret_cast<const __half2*>(&p[e + 1]));
                                const float2 fs = __half22float2(hs);
                                l0 += fs.x;
                                l1 += fs.y;
                            }
                            tmem_st_32x16(t_p + c * 16, p);
                        }
                    l_run += l0 + l1;
                    TMARK(4);
                    tmem_st_wait();
                } else if (sn > 0) {
                    if (!mbar_wait(pv_done, (sn - 1) & 1u, abort_flag)) ok = false;
                }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full);
                TMARK(5);
            }
            if (!ok) break;
            TMARK(0);
            ok = __all_sync(0xffffffffu, mbar_wait(o_full, on & 1u, abort_flag));
            if (!ok) break;
            TMARK(6);
            ++on;
            tc_fence_after();
            if (live) {
                uint32_t oa[32], ob[32];
                tmem_ld_32x32(t_o, oa);
                tmem_ld_32x32(t_o + 32, ob);
                tmem_ld_wait32(oa);
                tmem_ld_wait32(ob);
                tc_fence_before();
                const float l = l_run;
                const float inv = l > 0.f ? __frcp_rn(l) : 0.f;
                if (row_valid) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {  // 32 bytes (one sector) per store
                        uint32_t ow[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const int i0 = (q & 1) * 16 + 2 * e;
                            __half2 hh = q < 2 ? __floats2half2_rn(__uint_as_float(oa[i0]) * inv, __uint_as_float(oa[i0 + 1]) * inv)
                                               : __floats2half2_rn(__uint_as_float(ob[i0]) * inv, __uint_as_float(ob[i0 + 1]) * inv);
                            ow[e] = *reinterpret_cast<uint32_t*>(&hh);
                        }
                        st_global_v8(out + q * 16, ow);
                    }
                }
            }
            TMARK(7);
        }
        TFLUSH(0, threadIdx.x == 0);   // stream 0's first softmax thread
    }

    tc_fence_before();
    __syncthreads();
    if (warp == kFirstOtherWarp + 1) {
        tc_fence_after();
        tmem_dealloc(*tmem_slot, kStreams * kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_flag != 0 && status != nullptr) atomicExch(status, kStatusPipelineTimeout);
}

}  // namespace

#ifdef EOSB_ATTN_TIMING
extern "C" __attribute__((visibility("default"))) int eos_b200_debug_attn_timing(long long* out24, int reset) {
    long long zero[24] = {0};
    if (cudaMemcpyFromSymbol(out24, g_attn_timing, sizeof(zero)) != cudaSuccess) return 1;
    if (reset && cudaMemcpyToSymbol(g_attn_timing, zero, sizeof(zero)) != cudaSuccess) return 1;
    return 0;
}
#endif

std::string attn_tc_global_init() {
    cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAtSmemBytes);
    if (e != cudaSuccess) return std::string("cudaFuncSetAttribute(attn_tc_kernel): ") + cudaGetErrorString(e);
    return "";
}

std::string attn_tc_make_plan(AttnTcPlan* plan, const __half* qkv, int m_alloc, int hidden) {
    return encode_2d(&plan->tm_qkv, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, qkv, (uint64_t)3 * hidden, (uint64_t)m_alloc,
                     (uint64_t)3 * hidden * 2, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B);
}

void attn_tc_launch(const AttnTcPlan& plan, const SeqLayout& lay, int batch, int tokens, int hidden, int heads,
                    int window, __half* ctx, int* status, int sm_count, cudaStream_t stream) {
    attn_tc_kernel<<<sm_count, kAtThreads, kAtSmemBytes, stream>>>(plan.tm_qkv, lay.cu_qtiles, lay.qtile_info,
                                                                        lay.qtile_win, lay.row_src, batch, tokens,
                                                                        hidden, heads, window, ctx, status);
}

}  // namespace eosb
