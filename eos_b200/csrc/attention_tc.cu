// Multi-head self-attention, head_dim 64, sequences of up to 512 keys, on the 5th-generation
// tensor cores (tcgen05) with S and O in tensor memory.
//
// Reference semantics: bertSelfAttentionContextRange, runtime/backend/bert_encoder_layer_ops.go:326-379
// (device twin manta_bert_attention_context, runtime/backends/cuda/native_linux.go:2857-2969):
// per (query, head): logits q.k/sqrt(hd) over unmasked keys, max-subtracted softmax, sum p.v;
// no visible key -> zeros.  Masked rows never exist here (packed layout), so "unmasked keys" are the
// first key_count rows of the sequence.
//
// One persistent CTA per SM walks work items (sequence, 128-query tile, head):
//   warp 0       TMA producer: Q tile, then K tiles and V tiles (128 rows x 64, 128B swizzle) into rings.
//   warp 1       MMA issuer: S_j = Q K_j^T per key tile j (fp32, 128 TMEM columns each), then
//                O += P_j V_j (V as an MN-major operand, straight from the row-major tile TMA
//                delivered), O reusing the first 80 of S's columns.  Work is cut into sub-items of one key
//                tile = a quarter of tensor memory; the S phase runs two sub-items ahead of the P V phase,
//                so four sub-items are in flight per SM (S ready, in softmax, P V running, being retired).
//                The row sums l = P 1 come out of the same MMA: its B operand is [V | ones] (N = 80), so
//                they are the fp32 sums of exactly the f16 probabilities that multiply V.
//   warps 4-19   softmax (thread = query row, four warps per row split the columns of every tile): pass A
//                reads all S tiles for the row maximum (exchanged through shared memory), pass B re-reads
//                them, writes P = exp2(s - m) (packed f16 ex2) into the 128B-swizzled K-major layout the
//                second MMA consumes; finally O / l -> f16 -> global, 32 bytes (one sector) per thread.
//                Warps whose 32 query rows are padding of a sequence's last query tile only keep the
//                barrier protocol.
// All scores of a sub-item are resident in TMEM before any probability is formed, so O is never
// rescaled in place; a sequence longer than 128 keys is several sub-items whose partial (O, m, l) are
// merged in registers when they are retired.  All mbarrier waits are bounded (abort flag + status word).
#include "attention_tc.cuh"

#include "common.cuh"
#include "tma_util.cuh"

namespace eosb {

#ifdef EOSB_ATTN_TIMING
__device__ long long g_attn_timing[16];
__device__ long long g_attn_trace[3][2048];
#define TMARK(i) do { long long now__ = clock64(); tacc__[i] += now__ - tlast__; tlast__ = now__; if (blockIdx.x == 0 && threadIdx.x == 128 && tcnt__ < 2048) g_attn_trace[0][tcnt__++] = (now__ << 8) | (i); } while (0)
#else
#define TMARK(i) do { } while (0)
#endif
#ifdef EOSB_ATTN_TIMING
#define MMARK(i) do { long long now__ = clock64(); macc__[(i) - 8] += now__ - mlast__; mlast__ = now__; if (blockIdx.x == 0 && mcnt__ < 2048) g_attn_trace[1][mcnt__++] = (now__ << 8) | (i); } while (0)
#else
#define MMARK(i) do { } while (0)
#endif

namespace {

constexpr int kParts = 4;                       // softmax warps per TMEM lane quarter (column parts of a row)
constexpr int kSoftmaxWarps = 4 * kParts;
constexpr int kPartCols = 128 / kParts;          // S columns of one tile per softmax thread
constexpr int kPartOut = 64 / kParts;            // O columns per softmax thread
constexpr int kAtThreads = (4 + kSoftmaxWarps) * 32;
constexpr int kQStages = 3;
constexpr int kKvStages = 6;
constexpr uint32_t kTileBytes = 128 * 64 * 2;   // 16 KB: Q, K_j or V_j
constexpr uint32_t kPBytes = 128 * 128 * 2;     // 32 KB: one P tile (two 128x64 blocks)
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffKv = kOffQ + kQStages * kTileBytes;
constexpr uint32_t kOffP = kOffKv + kKvStages * kTileBytes;
constexpr uint32_t kOffOnes = kOffP + 2 * kPBytes;              // 16 x 64 f16 of 1.0: B operand of the row-sum MMA
constexpr uint32_t kOffRed = kOffOnes + 2048;                   // 2 buffers x kParts x 128 floats: row max exchange
constexpr uint32_t kOffBars = kOffRed + 2 * kParts * 128 * 4;
constexpr uint32_t kNumBars = 2 * kQStages + 2 * kKvStages + 4 + 4 + 4 + 2 + 2;
constexpr uint32_t kOffMisc = kOffBars + kNumBars * 8;
constexpr uint32_t kAtSmemBytes = kOffMisc + 16 + 1024;

struct WorkItem {
    int row0;    // first packed row of the sequence
    int nrows;   // query rows of the sequence
    int nkeys;   // key rows of the sequence
    int q0;      // first query of this tile (relative to row0)
    int head;
    int ntiles;  // key tiles of 128
};

__device__ __forceinline__ WorkItem decode_item(const int4 q, int head) {
    WorkItem it;
    it.row0 = q.x;
    it.nrows = q.y;
    it.nkeys = q.z > 512 ? 512 : q.z;  // the host only selects this kernel when tokens <= 512
    it.q0 = q.w;
    it.head = head;
    it.ntiles = (it.nkeys + 127) >> 7;
    return it;
}

// A work item is processed as sub-items of one key tile (128 keys) each: a sub-item needs a quarter of
// tensor memory, so four of them are in flight per SM; the partial softmax results of a sequence with
// more than 128 keys are merged in registers (same rule as split-key flash decoding).
// The walker keeps the descriptor of the item after the current one in flight (loaded one item
// ahead), so that stepping to the next item never waits for global memory.
struct Walker {
    int w, total;
    int qi, head;             // w = qi * heads + head
    int step_q, step_h, heads;
    const int4* info;
    int sub;
    unsigned item_no;  // items visited so far
    WorkItem wi;
    int4 pre;          // descriptor of item w + step (valid if that item exists)
    __device__ __forceinline__ void advance_index() {
        w += step_q * heads + step_h;
        qi += step_q;
        head += step_h;
        if (head >= heads) { head -= heads; ++qi; }
    }
    __device__ __forceinline__ void prefetch() {
        int q2 = qi + step_q, h2 = head + step_h;
        if (h2 >= heads) ++q2;
        if (w + step_q * heads + step_h < total) pre = __ldg(info + q2);
    }
    __device__ __forceinline__ void init(int first, int stride, int tot, int h, const int4* p) {
        w = first; total = tot; heads = h; info = p; sub = 0; item_no = 0;
        qi = first / h; head = first - qi * h;
        step_q = stride / h; step_h = stride - step_q * h;
        pre = make_int4(0, 0, 0, 0);
        if (w < total) {
            wi = decode_item(__ldg(info + qi), head);
            prefetch();
        }
    }
    __device__ __forceinline__ bool valid() const { return w < total; }
    __device__ __forceinline__ int nsub() const { return wi.ntiles > 1 ? wi.ntiles : 1; }
    __device__ __forceinline__ int tile0() const { return sub; }
    __device__ __forceinline__ int nt() const { return sub < wi.ntiles ? 1 : 0; }  // 0: a sequence without keys
    __device__ __forceinline__ bool first_sub() const { return sub == 0; }
    __device__ __forceinline__ bool last_sub() const { return sub + 1 == nsub(); }
    __device__ __forceinline__ void next() {
        if (sub + 1 < nsub()) { ++sub; return; }
        advance_index();
        sub = 0; ++item_no;
        if (w < total) {
            wi = decode_item(pre, head);
            prefetch();
        }
    }
};

// MN-major operand tile (V; row = K index, 64 contiguous MN elements = 128 bytes per row, 128B
// swizzle): 8-row groups of 1024 bytes along K (stride byte offset); the leading byte offset is the
// distance from one 64-wide MN block to the next (used when N > 64).  Its descriptor has the same
// high half as the K-major one.

__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&v)[16]) { tmem_ld_32x16(taddr, v); }
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&v)[32]) { tmem_ld_32x32(taddr, v); }

// 2^x for x <= 0 on the FMA and integer pipes (no MUFU): round-to-nearest split x = n + f with
// |f| <= 0.5 by the 1.5 * 2^23 trick, cubic for 2^f (maximum relative error 7.5e-5, a third of
// half an f16 ulp), n added to the exponent field.  x below -125 (masked keys: -inf) gives 2^-125,
// which rounds to 0 in f16.
__device__ __forceinline__ float exp2_fma(float x) {
    x = fmaxf(x, -125.0f);
    const float t = x + 12582912.0f;
    const float f = x - (t - 12582912.0f);
    float p = fmaf(0.05517132207751274f, f, 0.24261054396629333f);
    p = fmaf(p, f, 0.6932609677314758f);
    p = fmaf(p, f, 0.9999281167984009f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}
// A pair of probabilities as packed f16.  Every fourth pair is computed on the FMA pipe instead of the
// MUFU pipe (16 ex2 per clock per SM): measured 4% faster than all-MUFU; every third pair 2%, every second slower.
__device__ __forceinline__ uint32_t exp2_pair_fma(float x0, float x1) {
    __half2 h = __floats2half2_rn(exp2_fma(x0), exp2_fma(x1));
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ uint32_t ex2_f16x2(float x0, float x1) {
    __half2 h = __floats2half2_rn(x0, x1);
    uint32_t hx = *reinterpret_cast<uint32_t*>(&h), px;
    asm("ex2.approx.f16x2 %0, %1;" : "=r"(px) : "r"(hx));
    return px;
}
// pair_idx is a compile-time constant after unrolling
__device__ __forceinline__ uint32_t exp2_pair(int pair_idx, float x0, float x1) {
    return (pair_idx % 4) == 3 ? exp2_pair_fma(x0, x1) : ex2_f16x2(x0, x1);
}

__global__ void __launch_bounds__(kAtThreads, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tm_qkv, const int* __restrict__ cu_qtiles,
               const int4* __restrict__ qtile_info, int batch, int hidden, int heads, __half* __restrict__ ctx,
               int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const uint32_t bar0 = base + kOffBars;
    auto q_full = [&](int s) { return bar0 + 8u * s; };
    auto q_empty = [&](int s) { return bar0 + 8u * (kQStages + s); };
    auto kv_full = [&](int s) { return bar0 + 8u * (2 * kQStages + s); };
    auto kv_empty = [&](int s) { return bar0 + 8u * (2 * kQStages + kKvStages + s); };
    const uint32_t bar1 = bar0 + 8u * (2 * kQStages + 2 * kKvStages);
    auto s_full = [&](int slot) { return bar1 + 8u * slot; };             // [slot]: S of the sub-item is in tensor memory
    auto o_full = [&](int slot) { return bar1 + 8u * (4 + slot); };       // its O is complete
    auto slot_free = [&](int slot) { return bar1 + 8u * (8 + slot); };    // its O has been read: the slot may be reused
    auto p_full = [&](int s) { return bar1 + 8u * (12 + s); };
    auto p_empty = [&](int s) { return bar1 + 8u * (14 + s); };

    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + kOffMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + kOffMisc + 4);
    float* red = reinterpret_cast<float*>(sm + kOffRed);

    const int total_items = cu_qtiles[batch] * heads;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < kQStages; ++s) {
            mbar_init(q_full(s), 1);
            mbar_init(q_empty(s), 1);
        }
        for (int s = 0; s < kKvStages; ++s) {
            mbar_init(kv_full(s), 1);
            mbar_init(kv_empty(s), 1);
        }
        for (int slot = 0; slot < 4; ++slot) {
            mbar_init(s_full(slot), 1);
            mbar_init(o_full(slot), 1);
            mbar_init(slot_free(slot), kSoftmaxWarps);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(p_full(b), kSoftmaxWarps);
            mbar_init(p_empty(b), 1);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tm_qkv);
    }
    if (warp == 2) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
        tmem_relinquish();
    }
    if (warp == 3) {
        for (int i = lane; i < 2048 / 4; i += 32) reinterpret_cast<uint32_t*>(sm + kOffOnes)[i] = 0x3c003c00u;
        fence_proxy_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t kvc = 0;
            bool ok = true;
            auto load_q = [&](const Walker& wk) -> bool {
                const int qs = wk.item_no % kQStages;
                if (!mbar_wait(q_empty(qs), ((wk.item_no / kQStages) & 1u) ^ 1u, abort_flag)) return false;
                mbar_arrive_expect_tx(q_full(qs), kTileBytes);
                tma_load_2d(base + kOffQ + qs * kTileBytes, &tm_qkv, wk.wi.head * 64, wk.wi.row0 + wk.wi.q0, q_full(qs));
                return true;
            };
            auto load_kv = [&](const Walker& wk, int part) -> bool {  // part 1 = K, 2 = V
                const int x = part * hidden + wk.wi.head * 64;
                for (int t = 0; t < wk.nt(); ++t, ++kvc) {
                    const int s = kvc % kKvStages;
                    if (!mbar_wait(kv_empty(s), ((kvc / kKvStages) & 1u) ^ 1u, abort_flag)) return false;
#ifdef EOSB_ATTN_TIMING
                    if (blockIdx.x == 0 && kvc < 2048) g_attn_trace[2][kvc] = (clock64() << 8) | 20;
#endif
                    mbar_arrive_expect_tx(kv_full(s), kTileBytes);
                    tma_load_2d(base + kOffKv + s * kTileBytes, &tm_qkv, x, wk.wi.row0 + (wk.tile0() + t) * 128, kv_full(s));
                }
                return true;
            };
            // K/V tiles mostly come from HBM (one layer's q|k|v rows exceed L2), and the ring only holds about
            // one and a half sub-items: a third walker runs kL2Ahead sub-items in front of the loads and asks
            // L2 for those tiles, so that the ring's loads are L2 hits
            auto prefetch_l2 = [&](const Walker& wk) {
                if (wk.first_sub()) tma_prefetch_l2_2d(&tm_qkv, wk.wi.head * 64, wk.wi.row0 + wk.wi.q0);
                for (int t = 0; t < wk.nt(); ++t) {
                    const int y = wk.wi.row0 + (wk.tile0() + t) * 128;
                    tma_prefetch_l2_2d(&tm_qkv, hidden + wk.wi.head * 64, y);
                    tma_prefetch_l2_2d(&tm_qkv, 2 * hidden + wk.wi.head * 64, y);
                }
            };
            // order of the K/V ring = order of consumption by the MMA warp: K(0), K(1); then K(n+2), V(n) for n = 0, 1, ...
            constexpr int kL2Ahead = 2;
            Walker vs, ks, far;   // V loads, K loads (two sub-items ahead), L2 requests (kL2Ahead further)
            vs.init(blockIdx.x, gridDim.x, total_items, heads, qtile_info);
            ks = vs;
            auto load_qk = [&](Walker& wk) -> bool {
                if (!wk.valid()) return true;
                bool r = true;
                if (wk.first_sub()) r = load_q(wk);
                r = r && load_kv(wk, 1);
                wk.next();
                return r;
            };
            ok = load_qk(ks) && load_qk(ks);
            far = ks;
            for (int i = 0; i < kL2Ahead && far.valid(); ++i) {
                prefetch_l2(far);
                far.next();
            }
            while (ok && vs.valid()) {
                if (far.valid()) {
                    prefetch_l2(far);
                    far.next();
                }
                ok = load_qk(ks);
                ok = ok && load_kv(vs, 2);
                vs.next();
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc_f16(128, 128);
            // B = [V | ones]: 64 columns of V (MN-major, as TMA delivered it) and, as a second MN block, 16
            // columns of 1.0, so that columns 64..79 of the accumulator are the row sums of P
            constexpr uint32_t idesc_o = umma_idesc_f16(128, 80) | (1u << 16);
            uint32_t kvc = 0;
            bool ok = true;
#ifdef EOSB_ATTN_TIMING
            long long mlast__ = clock64();
            long long macc__[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            int mcnt__ = 0;
#endif
            // S phase of sub-item number n, into tensor-memory slot n & 3.  Every barrier completes exactly once per
            // sub-item (a sub-item without keys arrives by hand), so all parities follow from n alone.
            auto issue_s = [&](const Walker& wk, uint32_t n) -> bool {
                const int slot = n & 3u;
                MMARK(8);
                if (n >= 4 && !mbar_wait(slot_free(slot), ((n >> 2) - 1u) & 1u, abort_flag)) return false;
                MMARK(9);
                const int qs = wk.item_no % kQStages;
                if (wk.first_sub() && !mbar_wait(q_full(qs), (wk.item_no / kQStages) & 1u, abort_flag)) return false;
                tc_fence_after();
                if (wk.nt() > 0) {
                    const int s = kvc % kKvStages;
                    if (!mbar_wait(kv_full(s), (kvc / kKvStages) & 1u, abort_flag)) return false;
                    ++kvc;
                    tc_fence_after();
                    MMARK(10);
                    const uint32_t q_lo = umma_desc_sw128_lo(base + kOffQ + qs * kTileBytes);
                    const uint32_t k_lo = umma_desc_sw128_lo(base + kOffKv + s * kTileBytes);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)  // 32 bytes along K per step = 2 in descriptor units
                        umma_f16_split(tmem_base + slot * 128, q_lo + kk * 2, kDescSw128Hi, k_lo + kk * 2, kDescSw128Hi,
                                       idesc_s, kk > 0 ? 1u : 0u);
                    umma_commit(kv_empty(s));
                    umma_commit(s_full(slot));
                    MMARK(11);
                    if (wk.last_sub()) umma_commit(q_empty(qs));
                } else {
                    mbar_arrive(s_full(slot));
                    if (wk.last_sub()) mbar_arrive(q_empty(qs));
                }
                return true;
            };
            auto issue_pv = [&](const Walker& wk, uint32_t n) -> bool {
                const int slot = n & 3u;
                const int pb = n & 1u;
                MMARK(8);
                if (!mbar_wait(p_full(pb), (n >> 1) & 1u, abort_flag)) return false;
                MMARK(12);
                if (wk.nt() > 0) {
                    const int s = kvc % kKvStages;
                    if (!mbar_wait(kv_full(s), (kvc / kKvStages) & 1u, abort_flag)) return false;
                    ++kvc;
                    tc_fence_after();
                    MMARK(13);
                    const uint32_t p_addr = base + kOffP + pb * kPBytes;
                    const uint32_t v_addr = base + kOffKv + s * kTileBytes;
                    const uint32_t p_lo = umma_desc_sw128_lo(p_addr);
                    // MN-major V: start address and the leading offset (distance to the block of ones) both
                    // move by one 16-key slab (2048 bytes = 128 units) per step, in opposite directions
                    const uint32_t v_lo = ((v_addr >> 4) & 0x3fffu) | (((base + kOffOnes - v_addr) >> 4) << 16);
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk)
                        umma_f16_split(tmem_base + slot * 128, p_lo + (kk >> 2) * (kPBytes / 2 / 16) + (kk & 3) * 2,
                                       kDescSw128Hi, v_lo + kk * 128u - ((kk * 128u) << 16), kDescSw128Hi, idesc_o,
                                       kk > 0 ? 1u : 0u);
                    umma_commit(kv_empty(s));
                    umma_commit(p_empty(pb));
                    umma_commit(o_full(slot));
                    MMARK(14);
                } else {
                    mbar_arrive(p_empty(pb));
                    mbar_arrive(o_full(slot));
                }
                return true;
            };
            // S runs two sub-items ahead of P V: S(0), S(1); then S(n + 2), PV(n) for n = 0, 1, ...
            Walker ws, wp;
            wp.init(blockIdx.x, gridDim.x, total_items, heads, qtile_info);
            ws = wp;
            uint32_t ns = 0, np = 0;
            for (int i = 0; i < 2 && ok && ws.valid(); ++i) {
                ok = issue_s(ws, ns++);
                ws.next();
            }
            while (ok && wp.valid()) {
                if (ws.valid()) {
                    ok = issue_s(ws, ns++);
                    ws.next();
                }
                ok = ok && issue_pv(wp, np++);
                wp.next();
            }
#ifdef EOSB_ATTN_TIMING
            if (blockIdx.x == 0)
                for (int i = 0; i < 8; ++i) g_attn_timing[8 + i] += macc__[i];
#endif
        }
        __syncwarp();
    } else if (warp >= 4) {
        // ------------------------------------------------------------ softmax + epilogue
        const int w8 = warp - 4;
        const int quarter = warp & 3;          // TMEM lane quarter this warp may access
        const int part = w8 >> 2;              // which kPartCols columns of the tile
        const int r = quarter * 32 + lane;     // query row inside the tile
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const float sl2 = 0.125f * 1.4426950408889634f;  // 1/sqrt(64) * log2(e)
        bool ok = true;
        // running result of the item whose sub-items are being retired: O columns of this thread, maximum, row sum
        float acc_o[kPartOut], acc_m = 0.f, acc_l = 0.f;
#pragma unroll
        for (int e = 0; e < kPartOut; ++e) acc_o[e] = 0.f;

#ifdef EOSB_ATTN_TIMING
        long long tlast__ = clock64();
        long long tacc__[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        int tcnt__ = 0;
#endif
        // retire sub-item number n (two sub-items after its softmax, so that its P V MMAs are long done): fold its
        // partial (O, m, l) into the item's running result; after the item's last sub-item, O / l -> f16 -> global
        // What retiring a sub-item needs to know about it, two registers per thread: the offset of this thread's
        // output (row, head, column part) and flags.
        constexpr int kFirst = 1, kLast = 2, kHasKeys = 4, kRowsLive = 8, kRowValid = 16;
        auto epilogue = [&](int out_off, int fl, uint32_t n, float ms_n) -> bool {
            const int slot = n & 3u;
            float o[kPartOut], l = 0.f;
#pragma unroll
            for (int e = 0; e < kPartOut; ++e) o[e] = 0.f;
            if (!mbar_wait(o_full(slot), (n >> 2) & 1u, abort_flag)) return false;
            tc_fence_after();
            TMARK(6);
            if ((fl & (kHasKeys | kRowsLive)) == (kHasKeys | kRowsLive)) {
                uint32_t v[kPartOut], lv[1];
                __syncwarp();
                tmem_ld_cols(tmem_base + lane_addr + slot * 128 + part * kPartOut, v);
                tmem_ld_32x1(tmem_base + lane_addr + slot * 128 + 64, lv);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < kPartOut; ++e) o[e] = __uint_as_float(v[e]);
                l = __uint_as_float(lv[0]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(slot_free(slot));
            TMARK(7);
            if (fl & kFirst) {
#pragma unroll
                for (int e = 0; e < kPartOut; ++e) acc_o[e] = o[e];
                acc_m = ms_n;
                acc_l = l;
            } else {
                const float m = fmaxf(acc_m, ms_n);
                float a, b;  // both exponents are <= 0
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(a) : "f"(acc_m - m));
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(b) : "f"(ms_n - m));
#pragma unroll
                for (int e = 0; e < kPartOut; ++e) acc_o[e] = acc_o[e] * a + o[e] * b;
                acc_l = acc_l * a + l * b;
                acc_m = m;
            }
            if ((fl & (kLast | kRowValid)) == (kLast | kRowValid)) {
                const float inv = acc_l > 0.f ? __frcp_rn(acc_l) : 0.f;
                __half* out = ctx + (size_t)out_off;
#pragma unroll
                for (int q = 0; q < kPartOut / 16; ++q) {  // 32 bytes (one sector) per store
                    uint32_t ow[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        __half2 hh = __floats2half2_rn(acc_o[q * 16 + 2 * e] * inv, acc_o[q * 16 + 2 * e + 1] * inv);
                        ow[e] = *reinterpret_cast<uint32_t*>(&hh);
                    }
                    st_global_v8(out + q * 16, ow);
                }
            }
            return true;
        };

        Walker cur;
        cur.init(blockIdx.x, gridDim.x, total_items, heads, qtile_info);
        int off_prev1 = 0, off_prev2 = 0, fl_prev1 = 0, fl_prev2 = 0;   // sub-items n - 1 and n - 2
        uint32_t n = 0;
        float ms_prev1 = 0.f, ms_prev2 = 0.f;
        while (ok && cur.valid()) {
            const int slot = n & 3u;
            const int pb = n & 1u;
            const int nt = cur.nt();
            const int key0 = cur.tile0() * 128;           // first key of this sub-item
            const int nkeys = cur.wi.nkeys;
            // a warp whose 32 query rows are all padding of the last query tile keeps the barrier protocol
            // but computes nothing (its P rows and O rows are never used)
            const bool live = cur.wi.q0 + quarter * 32 < cur.wi.nrows;
            float ms = 0.f;
            if (!mbar_wait(s_full(slot), (n >> 2) & 1u, abort_flag)) break;
            tc_fence_after();
            TMARK(0);
            const int key_in_tile = part * kPartCols;
            const int col0 = key0 + key_in_tile;          // key index of this thread's first column
            const int lim = nkeys - col0;
            // pass A: row maximum over the visible keys of this sub-item
            float mx = -INFINITY;
            if (nt > 0 && live && lim > 0) {
                uint32_t v[kPartCols];
                __syncwarp();
                tmem_ld_cols(tmem_base + lane_addr + slot * 128 + key_in_tile, v);
                tmem_ld_wait();
                if (lim >= kPartCols) {
#pragma unroll
                    for (int e = 0; e < kPartCols; e += 2)
                        mx = fmaxf(mx, fmaxf(__uint_as_float(v[e]), __uint_as_float(v[e + 1])));
                } else {
#pragma unroll
                    for (int e = 0; e < kPartCols; ++e)
                        if (e < lim) mx = fmaxf(mx, __uint_as_float(v[e]));
                }
            }
            TMARK(1);
            // exchange with the warps that hold the other columns of these rows (one named barrier per group of
            // 32 rows); the buffer alternates per sub-item, and nobody can be two sub-items ahead of a warp that
            // has not yet read, because every sub-item passes this barrier
            {
                float* redn = red + (n & 1u) * (kParts * 128);
                redn[part * 128 + r] = mx;
                named_bar_sync(2 + quarter, kParts * 32);
#pragma unroll
                for (int q = 0; q < kParts; ++q) mx = fmaxf(mx, redn[q * 128 + r]);
            }
            // a sub-item with keys holds at least one visible key, so mx is finite for live rows
            if (nt > 0) ms = mx * sl2;
            TMARK(2);
            // the sub-item before last is retired here: its P V MMAs have had a whole sub-item to finish, and freeing
            // its slot lets the S phase two sub-items ahead start under pass B
            if (n >= 2) {
                ok = epilogue(off_prev2, fl_prev2, n - 2, ms_prev2);
                if (!ok) break;
            }
            TMARK(5);
            if (!mbar_wait(p_empty(pb), ((n >> 1) & 1u) ^ 1u, abort_flag)) break;
            TMARK(3);
            if (nt > 0 && live) {
                // pass B: probabilities, the P tile for the second MMA
                // P tile = two 128 x 64 K-major blocks; this thread's keys are kPartCols / 8 16-byte chunks of its row
                constexpr int kChunks = kPartCols / 8;
                uint8_t* prow = sm + kOffP + pb * kPBytes + (key_in_tile >> 6) * (kPBytes / 2) + (r >> 3) * 1024 + (r & 7) * 128;
                const int chunk0 = (key_in_tile & 63) >> 3;
                uint32_t packed[kPartCols / 2];
                if (lim > 0) {
                    uint32_t v[kPartCols];
                    __syncwarp();
                    tmem_ld_cols(tmem_base + lane_addr + slot * 128 + key_in_tile, v);
                    tmem_ld_wait();
                    if (lim >= kPartCols) {
#pragma unroll
                        for (int e = 0; e < kPartCols; e += 2)
                            packed[e >> 1] = exp2_pair(e >> 1, fmaf(__uint_as_float(v[e]), sl2, -ms), fmaf(__uint_as_float(v[e + 1]), sl2, -ms));
                    } else {  // the sequence's last, partial tile: masked keys get exp2(-inf) = 0
#pragma unroll
                        for (int e = 0; e < kPartCols; e += 2) {
                            const float a0 = e < lim ? fmaf(__uint_as_float(v[e]), sl2, -ms) : -INFINITY;
                            const float a1 = e + 1 < lim ? fmaf(__uint_as_float(v[e + 1]), sl2, -ms) : -INFINITY;
                            packed[e >> 1] = exp2_pair(e >> 1, a0, a1);
                        }
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < kPartCols / 2; ++e) packed[e] = 0u;
                }
#pragma unroll
                for (int q = 0; q < kChunks; ++q)
                    *reinterpret_cast<uint4*>(prow + (((chunk0 + q) ^ (r & 7)) << 4)) =
                        make_uint4(packed[q * 4], packed[q * 4 + 1], packed[q * 4 + 2], packed[q * 4 + 3]);
            }
            tc_fence_before();  // the S columns of this slot are about to be overwritten by O
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(pb));
            TMARK(4);
            off_prev2 = off_prev1;
            fl_prev2 = fl_prev1;
            ms_prev2 = ms_prev1;
            {
                const int qrow = cur.wi.q0 + r;
                off_prev1 = (cur.wi.row0 + qrow) * hidden + cur.wi.head * 64 + part * kPartOut;
                fl_prev1 = (cur.first_sub() ? kFirst : 0) | (cur.last_sub() ? kLast : 0) | (nt > 0 ? kHasKeys : 0) |
                           (live ? kRowsLive : 0) | (qrow < cur.wi.nrows ? kRowValid : 0);
            }
            ms_prev1 = ms;
            cur.next();
            ++n;
        }
        // retire the last two sub-items
        if (ok && n >= 2) ok = epilogue(off_prev2, fl_prev2, n - 2, ms_prev2);
        if (ok && n >= 1) ok = epilogue(off_prev1, fl_prev1, n - 1, ms_prev1);
#ifdef EOSB_ATTN_TIMING
        if (blockIdx.x == 0 && threadIdx.x == 128)
            for (int i = 0; i < 8; ++i) g_attn_timing[i] += tacc__[i];
#endif
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *abort_flag != 0 && status != nullptr) atomicExch(status, kStatusPipelineTimeout);
}

}  // namespace

#ifdef EOSB_ATTN_TIMING
extern "C" __attribute__((visibility("default"))) int eos_b200_debug_attn_timing(long long* out16, int reset) {
    long long zero[16] = {0};
    if (cudaMemcpyFromSymbol(out16, g_attn_timing, sizeof(zero)) != cudaSuccess) return 1;
    if (reset && cudaMemcpyToSymbol(g_attn_timing, zero, sizeof(zero)) != cudaSuccess) return 1;
    return 0;
}
extern "C" __attribute__((visibility("default"))) int eos_b200_debug_attn_trace(long long* out6144) {
    return cudaMemcpyFromSymbol(out6144, g_attn_trace, sizeof(long long) * 6144) != cudaSuccess;
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

void attn_tc_launch(const AttnTcPlan& plan, const SeqLayout& lay, int batch, int hidden, int heads, __half* ctx,
                    int* status, int sm_count, cudaStream_t stream) {
    attn_tc_kernel<<<sm_count, kAtThreads, kAtSmemBytes, stream>>>(plan.tm_qkv, lay.cu_qtiles, lay.qtile_info, batch,
                                                                    hidden, heads, ctx, status);
}

}  // namespace eosb
