// out[M,N] = epilogue( A[M,K] (f16) x W[N,K]^T ), W stored as 8-bit codes with per-output-channel
// scales (or as f16), on the 5th-generation tensor cores of sm_100a.
//
// This is the dense projection of the q8 encoder: it replaces the reference's
// cublasSgemm path (runtime/backends/cuda/native_linux.go:1267-1307, called per projection from
// runBGEFullEncoderHidden :7941-8190) and the host loop denseHFRange
// (runtime/backend/bert_encoder_layer_ops.go:452-462): y = x W^T + b with W in HF [out,in] layout.
//
// Design (one persistent CTA per SM, warp-specialised):
//   warp 0      TMA producer: A tile 128x64 f16 (128B swizzle) and the W tile 256x64 (8-bit codes, no
//               swizzle, or f16 with 128B swizzle) per k-block into a 4-stage ring, completion on mbarriers.
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=256, K=16, f16 x f16 -> f32) with
//               the accumulator in tensor memory; tcgen05.commit releases ring stages.
//   warp 2      allocates / frees tensor memory.
//   warps 4-7   (8-bit weights only) dequantisers: expand the codes to f16 in shared memory, written
//               directly in the 128B-swizzled K-major layout the MMA reads (int8 -> f16 is exact; the
//               per-channel scale is applied in fp32 in the epilogue, which is the same product:
//               sum_k a_k (s_n q_kn) = s_n sum_k a_k q_kn).
//   last 8      epilogue warps, two per TMEM lane quarter, each owning 128 of the tile's 256 columns:
//               tcgen05.ld (thread = row, software-pipelined 16 columns at a time), scale, bias, GELU or
//               residual add, f16.  A finished 32-row x 32-column slab leaves through a per-warp staging slab in the
//               64-byte TMA swizzle as one TMA store; the residual comes in through the same slab with coalesced
//               loads (8 rows x 64 contiguous bytes per instruction).
// Two accumulators (2 x 256 TMEM columns) let the epilogue of tile i overlap the main loop of tile i+1.
//
// CTA-pair mode (f16 weights): two CTAs of a cluster share one 256x256 output tile.  Each loads its
// own 128 rows of A and 128 of the 256 W rows (32 KB per k-block instead of 48 KB, 6 ring stages), the
// leader's MMA thread issues tcgen05.mma.cta_group::2 (M = 256) reading both CTAs' shared memory, and
// each CTA's epilogue drains its own 128 rows from its own tensor memory.  TMA completions of both
// CTAs count on the leader's full barrier; the MMA commits release both CTAs' ring stages; both
// epilogues arrive on the leader's accumulator-empty barrier.  Measured on the encoder's shapes it wins where the
// main loop dominates (K = 3072: 6 % faster, the operand feed per CTA drops by a third) and on wide outputs
// (N = 2304: 5 %), and loses on the K = N = 768 projection, so it serves K >= 2048 and N >= 2048 with K >= 768;
// environment EOS_B200_GEMM_CTA_PAIR=1 forces it for every f16 projection, =0 turns it off.
// Every mbarrier wait is bounded (common.cuh: mbar_wait); on a timeout the kernel raises a CTA-wide
// abort flag, all roles leave their loops, TMEM is freed and the status word is set.
#include "gemm_tc.cuh"

#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "tma_util.cuh"

namespace eosb {

#ifdef EOSB_GEMM_TIMING
__device__ long long g_gemm_timing[16];
// timing marks accumulate in registers (a read-modify-write of global memory per mark would itself
// stall the role being measured) and are flushed once per role
#define GMARK(i) do { long long now__ = clock64(); gacc__[(i) & 3] += now__ - tlast__; tlast__ = now__; } while (0)
#define GFLUSH(base) do { if (tm__) for (int i__ = 0; i__ < 4; ++i__) g_gemm_timing[(base) + i__] += gacc__[i__]; } while (0)
#else
#define GMARK(i) do { } while (0)
#define GFLUSH(base) do { } while (0)
#endif

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int kStagesB16 = 2;   // ring depth of the dequantised W tiles (8-bit mode)
constexpr int kTmemCols = 512;  // two 128x256 fp32 accumulators
constexpr uint32_t kBytesA = BM * BK * 2;
constexpr uint32_t kBytesB8 = BN * BK;
constexpr int kSlabCols = 32;                  // columns of the staging slab of one epilogue warp
constexpr uint32_t kSlabBytes = 32 * kSlabCols * 2;

template <bool kBInt8, bool kPair>
struct Cfg {
    static_assert(!(kBInt8 && kPair), "CTA-pair mode takes f16 weights");
    static constexpr int kStagesAB = kPair ? 6 : 4;          // ring depth of the TMA-fed stages
    static constexpr int kEpilogueWarps = 8;                 // 2 per TMEM lane quarter (a multiple of 4)
    static constexpr int kWarpCols = BN / (kEpilogueWarps / 4);  // tile columns one epilogue warp owns
    static constexpr int kBRows = kPair ? BN / 2 : BN;        // W rows this CTA holds per k-block
    static constexpr uint32_t kBytesB16 = kBRows * BK * 2;
    static constexpr int kTileM = kPair ? 2 * BM : BM;        // output rows per work item
    static constexpr int kDequantWarps = kBInt8 ? 8 : 0;
    static constexpr int kFirstEpilogueWarp = 4 + kDequantWarps;
    static constexpr int kThreads = (kFirstEpilogueWarp + kEpilogueWarps) * 32;
    static constexpr int kBStages = kBInt8 ? kStagesB16 : kStagesAB;  // f16 W tiles ride the TMA ring
    // shared memory map (offsets from a 1024-byte aligned base)
    static constexpr uint32_t kOffA = 0;
    static constexpr uint32_t kOffB16 = kOffA + kStagesAB * kBytesA;
    static constexpr uint32_t kOffB8 = kOffB16 + kBStages * kBytesB16;
    static constexpr uint32_t kOffSlab = kOffB8 + (kBInt8 ? kStagesAB * kBytesB8 : 0);
    static constexpr uint32_t kOffScaleBias = kOffSlab + kEpilogueWarps * kSlabBytes;  // 2 x 256 float2
    static constexpr uint32_t kOffBars = kOffScaleBias + 2 * BN * 8;
    static constexpr uint32_t kNumBars = 2 * kStagesAB + 2 * kStagesB16 + 4;
    static constexpr uint32_t kOffMisc = kOffBars + kNumBars * 8;
    static constexpr uint32_t kSmemBytes = kOffMisc + 16 + 1024;  // + alignment slack
};

// kMode >= 0 fixes the epilogue at compile time (the one-CTA kernels, which serve the encoder: the residual
// registers and the activation code of the other modes disappear); kMode < 0 reads it from the parameters.
template <bool kBInt8, bool kPair, int kMode>
__global__ void __launch_bounds__(Cfg<kBInt8, kPair>::kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
               const __grid_constant__ CUtensorMap tm_out, GemmParams p) {
    using C = Cfg<kBInt8, kPair>;
    const int mode = kMode >= 0 ? kMode : p.mode;
    constexpr int kStagesAB = C::kStagesAB;
    constexpr int kEpilogueWarps = C::kEpilogueWarps;
    constexpr int kWarpCols = C::kWarpCols;
    constexpr uint32_t kBytesB16 = C::kBytesB16;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const uint32_t bar0 = base + C::kOffBars;
    auto full_ab = [&](int s) { return bar0 + 8u * s; };
    auto empty_ab = [&](int s) { return bar0 + 8u * (kStagesAB + s); };
    auto full_b16 = [&](int s) { return bar0 + 8u * (2 * kStagesAB + s); };
    auto empty_b16 = [&](int s) { return bar0 + 8u * (2 * kStagesAB + kStagesB16 + s); };
    auto acc_full = [&](int s) { return bar0 + 8u * (2 * kStagesAB + 2 * kStagesB16 + s); };
    auto acc_empty = [&](int s) { return bar0 + 8u * (2 * kStagesAB + 2 * kStagesB16 + 2 + s); };

    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + C::kOffMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + C::kOffMisc + 4);
    // set by an epilogue warp whose wait ran out, read by all epilogue warps right after their next common
    // barrier: they leave the tile loop together, so the named barrier is never left waiting for warps that have gone
    volatile int* epi_stop = reinterpret_cast<volatile int*>(sm + C::kOffMisc + 8);
    float2* scale_bias = reinterpret_cast<float2*>(sm + C::kOffScaleBias);

    int m_rows = p.m_alloc;
    if (p.m_ptr != nullptr) {
        int v = *p.m_ptr;
        m_rows = v < p.m_alloc ? v : p.m_alloc;
        if (m_rows < 0) m_rows = 0;
    }
    const int m_tiles = (m_rows + C::kTileM - 1) / C::kTileM;
    const int n_tiles = (p.n + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;
    const int num_kb = (p.k + BK - 1) / BK;
    // work distribution: one worker = one CTA, or one CTA pair (cluster of 2: blocks 2i and 2i + 1)
    const uint32_t cta_rank = kPair ? cluster_ctarank() : 0u;
    const int worker = kPair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int num_workers = kPair ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int m_off = (int)cta_rank * BM;  // this CTA's rows inside the work item

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        *epi_stop = 0;
        for (int s = 0; s < kStagesAB; ++s) {
            mbar_init(full_ab(s), 1);
            mbar_init(empty_ab(s), 1 + C::kDequantWarps);  // MMA commit (+ dequantiser warps)
        }
        for (int s = 0; s < kStagesB16; ++s) {
            mbar_init(full_b16(s), kBInt8 ? C::kDequantWarps : 1);
            mbar_init(empty_b16(s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(acc_full(s), 1);
            mbar_init(acc_empty(s), kPair ? 2 * kEpilogueWarps : kEpilogueWarps);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        tma_prefetch_desc(&tm_out);
    }
    if (warp == 2) {
        if (kPair) {
            tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    if (kPair) cluster_sync_all(); else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
#ifdef EOSB_GEMM_TIMING
            long long tlast__ = clock64();
            long long gacc__[4] = {0, 0, 0, 0};
            const bool tm__ = blockIdx.x == 0;
#endif
            for (int tile = worker; ok && tile < total_tiles; tile += num_workers) {
                const int m0 = (tile / n_tiles) * C::kTileM + m_off;
                const int n0 = (tile % n_tiles) * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % kStagesAB;
                    const uint32_t ph = (it / kStagesAB) & 1u;
#ifdef EOSB_GEMM_TIMING
                    if (tm__) GMARK(9);
#endif
                    if (!mbar_wait(empty_ab(s), ph ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
#ifdef EOSB_GEMM_TIMING
                    if (tm__) GMARK(8);
#endif
                    if (kPair) {
                        // both CTAs' bytes are counted on the leader's barrier, which the leader arms
                        const uint32_t full_leader = mapa_shared(full_ab(s), 0);
                        if (cta_rank == 0) mbar_arrive_expect_tx(full_ab(s), 2 * (kBytesA + kBytesB16));
                        tma_load_2d_pair(base + C::kOffA + s * kBytesA, &tm_a, kb * BK, m0, full_leader);
                        tma_load_2d_pair(base + C::kOffB16 + s * kBytesB16, &tm_b, kb * BK, n0 + (int)cta_rank * C::kBRows,
                                         full_leader);
                    } else {
                        mbar_arrive_expect_tx(full_ab(s), kBytesA + (kBInt8 ? kBytesB8 : kBytesB16));
                        tma_load_2d(base + C::kOffA + s * kBytesA, &tm_a, kb * BK, m0, full_ab(s));
                        if (kBInt8)
                            tma_load_2d(base + C::kOffB8 + s * kBytesB8, &tm_b, kb * BK, n0, full_ab(s));
                        else
                            tma_load_2d(base + C::kOffB16 + s * kBytesB16, &tm_b, kb * BK, n0, full_ab(s));
                    }
                }
            }
#ifdef EOSB_GEMM_TIMING
            GFLUSH(8);
#endif
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0 && cta_rank == 0) {
            constexpr uint32_t idesc = umma_idesc_f16(C::kTileM, BN);
            uint32_t it = 0;
            uint32_t t = 0;
            bool ok = true;
#ifdef EOSB_GEMM_TIMING
            long long tlast__ = clock64();
            long long gacc__[4] = {0, 0, 0, 0};
            const bool tm__ = blockIdx.x == 0;
#endif
            for (int tile = worker; ok && tile < total_tiles; tile += num_workers, ++t) {
                const uint32_t ab = t & 1u;
                const uint32_t aph = (t >> 1) & 1u;
                if (!mbar_wait(acc_empty(ab), aph ^ 1u, abort_flag)) break;
                if (kPair) fence_acq_rel_cluster();  // half of the arrivals came from the partner CTA
                tc_fence_after();
#ifdef EOSB_GEMM_TIMING
                if (tm__) GMARK(0);
#endif
                const uint32_t d_tmem = tmem_base + ab * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % kStagesAB;
                    const uint32_t ph = (it / kStagesAB) & 1u;
                    if (!mbar_wait(full_ab(s), ph, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint32_t b_addr;
                    int c = 0;
                    if (kBInt8) {
                        c = it % kStagesB16;
                        const uint32_t cph = (it / kStagesB16) & 1u;
                        if (!mbar_wait(full_b16(c), cph, abort_flag)) {
                            ok = false;
                            break;
                        }
                        b_addr = base + C::kOffB16 + c * kBytesB16;
                    } else {
                        b_addr = base + C::kOffB16 + s * kBytesB16;
                    }
                    tc_fence_after();
#ifdef EOSB_GEMM_TIMING
                    if (tm__) GMARK(1);
#endif
                    const uint32_t a_lo = umma_desc_sw128_lo(base + C::kOffA + s * kBytesA);
                    const uint32_t b_lo = umma_desc_sw128_lo(b_addr);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {  // 32 bytes along K per step = 2 in descriptor units
                        if (kPair)
                            umma_f16_pair_split(d_tmem, a_lo + k * 2, kDescSw128Hi, b_lo + k * 2, kDescSw128Hi, idesc,
                                                (kb > 0 || k > 0) ? 1u : 0u);
                        else
                            umma_f16_split(d_tmem, a_lo + k * 2, kDescSw128Hi, b_lo + k * 2, kDescSw128Hi, idesc,
                                           (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    if (kPair) umma_commit_pair(empty_ab(s), 3); else umma_commit(empty_ab(s));
                    if (kBInt8) umma_commit(empty_b16(c));
#ifdef EOSB_GEMM_TIMING
                    if (tm__) GMARK(2);
#endif
                }
                if (ok) {
                    if (kPair) umma_commit_pair(acc_full(ab), 3); else umma_commit(acc_full(ab));
                }
            }
#ifdef EOSB_GEMM_TIMING
            GFLUSH(0);
#endif
        }
        __syncwarp();
    } else if (kBInt8 && warp >= 4 && warp < C::kFirstEpilogueWarp) {
        // ------------------------------------------------------------ dequantisers (8-bit weights)
        constexpr int kDqThreads = (C::kDequantWarps > 0 ? C::kDequantWarps : 1) * 32;
        const int tid = threadIdx.x - 128;
        const uint32_t bias1152 = 0x64806480u;  // half2(1152, 1152) = 1024 + 128
        uint32_t it = 0;
        bool ok = true;
        for (int tile = worker; ok && tile < total_tiles; tile += num_workers) {
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const int s = it % kStagesAB;
                const uint32_t ph = (it / kStagesAB) & 1u;
                const int c = it % kStagesB16;
                const uint32_t cph = (it / kStagesB16) & 1u;
                if (!mbar_wait(full_ab(s), ph, abort_flag) || !mbar_wait(empty_b16(c), cph ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                const uint8_t* src = sm + C::kOffB8 + s * kBytesB8;
                uint8_t* dst = sm + C::kOffB16 + c * kBytesB16;
#pragma unroll
                for (int i = 0; i < (BN * BK / 16) / kDqThreads; ++i) {
                    const int q = i * kDqThreads + tid;
                    const int r = q >> 2;
                    const int j = q & 3;
                    const uint4 raw8 = *reinterpret_cast<const uint4*>(src + r * BK + j * 16);
                    const uint32_t w[4] = {raw8.x, raw8.y, raw8.z, raw8.w};
                    uint32_t h[8];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        // bytes u = code + 128; 0x6400 | u is the f16 value 1024 + u, so
                        // (1024 + u) - 1152 = code, exactly.
                        uint32_t lo = __byte_perm(w[e], 0x64646464u, 0x5140);
                        uint32_t hi = __byte_perm(w[e], 0x64646464u, 0x7362);
                        __half2 l2 = __hsub2(*reinterpret_cast<__half2*>(&lo), *reinterpret_cast<const __half2*>(&bias1152));
                        __half2 h2 = __hsub2(*reinterpret_cast<__half2*>(&hi), *reinterpret_cast<const __half2*>(&bias1152));
                        h[2 * e] = *reinterpret_cast<uint32_t*>(&l2);
                        h[2 * e + 1] = *reinterpret_cast<uint32_t*>(&h2);
                    }
                    uint8_t* row = dst + (r >> 3) * 1024 + (r & 7) * 128;
                    const int x = r & 7;
                    *reinterpret_cast<uint4*>(row + (((2 * j) ^ x) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
                    *reinterpret_cast<uint4*>(row + (((2 * j + 1) ^ x) << 4)) = make_uint4(h[4], h[5], h[6], h[7]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(full_b16(c));
                    mbar_arrive(empty_ab(s));
                }
            }
        }
    } else if (warp >= C::kFirstEpilogueWarp) {
        // ------------------------------------------------------------ epilogue
        const int ew = warp - C::kFirstEpilogueWarp;               // 0..7
        const int etid = threadIdx.x - C::kFirstEpilogueWarp * 32;  // 0..255
        const int wrow0 = (warp & 3) * 32;                          // this warp's rows inside the tile
        const int epart = ew >> 2;                                  // which kWarpCols columns of the tile
        const uint32_t lane_base = (uint32_t)wrow0;
        uint8_t* slab = sm + C::kOffSlab + ew * kSlabBytes;         // [32 rows][8 x 16 B], chunk index ^ (row & 7)
#ifdef EOSB_GEMM_TIMING
        long long tlast__ = clock64();
        long long gacc__[4] = {0, 0, 0, 0};
        const bool tm__ = blockIdx.x == 0 && etid == 0;
#endif
        uint32_t t = 0;
        const uint32_t acc_empty_leader0 = kPair ? mapa_shared(acc_empty(0), 0) : acc_empty(0);
        const uint32_t acc_empty_leader1 = kPair ? mapa_shared(acc_empty(1), 0) : acc_empty(1);
        // (scale, bias) of output column n; one column of the 256-wide tile per epilogue thread
        static_assert(kEpilogueWarps * 32 >= BN, "one epilogue thread per tile column");
        auto fetch_scale_bias = [&](int n) {
            float2 v = make_float2(1.0f, 0.0f);
            if (etid < BN && n < p.n) {
                if (p.scale != nullptr) v.x = __ldg(p.scale + n);
                if (p.bias != nullptr) v.y = __ldg(p.bias + n);
            }
            return v;
        };
        float2 sb_next = make_float2(1.0f, 0.0f);
        if (worker < total_tiles) sb_next = fetch_scale_bias((worker % n_tiles) * BN + etid);
        for (int tile = worker; tile < total_tiles; tile += num_workers, ++t) {
            const int m0 = (tile / n_tiles) * C::kTileM + m_off;
            const int n0 = (tile % n_tiles) * BN;
            const uint32_t ab = t & 1u;
            const uint32_t aph = (t >> 1) & 1u;
            // this tile's column constants were requested one tile ago; request the next tile's now
            float2* sb = scale_bias + ab * BN;
            if (etid < BN) sb[etid] = sb_next;
            if (tile + num_workers < total_tiles) sb_next = fetch_scale_bias(((tile + num_workers) % n_tiles) * BN + etid);
            const int m = m0 + wrow0 + lane;  // this thread's accumulator row
            const bool row_ok = m < m_rows;
            const int rows_here = m_rows - (m0 + wrow0);  // rows of this warp's block that exist (may exceed 32)
            const uint32_t taddr = tmem_base + (lane_base << 16) + ab * BN;
            __half* out_row = p.out + (size_t)m * p.ldo;
            const __half* res_row = p.residual + (size_t)m * p.ldr;
            // coalesced access pattern of the slab copies: instruction i covers rows 8i .. 8i+7, 64 bytes each
            // slab layout: row pitch 64 B, 16-byte chunk c of row r at position c ^ ((r >> 1) & 3)
            const int crow = lane >> 2, cchunk = lane & 3;
            const bool residual = mode == kEpiBiasResidual;
            constexpr int kSlabs = kWarpCols / kSlabCols;

            // residual of the next slab is requested one slab ahead (the first one before the accumulator
            // is even complete)
            uint4 res_in[4];
            auto residual_fetch = [&](int slab_idx) {
                const int col = n0 + epart * kWarpCols + slab_idx * kSlabCols;
                if (slab_idx >= kSlabs || col + kSlabCols > p.n) return;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int rr = 8 * i + crow;
                    res_in[i] = make_uint4(0, 0, 0, 0);
                    if (rr < rows_here)
                        res_in[i] = *reinterpret_cast<const uint4*>(p.residual + (size_t)(m0 + wrow0 + rr) * p.ldr + col +
                                                                     cchunk * 8);
                }
            };
            if (residual) residual_fetch(0);
            named_bar_sync(1, kEpilogueWarps * 32);
            if (*epi_stop != 0) break;
#ifdef EOSB_GEMM_TIMING
            if (tm__) GMARK(4);
#endif
            if (!__all_sync(0xffffffffu, mbar_wait(acc_full(ab), aph, abort_flag))) {
                *epi_stop = 1;
                continue;   // to the next common barrier, where every epilogue warp sees the flag
            }
            tc_fence_after();
#ifdef EOSB_GEMM_TIMING
            if (tm__) GMARK(4);
#endif

            // accumulator chunks of 16 columns ping-pong between two register buffers: while one is being
            // turned into outputs the next tcgen05.ld fills the other
            uint32_t ra[16], rb[16];
            __syncwarp();
            tmem_ld_32x16(taddr + epart * kWarpCols, ra);
#pragma unroll 1
            for (int sl = 0; sl < kSlabs; ++sl) {
                const int col0 = epart * kWarpCols + sl * kSlabCols;  // first column of the slab inside the tile
                const int ncol0 = n0 + col0;
                if (ncol0 >= p.n) {
                    tmem_ld_wait();
                    break;
                }
                const bool fast = (ncol0 + kSlabCols <= p.n);
                uint4 res_own[4];
                // the slab of the previous iteration may still be read by its TMA store: the residual path needs the
                // slab now, the others only when the first chunk's results are written (see chunk below)
                if (residual) {
                    if (lane == 0) tma_store_wait_read();
                    __syncwarp();
                }
                if (fast && residual) {
                    // residual slab: coalesced registers -> staging -> this thread's own row
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int rr = 8 * i + crow;
                        *reinterpret_cast<uint4*>(slab + rr * 64 + ((cchunk ^ ((rr >> 1) & 3)) << 4)) = res_in[i];
                    }
                    __syncwarp();
#pragma unroll
                    for (int c4 = 0; c4 < 4; ++c4)
                        res_own[c4] = *reinterpret_cast<const uint4*>(slab + lane * 64 + ((c4 ^ ((lane >> 1) & 3)) << 4));
                    __syncwarp();
                    residual_fetch(sl + 1);
                }
#ifdef EOSB_GEMM_TIMING
                if (tm__) GMARK(5);
#endif
                // one chunk: 16 accumulator columns of this thread's row -> scale, bias, activation / residual, f16
                auto chunk = [&](const uint32_t (&r)[16], const int ch) {
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        const float4 f = *reinterpret_cast<const float4*>(&sb[col0 + ch * 16 + j]);
                        v[j] = fmaf(__uint_as_float(r[j]), f.x, f.y);
                        v[j + 1] = fmaf(__uint_as_float(r[j + 1]), f.z, f.w);
                    }
                    // both GELU forms are evaluated on f16 pairs (the output is f16 anyway)
                    const bool kHalfGelu = mode == kEpiBiasGeluErf || mode == kEpiBiasGeluTanh;
                    uint32_t hv[8];
                    if (kHalfGelu) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const __half2 x2 = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
                            const __half2 g = mode == kEpiBiasGeluErf ? gelu_erf_h2(x2) : gelu_tanh_h2(x2);
                            hv[j] = *reinterpret_cast<const uint32_t*>(&g);
                        }
                    }
                    if (!residual && ch == 0) {
                        if (lane == 0) tma_store_wait_read();
                        __syncwarp();
                    }
                    if (fast) {
                        if (residual) {
#pragma unroll
                            for (int q = 0; q < 2; ++q) {
                                const __half2* h = reinterpret_cast<const __half2*>(&res_own[ch * 2 + q]);
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const float2 f = __half22float2(h[e]);
                                    v[q * 8 + 2 * e] += f.x;
                                    v[q * 8 + 2 * e + 1] += f.y;
                                }
                            }
                        }
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            uint4 o;
                            if (kHalfGelu) {
                                *reinterpret_cast<uint4*>(slab + lane * 64 + (((ch * 2 + q) ^ ((lane >> 1) & 3)) << 4)) =
                                    make_uint4(hv[q * 4], hv[q * 4 + 1], hv[q * 4 + 2], hv[q * 4 + 3]);
                                continue;
                            }
                            __half2 h0 = __floats2half2_rn(v[q * 8 + 0], v[q * 8 + 1]);
                            __half2 h1 = __floats2half2_rn(v[q * 8 + 2], v[q * 8 + 3]);
                            __half2 h2 = __floats2half2_rn(v[q * 8 + 4], v[q * 8 + 5]);
                            __half2 h3 = __floats2half2_rn(v[q * 8 + 6], v[q * 8 + 7]);
                            o.x = *reinterpret_cast<uint32_t*>(&h0);
                            o.y = *reinterpret_cast<uint32_t*>(&h1);
                            o.z = *reinterpret_cast<uint32_t*>(&h2);
                            o.w = *reinterpret_cast<uint32_t*>(&h3);
                            *reinterpret_cast<uint4*>(slab + lane * 64 + (((ch * 2 + q) ^ ((lane >> 1) & 3)) << 4)) = o;
                        }
                    } else if (row_ok) {
                        // ragged right edge of the matrix: element-wise stores
                        const int nc = ncol0 + ch * 16;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (nc + j < p.n) {
                                float x = v[j];
                                if (kHalfGelu) {
                                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hv[j >> 1]));
                                    x = (j & 1) ? f.y : f.x;
                                }
                                if (residual) x += __half2float(res_row[nc + j]);
                                out_row[nc + j] = __float2half_rn(x);
                            }
                        }
                    }
                };
                static_assert(kSlabCols == 32, "a slab is two chunks of 16 columns");
                tmem_ld_wait16(ra);
                __syncwarp();
                tmem_ld_32x16(taddr + col0 + 16, rb);
                chunk(ra, 0);
                tmem_ld_wait16(rb);
                if (sl + 1 < kSlabs) {
                    __syncwarp();
                    tmem_ld_32x16(taddr + col0 + 32, ra);
                }
                chunk(rb, 1);
#ifdef EOSB_GEMM_TIMING
                if (tm__) GMARK(6);
#endif
                if (fast) {
                    // the slab (32 rows x 64 bytes, 16-byte chunk c of row r at c ^ ((r >> 1) & 3): the 64-byte TMA
                    // swizzle) leaves as one TMA store; rows past the end of the allocation are clipped, rows between
                    // the valid count and the allocation receive values nobody reads
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && m0 + wrow0 < p.m_alloc) tma_store_2d(&tm_out, smem_u32(slab), ncol0, m0 + wrow0);
                }
#ifdef EOSB_GEMM_TIMING
                if (tm__) GMARK(7);
#endif
            }
#ifdef EOSB_GEMM_TIMING
            if (tm__) GMARK(7);
#endif
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (kPair) mbar_arrive_cluster(ab ? acc_empty_leader1 : acc_empty_leader0); else mbar_arrive(acc_empty(ab));
            }
        }
        if (lane == 0) tma_store_wait_all();
        __syncwarp();
#ifdef EOSB_GEMM_TIMING
        GFLUSH(4);
#endif
    }

    // ---------------------------------------------------------------- teardown
    // (pair mode: no CTA may leave while its partner can still read its shared memory, arrive on
    // its barriers or use its tensor memory)
    tc_fence_before();
    if (kPair) cluster_sync_all(); else __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        if (kPair) tmem_dealloc_pair(tmem_base, kTmemCols); else tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) atomicExch(p.status, kStatusPipelineTimeout);
}

}  // namespace

#ifdef EOSB_GEMM_TIMING
extern "C" __attribute__((visibility("default"))) int eos_b200_debug_gemm_timing(long long* out16, int reset) {
    long long zero[16] = {0};
    if (cudaMemcpyFromSymbol(out16, g_gemm_timing, sizeof(zero)) != cudaSuccess) return 1;
    if (reset && cudaMemcpyToSymbol(g_gemm_timing, zero, sizeof(zero)) != cudaSuccess) return 1;
    return 0;
}
#endif

namespace {
int g_pair_clusters = -1;  // CTA pairs that can be resident at once; 0 = pair mode unavailable
bool g_pair_all = false;   // EOS_B200_GEMM_CTA_PAIR=1: every f16-weight projection runs on CTA pairs
// Shapes the pair kernel serves by default: deep projections (the operand feed per CTA drops by a third) and wide ones
// of at least the encoder's depth; measured per step at D = 768: FFN down 12.6 -> 11.8 ms, fused QKV 10.9 -> 10.4 ms,
// FFN up unchanged, attention output (K = N = 768) 4.8 -> 4.9 ms and therefore left on one CTA per tile.
bool pair_serves(int k, int n) { return g_pair_all || k >= 2048 || (n >= 2048 && k >= 768); }

cudaLaunchConfig_t pair_launch_config(int grid, cudaStream_t stream, cudaLaunchAttribute* attr) {
    attr->id = cudaLaunchAttributeClusterDimension;
    attr->val.clusterDim.x = 2;
    attr->val.clusterDim.y = 1;
    attr->val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(Cfg<false, true>::kThreads);
    cfg.dynamicSmemBytes = Cfg<false, true>::kSmemBytes;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cfg;
}
}  // namespace

std::string gemm_global_init() {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<true, false, kEpiBias>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg<true, false>::kSmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_tc_kernel<true, false, kEpiBiasGeluErf>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<true, false>::kSmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_tc_kernel<true, false, kEpiBiasResidual>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<true, false>::kSmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_tc_kernel<true, false, kEpiBiasGeluTanh>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<true, false>::kSmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_tc_kernel<false, false, kEpiBias>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<false, false>::kSmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_tc_kernel<false, false, kEpiBiasGeluErf>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<false, false>::kSmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_tc_kernel<false, false, kEpiBiasResidual>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<false, false>::kSmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_tc_kernel<false, false, kEpiBiasGeluTanh>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<false, false>::kSmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_tc_kernel<false, true, kEpiBias>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<false, true>::kSmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_tc_kernel<false, true, kEpiBiasGeluErf>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<false, true>::kSmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_tc_kernel<false, true, kEpiBiasResidual>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<false, true>::kSmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_tc_kernel<false, true, kEpiBiasGeluTanh>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<false, true>::kSmemBytes);
    if (e != cudaSuccess) return std::string("cudaFuncSetAttribute(gemm_tc_kernel): ") + cudaGetErrorString(e);
    if (g_pair_clusters < 0) {
        g_pair_clusters = 0;
        const char* on = getenv("EOS_B200_GEMM_CTA_PAIR");
        const bool off = on != nullptr && on[0] == '0';
        if (on != nullptr && on[0] != '\0' && !off) g_pair_all = true;
        if (!off) {
            int dev = 0, sms = 0, clusters = 0;
            cudaLaunchAttribute attr;
            if (cudaGetDevice(&dev) == cudaSuccess &&
                cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms >= 2) {
                cudaLaunchConfig_t cfg = pair_launch_config(sms & ~1, nullptr, &attr);
                if (cudaOccupancyMaxActiveClusters(&clusters, gemm_tc_kernel<false, true, kEpiBiasResidual>, &cfg) == cudaSuccess)
                    g_pair_clusters = clusters;
                else
                    (void)cudaGetLastError();
            }
        }
        if (getenv("EOS_B200_DEBUG") != nullptr) fprintf(stderr, "eos_b200: resident CTA pairs for the GEMM: %d\n", g_pair_clusters);
    }
    return "";
}

std::string gemm_make_plan(GemmPlan* plan, const __half* a, int lda, const void* w, int ldw, bool b_int8,
                           const GemmParams& params, int sm_count) {
    if (params.m_alloc <= 0 || params.n <= 0 || params.k <= 0) return "gemm: dimensions must be positive";
    if (params.ldo % 8 != 0) return "gemm: output row stride must be a multiple of 8 elements";
    if (params.mode == kEpiBiasResidual && (params.residual == nullptr || params.ldr % 8 != 0))
        return "gemm: residual epilogue needs a residual pointer with a row stride that is a multiple of 8";
    const bool pair = !b_int8 && g_pair_clusters > 0 && pair_serves(params.k, params.n);
    std::string err = encode_2d(&plan->tm_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a, (uint64_t)params.k,
                                (uint64_t)params.m_alloc, (uint64_t)lda * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!err.empty()) return "gemm A: " + err;
    if (b_int8)
        err = encode_2d(&plan->tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, w, (uint64_t)params.k, (uint64_t)params.n,
                        (uint64_t)ldw, BK, BN, CU_TENSOR_MAP_SWIZZLE_NONE);
    else
        err = encode_2d(&plan->tm_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, w, (uint64_t)params.k, (uint64_t)params.n,
                        (uint64_t)ldw * 2, BK, pair ? BN / 2 : BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!err.empty()) return "gemm W: " + err;
    err = encode_2d(&plan->tm_out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, params.out, (uint64_t)params.n, (uint64_t)params.m_alloc,
                    (uint64_t)params.ldo * 2, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B);
    if (!err.empty()) return "gemm out: " + err;
    plan->p = params;
    plan->b_int8 = b_int8;
    plan->pair = pair;
    const int tile_m = pair ? 2 * BM : BM;
    const int m_tiles = (params.m_alloc + tile_m - 1) / tile_m;
    const int n_tiles = (params.n + BN - 1) / BN;
    const long long tiles = (long long)m_tiles * n_tiles;
    if (pair) {
        int workers = sm_count / 2 < g_pair_clusters ? sm_count / 2 : g_pair_clusters;
        plan->grid = 2 * (int)(tiles < workers ? tiles : workers);
    } else {
        plan->grid = (int)(tiles < sm_count ? tiles : sm_count);
    }
    return "";
}

void gemm_launch(const GemmPlan& plan, cudaStream_t stream) {
    if (plan.pair) {
        cudaLaunchAttribute attr;
        cudaLaunchConfig_t cfg = pair_launch_config(plan.grid, stream, &attr);
        switch (plan.p.mode) {
            case kEpiBiasGeluErf:
                cudaLaunchKernelEx(&cfg, gemm_tc_kernel<false, true, kEpiBiasGeluErf>, plan.tm_a, plan.tm_b, plan.tm_out, plan.p);
                break;
            case kEpiBiasResidual:
                cudaLaunchKernelEx(&cfg, gemm_tc_kernel<false, true, kEpiBiasResidual>, plan.tm_a, plan.tm_b, plan.tm_out, plan.p);
                break;
            case kEpiBiasGeluTanh:
                cudaLaunchKernelEx(&cfg, gemm_tc_kernel<false, true, kEpiBiasGeluTanh>, plan.tm_a, plan.tm_b, plan.tm_out, plan.p);
                break;
            default:
                cudaLaunchKernelEx(&cfg, gemm_tc_kernel<false, true, kEpiBias>, plan.tm_a, plan.tm_b, plan.tm_out, plan.p);
                break;
        }
    } else if (plan.b_int8) {
        constexpr int kT = Cfg<true, false>::kThreads;
        constexpr uint32_t kS = Cfg<true, false>::kSmemBytes;
        switch (plan.p.mode) {
            case kEpiBiasGeluErf:
                gemm_tc_kernel<true, false, kEpiBiasGeluErf><<<plan.grid, kT, kS, stream>>>(plan.tm_a, plan.tm_b, plan.tm_out, plan.p);
                break;
            case kEpiBiasResidual:
                gemm_tc_kernel<true, false, kEpiBiasResidual><<<plan.grid, kT, kS, stream>>>(plan.tm_a, plan.tm_b, plan.tm_out, plan.p);
                break;
            case kEpiBiasGeluTanh:
                gemm_tc_kernel<true, false, kEpiBiasGeluTanh><<<plan.grid, kT, kS, stream>>>(plan.tm_a, plan.tm_b, plan.tm_out, plan.p);
                break;
            default:
                gemm_tc_kernel<true, false, kEpiBias><<<plan.grid, kT, kS, stream>>>(plan.tm_a, plan.tm_b, plan.tm_out, plan.p);
                break;
        }
    } else {
        constexpr int kT = Cfg<false, false>::kThreads;
        constexpr uint32_t kS = Cfg<false, false>::kSmemBytes;
        switch (plan.p.mode) {
            case kEpiBiasGeluErf:
                gemm_tc_kernel<false, false, kEpiBiasGeluErf><<<plan.grid, kT, kS, stream>>>(plan.tm_a, plan.tm_b, plan.tm_out, plan.p);
                break;
            case kEpiBiasResidual:
                gemm_tc_kernel<false, false, kEpiBiasResidual><<<plan.grid, kT, kS, stream>>>(plan.tm_a, plan.tm_b, plan.tm_out, plan.p);
                break;
            case kEpiBiasGeluTanh:
                gemm_tc_kernel<false, false, kEpiBiasGeluTanh><<<plan.grid, kT, kS, stream>>>(plan.tm_a, plan.tm_b, plan.tm_out, plan.p);
                break;
            default:
                gemm_tc_kernel<false, false, kEpiBias><<<plan.grid, kT, kS, stream>>>(plan.tm_a, plan.tm_b, plan.tm_out, plan.p);
                break;
        }
    }
}

}  // namespace eosb
