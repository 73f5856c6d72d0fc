// Batched TurboQuant scoring on the tensor cores, 256 queries per launch: the operand roles of
// turboquant_tc.cu swapped.  There the 128 queries are the MMA's M rows and a tile of 256 expanded documents
// its N columns, and the pace is set by the warps that expand the codes; here a tile of 128 documents is the
// A operand (M = 128, expanded into shared memory exactly as before) and 256 queries are the B operand
// (N = 256, 32 KB per k-block by TMA), so one expanded code meets twice as many queries and the expanders
// have half the work per multiply-add.  Same operator as the other scoring kernels: the reference's per-query
// loop (runtime/retrieval_turboquant.go ScoreTurboQuant* / turboquant_quantized_vector.go), for batches.
//
// One persistent CTA per SM walks the shard in tiles of 128 documents:
//   warp 0      TMA producer: rotated f16 queries, 256 rows x 64 coordinates per k-block (128B swizzle), 4-stage ring.
//   warp 1      MMA issuer: tcgen05.mma M128 x N256 x K16, two 256-column accumulators in tensor memory.
//   warp 2      allocates / frees tensor memory.
//   warps 4-11  expanders: one 16-document group each per k-block (4-stage ring of 16 KB).
//   warps 12-19 epilogue: a thread owns one document (its TMEM lane) and 128 of the 256 queries: score =
//               accumulator x its document's norm against the queries' thresholds in shared memory; the rare
//               survivors go to the CTA's list of that query in global memory (slot from a shared-memory
//               counter).  Between tiles thread i of the epilogue looks after query i: it picks up thresholds
//               other CTAs published, and a list that the next tile could overflow is cut to its k best by the
//               query's warp (bitonic sort in shared memory), the k-th key published with atomicMax.
// Seed mode (seed_scores != null): every score is written to seed_scores[query][row] instead.
// Every mbarrier wait is bounded (common.cuh: mbar_wait): on a timeout all roles leave their loops,
// tensor memory is freed and the status word is set.
#include "common.cuh"
#include "tma_util.cuh"
#include "turboquant.cuh"
#include "turboquant_dev.cuh"

namespace eosb {

namespace {

constexpr int TD = kTqTc256Docs;     // documents per tile (MMA M)
constexpr int TQ = kTqTc256Queries;  // queries per launch (MMA N)
constexpr int TK = 64;               // coordinates per k-block
constexpr int kStQ = 4;              // query ring (32 KB per stage)
constexpr int kStD = 4;              // expanded-document ring (16 KB per stage)
constexpr uint32_t kBytesQ = TQ * TK * 2;
constexpr uint32_t kBytesD = TD * TK * 2;
constexpr int kExpWarps = 8;
constexpr int kEpiWarps = 8;
constexpr int kFirstExp = 4;
constexpr int kFirstEpi = kFirstExp + kExpWarps;
constexpr int kThreads = (kFirstEpi + kEpiWarps) * 32;
constexpr int kTmemCols = 512;
constexpr int kCutAbove = 128;       // a list longer than this is cut before the next tile (which adds <= TD)

constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffD = kOffQ + kStQ * kBytesQ;
constexpr uint32_t kOffSort = kOffD + kStD * kBytesD;                 // 8 warps x 256 keys
constexpr uint32_t kOffTauKey = kOffSort + kEpiWarps * kSortCap * 8;  // [256] u64
constexpr uint32_t kOffTauF = kOffTauKey + TQ * 8;                    // [256] float
constexpr uint32_t kOffTauLo = kOffTauF + TQ * 4;                     // [256] float: the threshold one ulp lower
constexpr uint32_t kOffCnt = kOffTauLo + TQ * 4;                      // [256] int
constexpr uint32_t kOffBars = kOffCnt + TQ * 4;
constexpr uint32_t kNumBars = 2 * kStQ + 2 * kStD + 4;
constexpr uint32_t kOffMisc = kOffBars + kNumBars * 8;
constexpr uint32_t kSmemBytes = kOffMisc + 16 + 1024;

__device__ __forceinline__ float max3f(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

static_assert(TD / kTqDocsPerTile == kExpWarps, "one 16-document group per expander warp");
static_assert(kTqTcSegLen == kSortCap && kTqTcSegLen >= kCutAbove + TD && kTqMaxK <= kCutAbove, "list capacity");
static_assert(kEpiWarps * 32 == TQ, "one epilogue thread looks after one query");

__global__ void __launch_bounds__(kThreads, 1) tq_score_tc256_kernel(const __grid_constant__ CUtensorMap tm_q, TqTcArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const uint32_t bar0 = base + kOffBars;
    auto full_q = [&](int s) { return bar0 + 8u * s; };
    auto empty_q = [&](int s) { return bar0 + 8u * (kStQ + s); };
    auto full_d = [&](int s) { return bar0 + 8u * (2 * kStQ + s); };
    auto empty_d = [&](int s) { return bar0 + 8u * (2 * kStQ + kStD + s); };
    auto acc_full = [&](int s) { return bar0 + 8u * (2 * kStQ + 2 * kStD + s); };
    auto acc_empty = [&](int s) { return bar0 + 8u * (2 * kStQ + 2 * kStD + 2 + s); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + kOffMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + kOffMisc + 4);
    // set by an epilogue warp whose wait ran out, read by all epilogue warps right after their next common
    // barrier: they leave the tile loop together, so no named barrier is left waiting for warps that have gone
    volatile int* epi_stop = reinterpret_cast<volatile int*>(sm + kOffMisc + 8);

    const int chunks = (a.dim + kTqChunkCoords - 1) / kTqChunkCoords;
    const int num_kb = chunks * 2;
    const long long n_tiles = (a.n_docs + TD - 1) / TD;
    const long long n_tiles16 = (a.n_docs + kTqDocsPerTile - 1) / kTqDocsPerTile;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        *epi_stop = 0;
        for (int s = 0; s < kStQ; ++s) {
            mbar_init(full_q(s), 1);
            mbar_init(empty_q(s), 1);
        }
        for (int s = 0; s < kStD; ++s) {
            mbar_init(full_d(s), kExpWarps);
            mbar_init(empty_d(s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(acc_full(s), 1);
            mbar_init(acc_empty(s), kEpiWarps);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tm_q);
    }
    if (warp == 2) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (queries)
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % kStQ;
                    const uint32_t ph = (it / kStQ) & 1u;
                    if (!mbar_wait(empty_q(s), ph ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(full_q(s), kBytesQ);
                    tma_load_2d(base + kOffQ + s * kBytesQ, &tm_q, kb * TK, a.q_row0, full_q(s));
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (A = documents, B = queries)
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f16(TD, TQ);
            uint32_t it = 0, t = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++t) {
                const uint32_t ab = t & 1u;
                const uint32_t aph = (t >> 1) & 1u;
                if (!mbar_wait(acc_empty(ab), aph ^ 1u, abort_flag)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + ab * TQ;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % kStQ;
                    const int c = it % kStD;
                    if (!mbar_wait(full_q(s), (it / kStQ) & 1u, abort_flag) ||
                        !mbar_wait(full_d(c), (it / kStD) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t q_lo = umma_desc_sw128_lo(base + kOffQ + s * kBytesQ);
                    const uint32_t d_lo = umma_desc_sw128_lo(base + kOffD + c * kBytesD);
#pragma unroll
                    for (int k = 0; k < TK / 16; ++k)
                        umma_f16_split(d_tmem, d_lo + k * 2, kDescSw128Hi, q_lo + k * 2, kDescSw128Hi, idesc,
                                       (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(empty_q(s));
                    umma_commit(empty_d(c));
                }
                if (ok) umma_commit(acc_full(ab));
            }
        }
        __syncwarp();
    } else if (warp >= kFirstExp && warp < kFirstEpi) {
        // ------------------------------------------------------------ expanders (4-bit codes -> f16 operand tile)
        const int ew = warp - kFirstExp;          // owns the 16-document group ew of the tile
        const int g = lane & 7, t = lane >> 3;    // document g / g + 8 of the group, code-word column t
        const uint8_t* tiles = a.tiles;
        const size_t group_bytes = (size_t)chunks * 1024;
        const uint32_t lane_off = (uint32_t)(g * 4 + t) * 32;
        uint32_t cur[8], nxt[8];
        auto fetch = [&](long long tile, int c, uint32_t (&dst)[8]) {
            const long long grp = tile * (TD / kTqDocsPerTile) + ew;
            if (tile < n_tiles && grp < n_tiles16) {
                ld_global_v8(tiles + (size_t)grp * group_bytes + (size_t)c * 1024 + lane_off, dst);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) dst[i] = 0;
            }
        };
        uint32_t it = 0;
        bool ok = true;
        if ((long long)blockIdx.x < n_tiles) fetch(blockIdx.x, 0, cur);
        for (long long tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
            for (int c = 0; ok && c < chunks; ++c) {
                if (c + 1 < chunks) fetch(tile, c + 1, nxt);
                else fetch(tile + gridDim.x, 0, nxt);
#pragma unroll
                for (int half = 0; half < 2; ++half, ++it) {
                    const int s = it % kStD;
                    if (!mbar_wait(empty_d(s), ((it / kStD) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint8_t* dst = sm + kOffD + s * kBytesD;
#pragma unroll
                    for (int dh = 0; dh < 2; ++dh) {
                        // tile row of the document = 16 ew + 8 dh + g; row & 7 == g for both halves
                        uint8_t* row = dst + (ew * 2 + dh) * 1024 + g * 128;
#pragma unroll
                        for (int wi = 0; wi < 2; ++wi) {
                            uint32_t v[4];
                            dequant8(cur[dh * 4 + half * 2 + wi], a.mag_hi[0], a.mag_hi[1], a.mag_lo[0], a.mag_lo[1], v);
                            const int j = t + 4 * wi;
                            *reinterpret_cast<uint4*>(row + ((j ^ g) << 4)) = make_uint4(v[0], v[1], v[2], v[3]);
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full_d(s));
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) cur[i] = nxt[i];
            }
        }
    } else if (warp >= kFirstEpi) {
        // ------------------------------------------------------------ epilogue: thresholds and candidate lists
        const int ew = warp - kFirstEpi;
        const int etid = threadIdx.x - kFirstEpi * 32;  // 0..255: the query this thread looks after between tiles
        const int quarter = warp & 3;                   // TMEM lane quarter (documents 32 quarter .. + 31 of the tile)
        const int epart = ew >> 2;                      // queries 128 epart .. + 127
        const int n_segs = (int)gridDim.x;              // one list per CTA and query
        u64* const cand = reinterpret_cast<u64*>(a.cand_keys);
        u64* tau_key_s = reinterpret_cast<u64*>(sm + kOffTauKey);
        float* tau_f_s = reinterpret_cast<float*>(sm + kOffTauF);
        // The screening test of a tile is one fused multiply-add per score, accumulator x norm - threshold, and a
        // running maximum: its sign is the sign of the exact difference, while the score that is kept is the rounded
        // product.  A product that rounds up onto the threshold would be missed, so the screen uses the threshold one
        // ulp lower; what it lets through is tested again on the rounded score.
        float* tau_lo_s = reinterpret_cast<float*>(sm + kOffTauLo);
        auto set_tau_f = [&](int q, float t) {
            tau_f_s[q] = t;
            tau_lo_s[q] = (t == -INFINITY || t == INFINITY) ? t : nextafterf(t, -INFINITY);
        };
        int* cnt_s = reinterpret_cast<int*>(sm + kOffCnt);
        u64* sortbuf = reinterpret_cast<u64*>(sm + kOffSort) + ew * kSortCap;
        volatile u64* shared_tau = a.shared_tau;
        const bool q_live = etid < a.q_valid;
        tau_key_s[etid] = q_live ? 0ull : ~0ull;
        set_tau_f(etid, q_live ? -INFINITY : INFINITY);
        cnt_s[etid] = 0;
        const float kNoDoc = __int_as_float(0x7fc00000);  // NaN: a missing document never passes a comparison
        auto fetch_norm = [&](long long tile) {
            const long long doc = tile * TD + quarter * 32 + lane;
            return (tile < n_tiles && doc < a.n_docs) ? __ldg(a.norms + doc) : kNoDoc;
        };
        float norm_next = fetch_norm(blockIdx.x);
        uint32_t t = 0;
        bool stopped = false;
        for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++t) {
            const uint32_t ab = t & 1u;
            const uint32_t aph = (t >> 1) & 1u;
            const float norm = norm_next;
            norm_next = fetch_norm(tile + gridDim.x);
            // every append of the previous tile is done (and the initial values above are written)
            named_bar_sync(1, kEpiWarps * 32);
            if (*epi_stop != 0) {
                stopped = true;
                break;
            }
            // this thread's query: thresholds other CTAs published; a list the coming tile could overflow is cut
            if (q_live) {
                const u64 pub = shared_tau[etid];
                if (pub > tau_key_s[etid]) {
                    tau_key_s[etid] = pub;
                    set_tau_f(etid, ordered_to_float((uint32_t)(pub >> 32)));
                }
            }
            const int my_cnt = cnt_s[etid];
            unsigned need = __ballot_sync(0xffffffffu, my_cnt > kCutAbove);
            while (need != 0) {
                const int src = __ffs(need) - 1;
                need &= need - 1;
                const int n = __shfl_sync(0xffffffffu, my_cnt, src);
                u64* lst = cand + ((size_t)(ew * 32 + src) * n_segs + blockIdx.x) * kTqTcSegLen;
                __syncwarp();
                for (int i = lane; i < n; i += 32) sortbuf[i] = lst[i];
                warp_sort_desc(sortbuf, n, lane);
                for (int i = lane; i < a.k; i += 32) lst[i] = sortbuf[i];
                const u64 kth = sortbuf[a.k - 1];
                __syncwarp();
                if (lane == src) {
                    cnt_s[etid] = a.k;
                    if (kth > tau_key_s[etid]) {
                        tau_key_s[etid] = kth;
                        set_tau_f(etid, ordered_to_float((uint32_t)(kth >> 32)));
                    }
                    atomicMax(const_cast<u64*>(a.shared_tau) + etid, kth);
                }
            }
            named_bar_sync(2, kEpiWarps * 32);  // thresholds and counters of all 256 queries are in place
            if (!__all_sync(0xffffffffu, mbar_wait(acc_full(ab), aph, abort_flag))) {
                *epi_stop = 1;
                continue;   // to the next common barrier, where every epilogue warp sees the flag
            }
            tc_fence_after();

            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + ab * TQ + epart * (TQ / 2);
            const long long row = tile * TD + quarter * 32 + lane;        // this thread's document
            const uint32_t doc_id = a.id_base + (uint32_t)row;
            const int q0 = epart * (TQ / 2);
            auto chunk = [&](const uint32_t (&r)[16], const int c0) {
                if (a.seed_scores != nullptr) {
                    // seed mode: for one query the 32 lanes hold 32 consecutive rows
                    if (row < a.n_docs) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            a.seed_scores[(size_t)(q0 + c0 + j) * a.seed_stride + row] = __uint_as_float(r[j]) * norm;
                    }
                    return;
                }
                float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                    const float4 tl = *reinterpret_cast<const float4*>(tau_lo_s + q0 + c0 + j);
                    m0 = max3f(m0, fmaf(__uint_as_float(r[j]), norm, -tl.x), fmaf(__uint_as_float(r[j + 1]), norm, -tl.y));
                    m1 = max3f(m1, fmaf(__uint_as_float(r[j + 2]), norm, -tl.z), fmaf(__uint_as_float(r[j + 3]), norm, -tl.w));
                }
                if (fmaxf(m0, m1) >= 0.0f) {   // a missing document's NaN never gets here: max ignores it
                    float tf[16];
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        const float4 tv = *reinterpret_cast<const float4*>(tau_f_s + q0 + c0 + j);
                        tf[j] = tv.x;
                        tf[j + 1] = tv.y;
                        tf[j + 2] = tv.z;
                        tf[j + 3] = tv.w;
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float sc = __uint_as_float(r[j]) * norm;
                        const int q = q0 + c0 + j;
                        if (sc >= tf[j]) {
                            const u64 key = make_key(sc, doc_id);
                            if (key > tau_key_s[q]) {
                                const int pos = atomicAdd(&cnt_s[q], 1);  // <= 128 before the tile, <= 128 + TD after
                                cand[((size_t)q * n_segs + blockIdx.x) * kTqTcSegLen + pos] = key;
                            }
                        }
                    }
                }
            };
            uint32_t ra[16], rb[16];
            __syncwarp();
            tmem_ld_32x16(taddr, ra);
#pragma unroll 1
            for (int c0 = 0; c0 < TQ / 2; c0 += 32) {
                tmem_ld_wait16(ra);
                __syncwarp();
                tmem_ld_32x16(taddr + c0 + 16, rb);
                chunk(ra, c0);
                tmem_ld_wait16(rb);
                if (c0 + 32 < TQ / 2) {
                    __syncwarp();
                    tmem_ld_32x16(taddr + c0 + 32, ra);
                }
                chunk(rb, c0 + 16);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(ab));
        }
        if (!stopped) named_bar_sync(1, kEpiWarps * 32);
        a.cand_count[(size_t)etid * n_segs + blockIdx.x] = cnt_s[etid];
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_flag != 0 && a.status != nullptr) atomicExch(a.status, kStatusPipelineTimeout);
}

}  // namespace

cudaError_t tq_tc256_init() {
    return cudaFuncSetAttribute(tq_score_tc256_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
}

std::string tq_tc256_make_query_map(CUtensorMap* tm, const __half* qperm, int padded_dim, int rows) {
    return encode_2d(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, qperm, (uint64_t)padded_dim, (uint64_t)rows,
                     (uint64_t)padded_dim * 2, TK, TQ, CU_TENSOR_MAP_SWIZZLE_128B);
}

void launch_tq_score_tc256(const CUtensorMap& tm_q, const TqTcArgs& a, int grid, cudaStream_t stream) {
    tq_score_tc256_kernel<<<grid, kThreads, kSmemBytes, stream>>>(tm_q, a);
}

}  // namespace eosb
