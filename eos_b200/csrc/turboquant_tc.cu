// Batched TurboQuant scoring on the 5th-generation tensor cores: one launch scores 128 queries
// against every packed vector of the shard and keeps, per query, the candidates of the exact top-k.
//
// The streaming scan (turboquant.cu) reads the 4-bit codes once per 8 queries and is bound by the
// integer work of expanding them; with hundreds of queries in a batch the expansion is better
// amortised: here a 256-document x 64-coordinate block of codes is expanded once into shared memory
// (f16, in the K-major 128B-swizzled layout tcgen05.mma reads) and multiplied by 128 queries, so the
// codes are read once per 128 queries and the expansion costs 1/16 of the streaming kernel's per score.
// It serves the same operator as the streaming scan, the reference's per-query scoring loop
// (runtime/retrieval_turboquant.go ScoreTurboQuant* / turboquant_quantized_vector.go), for batches.
//
// One persistent CTA per SM walks the shard in tiles of 256 documents (tile = blockIdx.x, += gridDim.x):
//   warp 0      TMA producer: the rotated f16 queries, 128 rows x 64 coordinates per k-block (128B swizzle),
//               4-stage ring.  The coordinates of a k-block are stored in the order the code words hold them
//               (launch_tq_prepare writes that permuted copy), so a code word expands to 16 contiguous bytes.
//   warp 1      MMA issuer: tcgen05.mma M = 128 (queries) x N = 256 (documents) x K = 16, f32 accumulator in
//               tensor memory, two accumulators so that the epilogue of a tile overlaps the next tile.
//   warp 2      allocates / frees tensor memory.
//   warps 4-11  expanders: each lane loads 32 bytes of a scan tile per 128 coordinates (two documents x 32
//               codes, one chunk ahead in registers), expands the nibbles with byte permutes and writes
//               16-byte pieces of the operand tile (4-stage ring of 32 KB).
//   warps 12-19 epilogue: a thread owns one query (its TMEM lane) and 128 of the tile's documents: score =
//               accumulator x document norm, compared with the query's pruning threshold in a register;
//               the rare survivors are appended to the thread's own candidate list in global memory
//               (no atomics).  A list that could overflow during the next tile is cut to its k best by the
//               whole warp (bitonic sort in shared memory) and the k-th key is published with atomicMax as
//               the query's threshold for every CTA.
// Thresholds start from a sample: the caller first runs this kernel in its seed mode over the first rows of
// the shard (one tile per CTA; the epilogue writes every score, 32 bytes per store, instead of keeping lists)
// and takes each query's k-th best sample score, so in the steady state a few documents per thousand reach a list.
//
// Two variants of the same kernel.  kQInTmem = false is the one described above and the one used.  kQInTmem = true
// (padded dimension <= 768, opt-in) keeps the 128 queries in tensor memory for the whole launch (dim / 2 columns,
// written once with tcgen05.st) and issues tcgen05.mma with A from tensor memory, so that no query tile crosses
// shared memory.  Tensor memory then has room for one 128-column accumulator: a tile is 128 documents, its epilogue
// does not overlap the next tile's MMAs and every document costs twice the ring hand-offs; measured 0.42 ms per
// launch over 1.25 M rows against 0.26 ms, which shows that the expanders and the hand-offs, not the shared-memory
// bandwidth, set the pace.
// Every mbarrier wait is bounded (common.cuh: mbar_wait): on a timeout all roles leave their loops,
// tensor memory is freed and the status word is set.
#include "common.cuh"
#include "tma_util.cuh"
#include "turboquant.cuh"
#include "turboquant_dev.cuh"

namespace eosb {

namespace {

constexpr int TQ = kTqTcQueries;    // queries per launch (MMA M)
constexpr int TK = 64;              // coordinates per k-block
constexpr int kStQ = 4;             // query ring (shared-memory variant)
constexpr uint32_t kBytesQ = TQ * TK * 2;
constexpr int kEpiWarps = 8;
constexpr int kFirstExp = 4;
constexpr int kTmemCols = 512;
constexpr int kCutAbove = 128;      // a list longer than this is cut before the next tile (which adds <= 128)
constexpr int kQTmemCol = 128;      // first tensor-memory column of the resident queries (after the accumulator)

template <bool kQInTmem>
struct Cfg {
    static constexpr int TD = kQInTmem ? kTqTcDocsQ : kTqTcDocs;   // documents per tile (MMA N)
    static constexpr int kAccBufs = kQInTmem ? 1 : 2;
    static constexpr int kStD = kQInTmem ? 8 : 4;                  // expanded-document ring
    static constexpr uint32_t kBytesD = TD * TK * 2;
    static constexpr int kExpWarps = 8;
    static constexpr int kFirstEpi = kFirstExp + kExpWarps;
    static constexpr int kThreads = (kFirstEpi + kEpiWarps) * 32;
    static constexpr int kGroups = TD / kTqDocsPerTile / kExpWarps;  // 16-document groups per expander warp
    static constexpr uint32_t kOffQ = 0;
    static constexpr uint32_t kOffD = kOffQ + (kQInTmem ? 0 : kStQ * kBytesQ);
    static constexpr uint32_t kOffNorm = kOffD + kStD * kBytesD;            // 2 x TD floats
    static constexpr uint32_t kOffSort = kOffNorm + 2 * TD * 4;             // 8 warps x 256 keys
    static constexpr uint32_t kOffBars = kOffSort + kEpiWarps * kSortCap * 8;
    static constexpr uint32_t kNumBars = 2 * kStQ + 2 * kStD + 4;
    static constexpr uint32_t kOffMisc = kOffBars + kNumBars * 8;
    static constexpr uint32_t kSmemBytes = kOffMisc + 16 + 1024;
    static_assert(kGroups >= 1 && TD / 2 <= 128 && kTqTcSegLen >= kCutAbove + TD / 2, "tile shape / list capacity");
};

static_assert(kTqTcSegLen == kSortCap, "a list is sorted in one piece");
static_assert(kTqMaxK <= kCutAbove, "a cut keeps k <= 128 keys");

template <bool kQInTmem>
__global__ void __launch_bounds__(Cfg<kQInTmem>::kThreads, 1) tq_score_tc_kernel(const __grid_constant__ CUtensorMap tm_q, TqTcArgs a) {
    using C = Cfg<kQInTmem>;
    constexpr int TD = C::TD;
    constexpr int kStD = C::kStD;
    constexpr int kExpWarps = C::kExpWarps, kFirstEpi = C::kFirstEpi;
    constexpr uint32_t kBytesD = C::kBytesD;
    constexpr uint32_t kOffQ = C::kOffQ, kOffD = C::kOffD, kOffNorm = C::kOffNorm, kOffSort = C::kOffSort;
    constexpr uint32_t kOffBars = C::kOffBars, kOffMisc = C::kOffMisc;
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
    // barrier: they leave the tile loop together, so the named barrier is never left waiting for warps that have gone
    volatile int* epi_stop = reinterpret_cast<volatile int*>(sm + kOffMisc + 8);

    const int chunks = (a.dim + kTqChunkCoords - 1) / kTqChunkCoords;
    const int num_kb = chunks * 2;
    // up to 256 coordinates the launch's queries fit the query ring and are loaded once instead of once per tile
    const bool q_resident = !kQInTmem && num_kb <= kStQ;
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
        if (!kQInTmem) tma_prefetch_desc(&tm_q);
    }
    if (warp == 2) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (kQInTmem) {
        // the launch's 128 queries move into tensor memory once: lane = query, column kQTmemCol + w = the w-th
        // 32-bit word (two consecutive f16 coordinates) of its permuted row
        if (warp >= kFirstEpi && warp < kFirstEpi + 4) {
            const int quarter = warp & 3;
            const uint4* src = reinterpret_cast<const uint4*>(a.qperm + (size_t)(a.q_row0 + quarter * 32 + lane) * (num_kb * TK));
            for (int kb = 0; kb < num_kb; ++kb) {
                uint32_t r[32];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint4 v = __ldg(src + kb * 8 + i);
                    r[4 * i] = v.x;
                    r[4 * i + 1] = v.y;
                    r[4 * i + 2] = v.z;
                    r[4 * i + 3] = v.w;
                }
                tmem_st_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + kQTmemCol + kb * 32, r);
            }
            tmem_st_wait();
        }
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
    }

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (queries; shared-memory variant)
        if (!kQInTmem && lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            if (q_resident) {
                // the whole query block fits the ring: it is loaded once and stays (stage = k-block)
                if ((long long)blockIdx.x < n_tiles) {
                    for (int kb = 0; kb < num_kb; ++kb) {
                        mbar_arrive_expect_tx(full_q(kb), kBytesQ);
                        tma_load_2d(base + kOffQ + kb * kBytesQ, &tm_q, kb * TK, a.q_row0, full_q(kb));
                    }
                }
                ok = false;
            }
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
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f16(TQ, TD);
            uint32_t it = 0, t = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++t) {
                const uint32_t ab = t % C::kAccBufs;
                const uint32_t aph = (t / C::kAccBufs) & 1u;
                if (!mbar_wait(acc_empty(ab), aph ^ 1u, abort_flag)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + ab * TD;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = q_resident ? kb : (int)(it % kStQ);
                    const int c = it % kStD;
                    if ((!kQInTmem && !mbar_wait(full_q(s), q_resident ? 0u : ((it / kStQ) & 1u), abort_flag)) ||
                        !mbar_wait(full_d(c), (it / kStD) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t q_lo = umma_desc_sw128_lo(base + kOffQ + s * kBytesQ);
                    const uint32_t d_lo = umma_desc_sw128_lo(base + kOffD + c * kBytesD);
#pragma unroll
                    for (int k = 0; k < TK / 16; ++k) {
                        if (kQInTmem)
                            umma_f16_tmem_a(d_tmem, tmem_base + kQTmemCol + kb * 32 + k * 8, d_lo + k * 2, kDescSw128Hi, idesc,
                                            (kb > 0 || k > 0) ? 1u : 0u);
                        else
                            umma_f16_split(d_tmem, q_lo + k * 2, kDescSw128Hi, d_lo + k * 2, kDescSw128Hi, idesc,
                                           (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    if (!kQInTmem && !q_resident) umma_commit(empty_q(s));
                    umma_commit(empty_d(c));
                }
                if (ok) umma_commit(acc_full(ab));
            }
        }
        __syncwarp();
    } else if (warp >= kFirstExp && warp < kFirstEpi) {
        // ------------------------------------------------------------ expanders (4-bit codes -> f16 operand tile)
        constexpr int G = C::kGroups;              // 16-document groups per warp
        const int ew = warp - kFirstExp;          // owns the groups G ew .. G ew + G - 1 of the tile
        const int g = lane & 7, t = lane >> 3;    // document g / g + 8 of the group, code-word column t
        const uint8_t* tiles = a.tiles;
        const size_t group_bytes = (size_t)chunks * 1024;
        const uint32_t lane_off = (uint32_t)(g * 4 + t) * 32;
        uint32_t cur[G][8], nxt[G][8];
        auto fetch = [&](long long tile, int c, uint32_t (&dst)[G][8]) {
#pragma unroll
            for (int u = 0; u < G; ++u) {
                const long long grp = tile * (TD / kTqDocsPerTile) + ew * G + u;
                if (tile < n_tiles && grp < n_tiles16) {
                    ld_global_v8(tiles + (size_t)grp * group_bytes + (size_t)c * 1024 + lane_off, dst[u]);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) dst[u][i] = 0;
                }
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
                    for (int u = 0; u < G; ++u) {
#pragma unroll
                        for (int dh = 0; dh < 2; ++dh) {
                            // tile row of the document; row & 7 == g for both halves
                            uint8_t* row = dst + ((ew * G + u) * 2 + dh) * 1024 + g * 128;
#pragma unroll
                            for (int wi = 0; wi < 2; ++wi) {
                                uint32_t v[4];
                                dequant8(cur[u][dh * 4 + half * 2 + wi], a.mag_hi[0], a.mag_hi[1], a.mag_lo[0], a.mag_lo[1],
                                         v);
                                const int j = t + 4 * wi;
                                *reinterpret_cast<uint4*>(row + ((j ^ g) << 4)) = make_uint4(v[0], v[1], v[2], v[3]);
                            }
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full_d(s));
                }
#pragma unroll
                for (int u = 0; u < G; ++u)
#pragma unroll
                    for (int i = 0; i < 8; ++i) cur[u][i] = nxt[u][i];
            }
        }
    } else if (warp >= kFirstEpi) {
        // ------------------------------------------------------------ epilogue: thresholds and candidate lists
        const int ew = warp - kFirstEpi;
        const int etid = threadIdx.x - kFirstEpi * 32;  // 0..255
        const int quarter = warp & 3;                   // TMEM lane quarter this warp may read
        const int epart = ew >> 2;                      // which 128 documents of the tile
        const int qrow = quarter * 32 + lane;           // this thread's query inside the launch
        const int seg = (int)blockIdx.x * 2 + epart;
        const int n_segs = (int)gridDim.x * 2;
        u64* const cand = reinterpret_cast<u64*>(a.cand_keys);
        // MaxSim mode: the first thread of every group of maxsim_group query vectors owns the query's list
        const bool maxsim = a.maxsim_children > 0;
        const int group = maxsim ? a.maxsim_group : 1;
        const bool owner = (lane & (group - 1)) == 0;
        const int qtau = maxsim ? qrow / group : qrow;                      // threshold index of this thread
        const int qlist = maxsim ? a.maxsim_list_base + qtau : qrow;       // list / count index of this thread
        u64* my_list = cand + ((size_t)qlist * n_segs + seg) * kTqTcSegLen;
        u64* sortbuf = reinterpret_cast<u64*>(sm + kOffSort) + ew * kSortCap;
        float* norm_s = reinterpret_cast<float*>(sm + kOffNorm);
        volatile u64* shared_tau = a.shared_tau;
        const bool q_live = qrow < a.q_valid && owner;
        u64 tau_key = q_live ? 0ull : ~0ull;
        float tau_f = q_live ? -INFINITY : INFINITY;
        int cnt = 0;
        auto raise_tau = [&](u64 key) {
            if (key > tau_key) {
                tau_key = key;
                tau_f = ordered_to_float((uint32_t)(key >> 32));
            }
        };
        const float kNoDoc = __int_as_float(0x7fc00000);  // NaN: a missing document never passes a comparison
        auto fetch_norm = [&](long long tile) {
            const long long doc = tile * TD + etid;
            return (etid < TD && tile < n_tiles && doc < a.n_docs) ? __ldg(a.norms + doc) : kNoDoc;
        };
        float norm_next = fetch_norm(blockIdx.x);
        uint32_t t = 0;
        for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++t) {
            const uint32_t ab = t % C::kAccBufs;
            const uint32_t aph = (t / C::kAccBufs) & 1u;
            float* nrm = norm_s + (t & 1u) * TD;
            if (etid < TD) nrm[etid] = norm_next;
            norm_next = fetch_norm(tile + gridDim.x);
            named_bar_sync(1, kEpiWarps * 32);
            if (*epi_stop != 0) break;
            // thresholds other CTAs published; lists that the coming tile could overflow are cut to their k best
            if (q_live) raise_tau(shared_tau[qtau]);
            unsigned need = __ballot_sync(0xffffffffu, cnt > kCutAbove);
            while (need != 0) {
                const int src = __ffs(need) - 1;
                need &= need - 1;
                const int n = __shfl_sync(0xffffffffu, cnt, src);
                u64* lst = cand + ((size_t)((maxsim ? a.maxsim_list_base : 0) + (quarter * 32 + src) / group) * n_segs + seg) * kTqTcSegLen;
                __syncwarp();
                for (int i = lane; i < n; i += 32) sortbuf[i] = lst[i];
                warp_sort_desc(sortbuf, n, lane);
                for (int i = lane; i < a.k; i += 32) lst[i] = sortbuf[i];
                const u64 kth = sortbuf[a.k - 1];
                __syncwarp();
                if (lane == src) {
                    cnt = a.k;
                    raise_tau(kth);
                    atomicMax(const_cast<u64*>(a.shared_tau) + qtau, kth);
                }
            }
            if (!__all_sync(0xffffffffu, mbar_wait(acc_full(ab), aph, abort_flag))) {
                *epi_stop = 1;
                continue;   // to the next common barrier, where every epilogue warp sees the flag
            }
            tc_fence_after();

            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + ab * TD + epart * (TD / 2);
            const uint32_t doc0 = a.id_base + (uint32_t)(tile * TD) + (uint32_t)(epart * (TD / 2));
            const float* nrm_w = nrm + epart * (TD / 2);
            float* seed_row = a.seed_scores != nullptr
                                  ? a.seed_scores + (size_t)qrow * a.seed_stride + (size_t)tile * TD + epart * (TD / 2)
                                  : nullptr;
            float child_max = -INFINITY;   // MaxSim: best child score of the current parent for this query vector
            auto chunk = [&](const uint32_t (&r)[16], const int c0) {
                float sc[16];
                bool any = false;
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                    const float4 nv = *reinterpret_cast<const float4*>(nrm_w + c0 + j);
                    sc[j] = __uint_as_float(r[j]) * nv.x;
                    sc[j + 1] = __uint_as_float(r[j + 1]) * nv.y;
                    sc[j + 2] = __uint_as_float(r[j + 2]) * nv.z;
                    sc[j + 3] = __uint_as_float(r[j + 3]) * nv.w;
                    any |= (sc[j] >= tau_f) | (sc[j + 1] >= tau_f) | (sc[j + 2] >= tau_f) | (sc[j + 3] >= tau_f);
                }
                if (maxsim) {
                    // a missing child has a NaN norm: fmaxf ignores it
#pragma unroll
                    for (int j = 0; j < 16; ++j) child_max = fmaxf(child_max, sc[j]);
                    if (((c0 + 16) & (a.maxsim_children - 1)) == 0) {
                        // the parent's last columns: sum the best child scores over the query's vectors (lanes of one
                        // group), the group's first lane keeps the candidate
                        float v = child_max;
                        for (int o = 1; o < group; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                        child_max = -INFINITY;
                        if (v >= tau_f) {   // false for NaN / -inf (a parent without children) and for non-owners
                            const uint32_t parent = (doc0 + (uint32_t)(c0 + 16 - a.maxsim_children)) / (uint32_t)a.maxsim_children;
                            const u64 key = make_key(v, parent);
                            if (key > tau_key) my_list[cnt++] = key;
                        }
                    }
                } else if (seed_row != nullptr) {
                    // seed mode: the thread's 16 scores are 64 contiguous bytes of its query's row
                    uint32_t lo8[8], hi8[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        lo8[j] = __float_as_uint(sc[j]);
                        hi8[j] = __float_as_uint(sc[8 + j]);
                    }
                    st_global_v8(seed_row + c0, lo8);
                    st_global_v8(seed_row + c0 + 8, hi8);
                } else if (any) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (sc[j] >= tau_f) {
                            const u64 key = make_key(sc[j], doc0 + (uint32_t)(c0 + j));
                            if (key > tau_key) my_list[cnt++] = key;  // cnt <= 128 before the tile, <= 128 + TD / 2 after
                        }
                    }
                }
            };
            uint32_t ra[16], rb[16];
            __syncwarp();
            tmem_ld_32x16(taddr, ra);
#pragma unroll 1
            for (int c0 = 0; c0 < TD / 2; c0 += 32) {
                tmem_ld_wait16(ra);
                __syncwarp();
                tmem_ld_32x16(taddr + c0 + 16, rb);
                chunk(ra, c0);
                tmem_ld_wait16(rb);
                if (c0 + 32 < TD / 2) {
                    __syncwarp();
                    tmem_ld_32x16(taddr + c0 + 32, ra);
                }
                chunk(rb, c0 + 16);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(ab));
        }
        if (!maxsim || owner) a.cand_count[(size_t)qlist * n_segs + seg] = cnt;
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

cudaError_t tq_tc_init() {
    cudaError_t e = cudaFuncSetAttribute(tq_score_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg<false>::kSmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(tq_score_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<true>::kSmemBytes);
    return e;
}

std::string tq_tc_make_query_map(CUtensorMap* tm, const __half* qperm, int padded_dim, int rows) {
    return encode_2d(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, qperm, (uint64_t)padded_dim, (uint64_t)rows,
                     (uint64_t)padded_dim * 2, TK, TQ, CU_TENSOR_MAP_SWIZZLE_128B);
}

bool tq_tc_queries_fit_tmem(int dim) {
    const int padded = (dim + kTqChunkCoords - 1) / kTqChunkCoords * kTqChunkCoords;
    return kQTmemCol + padded / 2 <= kTmemCols;
}

void launch_tq_score_tc(const CUtensorMap& tm_q, const TqTcArgs& a, bool q_in_tmem, int grid, cudaStream_t stream) {
    if (q_in_tmem) tq_score_tc_kernel<true><<<grid, Cfg<true>::kThreads, Cfg<true>::kSmemBytes, stream>>>(tm_q, a);
    else tq_score_tc_kernel<false><<<grid, Cfg<false>::kThreads, Cfg<false>::kSmemBytes, stream>>>(tm_q, a);
}

}  // namespace eosb
