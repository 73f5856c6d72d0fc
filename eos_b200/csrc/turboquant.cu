// TurboQuant (Hadamard/MSE variant) on sm_100a: code packing, scan layout, query preparation,
// scoring scan with exact per-CTA top-k, and the k-way merge.
//
// Reference call sites / semantics (file:line inside the Eos project):
//   encode structure          runtime/backends/cuda/native_linux.go:1812-1957 (manta_turboq_encode)
//   corpus quantise loop      runtime/retrieval_turboquant.go:700-711
//   per-query scoring + heap  runtime/retrieval_turboquant.go:1853-1916
//   order of results          runtime/retrieval_eval.go:1153-1161 (score desc, then id asc)
//
// Scoring: <q, doc> ~= norm * sum_c Rq[c] * centroid[code[c]] with R the quantiser's orthogonal
// rotation.  The scan streams the packed codes once per pass for a tile of 8/16/32 queries:
// every warp owns 16 documents, expands their 4-bit codes to f16 in registers with byte
// permutes (no shared-memory round trip) straight into mma.sync A fragments, and multiplies by
// the rotated queries held as B fragments.  The codebook of a symmetric density is symmetric,
// so a code is stored as sign + 3-bit magnitude and the 8 magnitudes fit the two 8-byte pools of
// a byte permute.
#include "turboquant.cuh"

#include "common.cuh"
#include "turboquant_dev.cuh"

namespace eosb {

namespace {


// ------------------------------------------------------------------------------------------
// packing
// ------------------------------------------------------------------------------------------
// rotated[perm[i]] = FWHT(x[perm[.]] * prescale * signs1)[i] * signs2[i]; x and the result live in
// shared memory (work, rot), one warp.
__device__ void warp_rotate(const float* x, float prescale, const TqSpec& s, float* work, float* rot, int lane) {
    for (int i = lane; i < s.dim; i += 32) work[i] = __fmul_rn(__fmul_rn(x[s.perm[i]], prescale), s.signs1[i]);
    __syncwarp();
    warp_fwht_blocks(work, s.dim, lane);
    for (int i = lane; i < s.dim; i += 32) rot[s.perm[i]] = __fmul_rn(work[i], s.signs2[i]);
    __syncwarp();
}

// norms[v] = sqrt of the sequential float sum of squares of vector v, in index order: the order of the reference's
// one-thread-per-vector kernel (manta_turboq_encode, runtime/backends/cuda/native_linux.go:1906-1957), so the bits
// are the same.  A sequential sum cannot be split over lanes, so each lane sums a vector of its own: 32 vectors per
// warp advance together (a lane's 16-byte loads walk its own row; a 32-byte sector serves two of them from L1).
__global__ void __launch_bounds__(256)
tq_norms_kernel(const float* __restrict__ x, long long n, int dim, float* __restrict__ norms) {
    const long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= n) return;
    const float* xv = x + v * dim;
    float sq = 0.f;
    if ((dim & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
        const float4* x4 = reinterpret_cast<const float4*>(xv);
#pragma unroll 4
        for (int c = 0; c < (dim >> 2); ++c) {
            const float4 f = __ldg(x4 + c);
            sq = __fadd_rn(sq, __fmul_rn(f.x, f.x));
            sq = __fadd_rn(sq, __fmul_rn(f.y, f.y));
            sq = __fadd_rn(sq, __fmul_rn(f.z, f.z));
            sq = __fadd_rn(sq, __fmul_rn(f.w, f.w));
        }
    } else {
        for (int c = 0; c < dim; ++c) {
            const float f = __ldg(xv + c);
            sq = __fadd_rn(sq, __fmul_rn(f, f));
        }
    }
    norms[v] = __fsqrt_rn(sq);
}

// One warp per vector: unit-normalise (norm from tq_norms_kernel), rotate, nearest centroid per coordinate by
// bisection over the boundaries, pack.
__global__ void __launch_bounds__(256)
tq_pack_kernel(const float* __restrict__ x, long long n, TqSpec s, uint8_t* __restrict__ codes,
               const float* __restrict__ norms) {
    extern __shared__ float sm_f[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps = blockDim.x >> 5;
    float* work = sm_f + (size_t)warp * 2 * s.dim;
    float* rot = work + s.dim;
    const int levels = 1 << s.bits;
    const int per_byte = 8 / s.bits;
    const long long cb = ((long long)s.dim * s.bits + 7) / 8;
    for (long long v = (long long)blockIdx.x * warps + warp; v < n; v += (long long)gridDim.x * warps) {
        const float* xv = x + v * s.dim;
        // the vector moves to shared memory with coalesced loads (rot serves as the staging buffer: the rotation
        // reads all of it before it writes any of it)
        if ((s.dim & 3) == 0 && (reinterpret_cast<uintptr_t>(xv) & 15u) == 0) {
            for (int i = lane; i < (s.dim >> 2); i += 32)
                reinterpret_cast<float4*>(rot)[i] = __ldg(reinterpret_cast<const float4*>(xv) + i);
        } else {
            for (int i = lane; i < s.dim; i += 32) rot[i] = __ldg(xv + i);
        }
        const float norm = __ldg(norms + v);
        __syncwarp();
        const float scale = norm > 1.0e-12f ? __fdiv_rn(1.0f, norm) : 1.0f;
        warp_rotate(rot, scale, s, work, rot, lane);
        uint8_t* cv = codes + v * cb;
        for (long long byte = lane; byte < cb; byte += 32) {
            unsigned out = 0;
            for (int e = 0; e < per_byte; ++e) {
                const int c = (int)byte * per_byte + e;
                if (c < s.dim) {
                    const float val = rot[c];
                    int lo = 0, hi = levels - 1;
                    while (lo < hi) {
                        const int mid = (lo + hi) >> 1;
                        if (s.boundaries[mid] > val) hi = mid; else lo = mid + 1;
                    }
                    out |= (unsigned)lo << (e * s.bits);
                }
            }
            cv[byte] = (uint8_t)out;
        }
        __syncwarp();
    }
}

__global__ void __launch_bounds__(256)
tq_transcode_kernel(const uint8_t* __restrict__ codes, long long n, int dim, int bits, uint32_t* __restrict__ tiles) {
    const int chunks = (dim + kTqChunkCoords - 1) / kTqChunkCoords;
    const long long words_per_tile = (long long)chunks * 32 * 8;  // 8 words per lane per chunk
    const long long n_tiles = (n + kTqDocsPerTile - 1) / kTqDocsPerTile;
    const long long total = n_tiles * words_per_tile;
    const int half_levels = 1 << (bits - 1);
    const int per_byte = 8 / bits;
    const int code_mask = (1 << bits) - 1;
    const long long cb = ((long long)dim * bits + 7) / 8;
    for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < total;
         w += (long long)gridDim.x * blockDim.x) {
        const long long tile = w / words_per_tile;
        const int r = (int)(w % words_per_tile);
        const int c = r / 256;
        const int lane = (r % 256) / 8;
        const int sub = r % 8;  // 0..3: document g, 4..7: document g+8
        const int i = sub & 3;
        const int g = lane >> 2, t = lane & 3;
        const long long doc = tile * kTqDocsPerTile + g + (sub >> 2) * 8;
        uint32_t out = 0;
        if (doc < n) {
            const uint8_t* cv = codes + doc * cb;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int coord = scan_coord(c, i, t, e);
                if (coord < dim) {
                    const int code = (cv[coord / per_byte] >> ((coord % per_byte) * bits)) & code_mask;
                    const int neg = code < half_levels;
                    const int mag = neg ? (half_levels - 1 - code) : (code - half_levels);
                    out |= (uint32_t)mag << (4 * e);
                    out |= (uint32_t)neg << (e < 4 ? 8 * e + 7 : 8 * (e - 4) + 3);
                }
            }
        }
        tiles[w] = out;
    }
}

// ------------------------------------------------------------------------------------------
// query preparation: rotate, round to f16, lay out as mma.sync B fragments.
// bfrag[(tile*ksteps + s)*32 + lane] = { half2(q[16s+2t], q[16s+2t+1]), half2(q[16s+2t+8], q[16s+2t+9]) }
// for query tile*8 + g.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
tq_prepare_kernel(const float* __restrict__ queries, int nq, int q_fill, TqSpec s, int ksteps,
                  uint2* __restrict__ bfrag, float* __restrict__ rotated_out, __half* __restrict__ qperm) {
    extern __shared__ float sm_f[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps = blockDim.x >> 5;
    float* xin = sm_f + (size_t)warp * 3 * s.dim;
    float* work = xin + s.dim;
    float* rot = work + s.dim;
    const int q_padded = q_fill;
    for (int q = blockIdx.x * warps + warp; q < q_padded; q += gridDim.x * warps) {
        if (q < nq) {
            for (int i = lane; i < s.dim; i += 32) xin[i] = queries[(size_t)q * s.dim + i];
            __syncwarp();
            warp_rotate(xin, 1.0f, s, work, rot, lane);
            if (rotated_out != nullptr)
                for (int i = lane; i < s.dim; i += 32) rotated_out[(size_t)q * s.dim + i] = rot[i];
        } else {
            for (int i = lane; i < s.dim; i += 32) rot[i] = 0.f;  // padding queries score 0
            __syncwarp();
        }
        if (qperm != nullptr) {
            // row-major f16 copy for the tensor-core kernel: inside every block of 64 coordinates, 16-byte piece j
            // holds the 8 coordinates of code word (2 (kb & 1) + (j >> 2), column j & 3) of the scan layout
            const int dimp = ksteps * 16;
            for (int idx = lane; idx < dimp; idx += 32) {
                const int kb = idx >> 6, j = (idx >> 3) & 7, e = idx & 7;
                const int coord = scan_coord(kb >> 1, 2 * (kb & 1) + (j >> 2), j & 3, e);
                qperm[(size_t)q * dimp + idx] = __float2half_rn(coord < s.dim ? rot[coord] : 0.f);
            }
        }
        const int tile = q >> 3, g = q & 7;
        for (int idx = lane; bfrag != nullptr && idx < ksteps * 4; idx += 32) {
            const int st = idx >> 2, t = idx & 3;
            const int c0 = 16 * st + 2 * t;
            float v[4];
            const int cc[4] = {c0, c0 + 1, c0 + 8, c0 + 9};
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = cc[e] < s.dim ? rot[cc[e]] : 0.f;
            __half2 h0 = __floats2half2_rn(v[0], v[1]), h1 = __floats2half2_rn(v[2], v[3]);
            uint2 o;
            o.x = *reinterpret_cast<uint32_t*>(&h0);
            o.y = *reinterpret_cast<uint32_t*>(&h1);
            bfrag[((size_t)tile * ksteps + st) * 32 + g * 4 + t] = o;
        }
        __syncwarp();
    }
}

// ------------------------------------------------------------------------------------------
// the scan
// ------------------------------------------------------------------------------------------
constexpr int kScanCap = kTqMaxK + kTqScanWarps * kTqDocsPerTile;  // 384 keys per query buffer

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int J>
__global__ void __launch_bounds__(kTqScanWarps * 32, 1) tq_scan_kernel(TqScanArgs a) {
    extern __shared__ __align__(16) uint8_t sm_raw[];
    constexpr int QB = 8 * J;
    const int ksteps = tq_ksteps(a.dim);
    const int chunks = ksteps / 8;
    uint2* bfr = reinterpret_cast<uint2*>(sm_raw);                                  // [J][ksteps][32]
    u64* buf = reinterpret_cast<u64*>(sm_raw + (size_t)J * ksteps * 32 * 8);        // [QB][kScanCap]
    u64* tau = buf + (size_t)QB * kScanCap;                                          // [QB]
    int* cnt = reinterpret_cast<int*>(tau + QB);                                     // [QB]
    unsigned* hist = reinterpret_cast<unsigned*>(cnt + QB);                          // [warps][256]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    for (int i = threadIdx.x; i < J * ksteps * 32; i += blockDim.x) bfr[i] = a.bfrag[i];
    for (int i = threadIdx.x; i < QB; i += blockDim.x) {
        tau[i] = 0;
        cnt[i] = 0;
    }
    __syncthreads();

    const long long n_tiles = (a.n_docs + kTqDocsPerTile - 1) / kTqDocsPerTile;
    const size_t tile_u4 = (size_t)chunks * 64;  // uint4 per tile
    const uint4* tiles = reinterpret_cast<const uint4*>(a.tiles);
    const long long stride_tiles = (long long)gridDim.x * kTqScanWarps;
    const long long iters = (n_tiles + stride_tiles - 1) / stride_tiles;
    volatile u64* vtau = tau;

    for (long long it = 0; it < iters; ++it) {
        const long long tile = it * stride_tiles + (long long)blockIdx.x * kTqScanWarps + warp;
        if (tile < n_tiles) {
            const uint4* tp = tiles + tile * tile_u4 + lane * 2;
            float acc[J][4];
#pragma unroll
            for (int j = 0; j < J; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
            uint4 da = __ldg(tp), db = __ldg(tp + 1);
            for (int c = 0; c < chunks; ++c) {
                const uint4 ca = da, cb = db;
                if (c + 1 < chunks) {
                    da = __ldg(tp + (c + 1) * 64);
                    db = __ldg(tp + (c + 1) * 64 + 1);
                }
                const uint32_t wa[4] = {ca.x, ca.y, ca.z, ca.w};
                const uint32_t wb[4] = {cb.x, cb.y, cb.z, cb.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t va[4], vb[4];
                    dequant8(wa[i], a.mag_hi[0], a.mag_hi[1], a.mag_lo[0], a.mag_lo[1], va);
                    dequant8(wb[i], a.mag_hi[0], a.mag_hi[1], a.mag_lo[0], a.mag_lo[1], vb);
                    const int s0 = c * 8 + 2 * i;
#pragma unroll
                    for (int j = 0; j < J; ++j) {
                        const uint2 b0 = bfr[(j * ksteps + s0) * 32 + lane];
                        const uint2 b1 = bfr[(j * ksteps + s0 + 1) * 32 + lane];
                        mma16816(acc[j], va[0], vb[0], va[1], vb[1], b0.x, b0.y);
                        mma16816(acc[j], va[2], vb[2], va[3], vb[3], b1.x, b1.y);
                    }
                }
            }
            // epilogue: scale by the document norms, keep candidates that beat the running k-th
            const long long d0 = tile * kTqDocsPerTile + g;
            const long long d1 = d0 + 8;
            const float n0 = d0 < a.n_docs ? __ldg(a.norms + d0) : 0.f;
            const float n1 = d1 < a.n_docs ? __ldg(a.norms + d1) : 0.f;
#pragma unroll
            for (int j = 0; j < J; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const long long doc = (e & 2) ? d1 : d0;
                    if (doc < a.n_docs) {
                        const int q = j * 8 + 2 * t + (e & 1);
                        const float sc = acc[j][e] * ((e & 2) ? n1 : n0);
                        if (a.all_scores != nullptr) {
                            a.all_scores[(long long)q * a.all_stride + doc] = sc;
                            continue;
                        }
                        const u64 key = make_key(sc, a.id_base + (uint32_t)doc);
                        if (key > vtau[q]) {
                            const int pos = atomicAdd(&cnt[q], 1);
                            buf[(size_t)q * kScanCap + pos] = key;  // pos < kScanCap by construction
                        }
                    }
                }
            }
        }
        __syncthreads();
        // buffers that could overflow in the next round are cut back to their k best
        for (int q = warp; q < QB; q += kTqScanWarps) {
            const int n = cnt[q];
            if (n > kTqMaxK) {
                u64* keys = buf + (size_t)q * kScanCap;
                const u64 thr = warp_kth_largest(keys, n, a.k, hist + warp * 256, lane);
                u64 mine[kScanCap / 32];
#pragma unroll
                for (int r = 0; r < kScanCap / 32; ++r) {
                    const int i = r * 32 + lane;
                    mine[r] = i < n ? keys[i] : 0;
                }
                __syncwarp();
                int base = 0;
#pragma unroll
                for (int r = 0; r < kScanCap / 32; ++r) {
                    const bool keep = mine[r] >= thr && mine[r] != 0;
                    const unsigned bal = __ballot_sync(0xffffffffu, keep);
                    if (keep) keys[base + __popc(bal & ((1u << lane) - 1u))] = mine[r];
                    base += __popc(bal);
                }
                __syncwarp();
                if (lane == 0) {
                    cnt[q] = base;
                    tau[q] = thr;
                }
            }
        }
        __syncthreads();
    }
    if (a.all_scores != nullptr) return;
    // final cut to k and write-out
    for (int q = warp; q < QB; q += kTqScanWarps) {
        int n = cnt[q];
        u64* keys = buf + (size_t)q * kScanCap;
        u64 thr = 0;
        if (n > a.k) thr = warp_kth_largest(keys, n, a.k, hist + warp * 256, lane);
        u64* out = reinterpret_cast<u64*>(a.cand_keys) + ((size_t)q * a.grid + blockIdx.x) * kTqMaxK;
        int base = 0;
        for (int r = 0; r < kScanCap / 32; ++r) {
            const int i = r * 32 + lane;
            const u64 key = i < n ? keys[i] : 0;
            const bool keep = key != 0 && key >= thr;
            const unsigned bal = __ballot_sync(0xffffffffu, keep);
            if (keep) out[base + __popc(bal & ((1u << lane) - 1u))] = key;
            base += __popc(bal);
        }
        if (lane == 0) a.cand_count[(size_t)q * a.grid + blockIdx.x] = base;
    }
}

// ------------------------------------------------------------------------------------------
// the scan, streaming form for 8 queries per pass.  Differences to tq_scan_kernel:
//   * code tiles arrive by bulk-async copies (cp.async.bulk, completion on an mbarrier) into two
//     private 1-tile slots per warp, so every warp keeps up to two tiles (12 KB at dim 768) in flight
//     and never waits for another warp;
//   * the rotated queries live in registers as MMA B fragments for the whole kernel;
//   * candidates go to a small per-warp staging area and are folded into the CTA's per-query list
//     under a per-query lock only when the staging area is half full, so there is no block-wide
//     barrier inside the scan loop.
// ------------------------------------------------------------------------------------------
constexpr int kStreamWarps = 12;
constexpr int kStreamStage = 32;             // staged keys per (warp, query)
constexpr int kStreamList = kSortCap;               // CTA list slots per query (at most kTqMaxK + kStreamStage in use)

__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_dst),
                 "l"(gsrc), "r"(bytes), "r"(bar)
                 : "memory");
}

#ifdef EOSB_SCAN_TIMING
__device__ long long g_scan_timing[8];
#define SMARK(i) do { if (blockIdx.x == 0 && threadIdx.x == 0) g_scan_timing[i] = clock64(); } while (0)
#else
#define SMARK(i) do { } while (0)
#endif

template <int KSTEPS>
__global__ void __launch_bounds__(kStreamWarps * 32, 1) tq_scan_stream_kernel(TqScanArgs a) {
    extern __shared__ __align__(16) uint8_t sm_raw[];
    SMARK(0);
    constexpr int CHUNKS = KSTEPS / 8;
    constexpr uint32_t TILE_BYTES = CHUNKS * 1024;
    uint8_t* slots = sm_raw;                                                            // [warps][2][TILE_BYTES]
    u64* list = reinterpret_cast<u64*>(sm_raw + (size_t)kStreamWarps * 2 * TILE_BYTES); // [8][kStreamList]
    u64* stage = list + 8 * kStreamList;                                                 // [warps][8][kStreamStage]
    u64* tau = stage + (size_t)kStreamWarps * 8 * kStreamStage;                          // [8]
    u64* bars = tau + 8;                                                                 // [warps][2] mbarriers
    int* lcnt = reinterpret_cast<int*>(bars + kStreamWarps * 2);                         // [8] list counts
    int* locks = lcnt + 8;                                                               // [8]
    int* wcnt = locks + 8;                                                               // [warps][8] staged counts
    __shared__ int abort_flag_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    if (threadIdx.x == 0) abort_flag_s = 0;
    for (int i = threadIdx.x; i < 8; i += blockDim.x) {
        tau[i] = a.shared_tau != nullptr ? a.shared_tau[i] : 0;  // seeded by the host from a sample, or 0
        lcnt[i] = 0;
        locks[i] = 0;
    }
    for (int i = threadIdx.x; i < kStreamWarps * 8; i += blockDim.x) wcnt[i] = 0;
    if (lane == 0) {
        mbar_init(smem_u32(&bars[warp * 2]), 1);
        mbar_init(smem_u32(&bars[warp * 2 + 1]), 1);
        mbar_fence_init();
    }
    // rotated queries as B fragments, resident in registers
    uint2 bq[KSTEPS];
#pragma unroll
    for (int s = 0; s < KSTEPS; ++s) bq[s] = __ldg(a.bfrag + s * 32 + lane);
    __syncthreads();
    volatile int* abort_flag = &abort_flag_s;
    volatile u64* vtau = tau;

    const long long n_tiles = (a.n_docs + kTqDocsPerTile - 1) / kTqDocsPerTile;
    const long long stride_tiles = (long long)gridDim.x * kStreamWarps;
    const long long first = (long long)blockIdx.x * kStreamWarps + warp;
    const uint8_t* gt = a.tiles;
    uint8_t* my_slots = slots + (size_t)warp * 2 * TILE_BYTES;
    const uint32_t bar_addr[2] = {smem_u32(&bars[warp * 2]), smem_u32(&bars[warp * 2 + 1])};

    auto issue = [&](long long tile, int slot) {
        if (lane == 0 && tile < n_tiles) {
            mbar_arrive_expect_tx(bar_addr[slot], TILE_BYTES);
            bulk_load(smem_u32(my_slots + slot * TILE_BYTES), gt + (size_t)tile * TILE_BYTES, TILE_BYTES, bar_addr[slot]);
        }
    };
    // fold this warp's staged keys of query q into the CTA list (lane-parallel, under the query's lock)
    auto flush = [&](int q) -> bool {
        const int m = wcnt[warp * 8 + q];
        if (m == 0) return true;
        int got = 0;
        if (lane == 0) {
            for (int spin = 0; spin < (1 << 24); ++spin) {
                if (atomicCAS(&locks[q], 0, 1) == 0) {
                    got = 1;
                    break;
                }
                if (*abort_flag) break;
            }
            if (!got) *abort_flag = 1;
        }
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) return false;
        __threadfence_block();
        u64* keys = list + q * kStreamList;
        int n = *reinterpret_cast<volatile int*>(&lcnt[q]);
        u64 cur_tau = vtau[q];
        if (a.shared_tau != nullptr) {
            // the k-th best key any CTA holds is a lower bound of the global k-th best key
            const u64 g_tau = *reinterpret_cast<volatile u64*>(a.shared_tau + q);
            if (g_tau > cur_tau) {
                cur_tau = g_tau;
                if (lane == 0) tau[q] = g_tau;
            }
        }
        const u64* st = stage + ((size_t)warp * 8 + q) * kStreamStage;
        // staged keys that still beat the (possibly raised) threshold
        const u64 mine = lane < m ? st[lane] : 0;
        const bool keep = mine > cur_tau;
        const unsigned bal = __ballot_sync(0xffffffffu, keep);
        if (keep) keys[n + __popc(bal & ((1u << lane) - 1u))] = mine;
        n += __popc(bal);
        __syncwarp();
        if (n > kStreamList - kStreamStage) {
            // the list cannot take another flush: cut it back to the k best (sort, slots past n cleared first, keep
            // the head).  Cutting only when the 256 slots are nearly full makes cuts four times rarer than cutting at
            // k + 32, for a threshold that is a little staler in between
            warp_sort_desc(keys, n, lane);
            n = a.k;
            const u64 thr = keys[a.k - 1];
            if (lane == 0) {
                tau[q] = thr;
                if (a.shared_tau != nullptr) atomicMax(a.shared_tau + q, thr);
            }
        }
        __syncwarp();
        if (lane == 0) {
            lcnt[q] = n;
            wcnt[warp * 8 + q] = 0;
            __threadfence_block();
            atomicExch(&locks[q], 0);
        }
        __syncwarp();
        return true;
    };

    SMARK(1);
    issue(first, 0);
    issue(first + stride_tiles, 1);
    bool ok = true;
    long long k = 0;
    for (long long tile = first; ok && tile < n_tiles; tile += stride_tiles, ++k) {
        const int slot = (int)(k & 1);
        if (!mbar_wait(bar_addr[slot], (uint32_t)((k >> 1) & 1), abort_flag)) {
            ok = false;
            break;
        }
        const uint4* tp = reinterpret_cast<const uint4*>(my_slots + slot * TILE_BYTES) + lane * 2;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const uint4 ca = tp[c * 64], cb = tp[c * 64 + 1];
            const uint32_t wa[4] = {ca.x, ca.y, ca.z, ca.w};
            const uint32_t wb[4] = {cb.x, cb.y, cb.z, cb.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t va[4], vb[4];
                dequant8(wa[i], a.mag_hi[0], a.mag_hi[1], a.mag_lo[0], a.mag_lo[1], va);
                dequant8(wb[i], a.mag_hi[0], a.mag_hi[1], a.mag_lo[0], a.mag_lo[1], vb);
                const int s0 = c * 8 + 2 * i;
                mma16816(acc, va[0], vb[0], va[1], vb[1], bq[s0].x, bq[s0].y);
                mma16816(acc, va[2], vb[2], va[3], vb[3], bq[s0 + 1].x, bq[s0 + 1].y);
            }
        }
        // the slot has been read: refill it with the tile after next
        __syncwarp();
        if (lane == 0) fence_proxy_async_smem();
        issue(tile + 2 * stride_tiles, slot);
        // epilogue: scale by the document norms, stage candidates that beat the running k-th
        const long long d0 = tile * kTqDocsPerTile + g;
        const long long d1 = d0 + 8;
        const float n0 = d0 < a.n_docs ? __ldg(a.norms + d0) : 0.f;
        const float n1 = d1 < a.n_docs ? __ldg(a.norms + d1) : 0.f;
        if (a.all_scores != nullptr) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const long long doc = (e & 2) ? d1 : d0;
                if (doc < a.n_docs)
                    a.all_scores[(long long)(2 * t + (e & 1)) * a.all_stride + doc] = acc[e] * ((e & 2) ? n1 : n0);
            }
        } else {
            // keys of documents past the end are 0 and never beat a threshold
            u64 key[4];
            bool any_pass = false;
            const u64 t0 = vtau[2 * t], t1 = vtau[2 * t + 1];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const long long doc = (e & 2) ? d1 : d0;
                key[e] = doc < a.n_docs ? make_key(acc[e] * ((e & 2) ? n1 : n0), a.id_base + (uint32_t)doc) : 0;
                any_pass |= key[e] > ((e & 1) ? t1 : t0);
            }
            if (__any_sync(0xffffffffu, any_pass)) {  // rare once the lists have warmed up
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int q = 2 * t + (e & 1);
                    if (key[e] > ((e & 1) ? t1 : t0)) {
                        const int pos = atomicAdd(&wcnt[warp * 8 + q], 1);
                        stage[((size_t)warp * 8 + q) * kStreamStage + pos] = key[e];  // pos < 32: flushed above 16
                    }
                }
            }
        }
        __syncwarp();
        if (a.all_scores == nullptr && a.shared_tau != nullptr && (k & 7) == 7 && lane < 8) {
            // pick up the thresholds the other CTAs have published (monotonic, so a stale value is only less sharp)
            const u64 g_tau = *reinterpret_cast<volatile u64*>(a.shared_tau + lane);
            if (g_tau > vtau[lane]) atomicMax(&tau[lane], g_tau);
        }
        if (a.all_scores == nullptr) {
            const int pending = lane < 8 ? wcnt[warp * 8 + lane] : 0;
            unsigned need = __ballot_sync(0xffffffffu, pending > kStreamStage / 2);
            while (need && ok) {
                const int q = __ffs(need) - 1;
                need &= need - 1;
                ok = flush(q);
            }
        }
    }
    SMARK(2);
    if (a.all_scores == nullptr) {
        for (int q = 0; q < 8 && ok; ++q) ok = flush(q);
    }
    SMARK(3);
    __syncthreads();
    SMARK(4);
    if (a.all_scores != nullptr) return;
    // final cut to k and write-out: warp q finishes query q
    if (warp < 8) {
        const int q = warp;
        u64* keys = list + q * kStreamList;
        const int n = lcnt[q];
        int n_out = n;
        if (n > a.k) {
            warp_sort_desc(keys, n, lane);
            n_out = a.k;
        }
        u64* out = reinterpret_cast<u64*>(a.cand_keys) + ((size_t)q * a.grid + blockIdx.x) * kTqMaxK;
        for (int i = lane; i < n_out; i += 32) out[i] = keys[i];
        if (lane == 0) a.cand_count[(size_t)q * a.grid + blockIdx.x] = n_out;
    }
    SMARK(5);
    if (threadIdx.x == 0 && abort_flag_s != 0 && a.status != nullptr) atomicExch(a.status, kStatusPipelineTimeout);
}

#ifdef EOSB_SCAN_TIMING
extern "C" __attribute__((visibility("default"))) int eos_b200_debug_scan_timing(long long* out8) {
    return cudaMemcpyFromSymbol(out8, g_scan_timing, sizeof(long long) * 8) != cudaSuccess;
}
#endif

template <int KSTEPS>
size_t tq_stream_smem() {
    return (size_t)kStreamWarps * 2 * (KSTEPS / 8) * 1024 + (size_t)8 * kStreamList * 8 +
           (size_t)kStreamWarps * 8 * kStreamStage * 8 + 8 * 8 + (size_t)kStreamWarps * 2 * 8 + 8 * 4 + 8 * 4 +
           (size_t)kStreamWarps * 8 * 4 + 128;
}


// ------------------------------------------------------------------------------------------
// dense candidates: dotRows / cosineRows (runtime/backend/tensor_ops.go:1967-2057, device bodies
// compiler/compiler.go:837-863) and the rerank loops topDenseRerankScores / topFP16RerankScores
// (runtime/retrieval_turboquant.go:1610-1662).  One warp per (document row, group of queries): the
// row is read once into registers (fp32, or f16 widened to fp32 as halfToFloat32 does), every query
// of the group is dotted against it in fp32, the result becomes a sortable key.  With a candidate
// list the group is one query and the row is that query's j-th candidate (id < 0 = absent, key 0).
// ------------------------------------------------------------------------------------------
constexpr int kDenseMaxPerLane = 32;  // dim <= 1024
constexpr int kDenseQueryGroup = 4;

template <bool kHalf>
__global__ void __launch_bounds__(256)
dense_keys_kernel(const void* __restrict__ docs, long long n_rows, int dim, const float* __restrict__ queries, int nq,
                  const long long* __restrict__ cand_ids, long long cand, int metric, u64* __restrict__ keys) {
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    const int group = cand_ids != nullptr ? 1 : kDenseQueryGroup;
    const int qgroups = (nq + group - 1) / group;
    const long long items = (long long)qgroups * cand;
    for (long long it = warp; it < items; it += warps) {
        const int qg = (int)(it / cand);
        const long long j = it % cand;
        long long row = j;
        if (cand_ids != nullptr) row = cand_ids[(long long)qg * cand + j];
        if (row < 0 || row >= n_rows) {
            if (lane == 0)
                for (int qi = qg * group; qi < nq && qi < (qg + 1) * group; ++qi) keys[(long long)qi * cand + j] = 0;
            continue;
        }
        float d[kDenseMaxPerLane];
        float dn = 0.f;
#pragma unroll
        for (int c = 0; c < kDenseMaxPerLane; ++c) {
            const int col = c * 32 + lane;
            d[c] = 0.f;
            if (col < dim) {
                if (kHalf) d[c] = __half2float(reinterpret_cast<const __half*>(docs)[(size_t)row * dim + col]);
                else d[c] = reinterpret_cast<const float*>(docs)[(size_t)row * dim + col];
            }
            dn = fmaf(d[c], d[c], dn);
        }
        if (metric == 1) dn = warp_sum(dn);
        for (int qi = qg * group; qi < nq && qi < (qg + 1) * group; ++qi) {
            const float* q = queries + (size_t)qi * dim;
            float dot = 0.f, qn = 0.f;
#pragma unroll
            for (int c = 0; c < kDenseMaxPerLane; ++c) {
                const int col = c * 32 + lane;
                const float qv = col < dim ? __ldg(q + col) : 0.f;
                dot = fmaf(qv, d[c], dot);
                qn = fmaf(qv, qv, qn);
            }
            dot = warp_sum(dot);
            float score = dot;
            if (metric == 1) {
                qn = warp_sum(qn);
                const float denom = sqrtf(qn) * sqrtf(dn);
                score = denom == 0.f ? 0.f : dot / denom;
            }
            // the id inside the key is the row, so that ties go to the smaller row (topKTensor, retrievalScoreBetter)
            if (lane == 0) keys[(long long)qi * cand + j] = make_key(score, (uint32_t)row);
        }
    }
}

// ------------------------------------------------------------------------------------------
// merge of counted candidate lists (the tensor-core batch kernel's output: n_segs lists of up to seg_len keys
// per query, cnts entries in use).  One CTA per query.  The counts are prefix-summed in shared memory, the
// keys are gathered once from global memory (independent, unrolled loads: the lists are short and scattered,
// so a pass over them is latency-bound) into shared memory, and the radix select, the gather of the k best
// and the sort run there.  A query with more candidates than the buffer holds selects from global memory.
// ------------------------------------------------------------------------------------------
// Radix-select step by one warp: hist[256] counts keys by digit; picks the digit d that holds the want-th largest key
// (digits descending) and the rank wanted inside it.  Lane l owns digits 8l .. 8l+7.  All 32 lanes call it.
__device__ __forceinline__ void warp_pick_digit(const unsigned* hist, unsigned want, int lane, int* d_out,
                                                unsigned* want_out) {
    unsigned c[8], s = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        c[j] = hist[lane * 8 + j];
        s += c[j];
    }
    unsigned incl = s;  // sum over lanes >= this one (higher lanes own higher digits)
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned t = __shfl_down_sync(0xffffffffu, incl, o);
        if (lane + o < 32) incl += t;
    }
    const unsigned above = incl - s;
    const bool mine = above < want && want <= incl;
    int d = 0;
    unsigned nw = 0;
    if (mine) {
        unsigned run = above;
#pragma unroll
        for (int j = 7; j >= 0; --j) {
            if (nw == 0) {
                if (run + c[j] >= want) {
                    d = lane * 8 + j;
                    nw = want - run;
                } else {
                    run += c[j];
                }
            }
        }
    }
    const unsigned bal = __ballot_sync(0xffffffffu, mine);
    const int src = bal != 0 ? __ffs(bal) - 1 : 0;
    *d_out = __shfl_sync(0xffffffffu, d, src);
    *want_out = __shfl_sync(0xffffffffu, nw, src);
}

constexpr int kListThreads = 512;
constexpr int kListMaxSegs = 1024;
constexpr int kListCapKeys = 8192;    // 64 KB of keys: three CTAs per SM, a launch of 256 queries is one wave
constexpr int kSeedCapScores = 40960; // 80 KB of 16-bit scores: two CTAs per SM

// prefix[0] = 0, prefix[i + 1] = sum of min(cnts[j], seg_len) for j <= i; returns the total.  Whole block.
__device__ int list_prefix(const int* __restrict__ cnts, int n_segs, int seg_len, int* prefix) {
    for (int i = threadIdx.x; i < n_segs; i += blockDim.x) prefix[i + 1] = min(max(cnts[i], 0), seg_len);
    if (threadIdx.x == 0) prefix[0] = 0;
    __syncthreads();
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        int carry = 0;
        for (int b = 0; b < n_segs; b += 32) {
            int v = b + lane < n_segs ? prefix[b + lane + 1] : 0;
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += t;
            }
            if (b + lane < n_segs) prefix[b + lane + 1] = v + carry;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
    }
    __syncthreads();
    return prefix[n_segs];
}
// list that holds flat entry i: the largest seg with prefix[seg] <= i
__device__ __forceinline__ int list_find(const int* prefix, int n_segs, int i) {
    int lo = 0, hi = n_segs;  // invariant: prefix[lo] <= i < prefix[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (prefix[mid] <= i) lo = mid; else hi = mid;
    }
    return lo;
}

__global__ void __launch_bounds__(kListThreads)
tq_merge_lists_kernel(const u64* __restrict__ cand, long long query_stride, long long seg_stride, int n_segs, int seg_len,
                      const int* __restrict__ counts, int k, long long* __restrict__ out_ids,
                      float* __restrict__ out_scores, u64* __restrict__ out_keys) {
    extern __shared__ __align__(16) uint8_t lsm[];
    u64* buf = reinterpret_cast<u64*>(lsm);                       // [kListCapKeys]
    int* prefix = reinterpret_cast<int*>(buf + kListCapKeys);      // [n_segs + 1]
    __shared__ unsigned hist[256];
    __shared__ u64 s_prefix, s_mask;
    __shared__ unsigned s_want;
    __shared__ int s_fill;
    __shared__ u64 sel[kTqMaxK];
    const int qi = blockIdx.x;
    const u64* base = cand + (long long)qi * query_stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int total = list_prefix(counts + (long long)qi * n_segs, n_segs, seg_len, prefix);
    const bool in_smem = total <= kListCapKeys;
    auto global_key = [&](int i) {
        const int seg = list_find(prefix, n_segs, i);
        return base[(long long)seg * seg_stride + (i - prefix[seg])];
    };
    if (in_smem) {
        for (int i0 = threadIdx.x; i0 < total; i0 += 4 * kListThreads) {
            u64 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * kListThreads;
                v[u] = i < total ? global_key(i) : 0;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * kListThreads;
                if (i < total) buf[i] = v[u];
            }
        }
    }
    if (threadIdx.x == 0) s_fill = 0;
    for (int i = threadIdx.x; i < kTqMaxK; i += blockDim.x) sel[i] = 0;
    __syncthreads();
    auto key_at = [&](int i) { return in_smem ? buf[i] : global_key(i); };
    const int kk = total < k ? total : k;
    u64 thr = 1;  // keep every key
    if (total > k) {
        if (threadIdx.x == 0) {
            s_prefix = 0;
            s_mask = 0;
            s_want = (unsigned)k;
        }
        for (int shift = 56; shift >= 0; shift -= 8) {
            for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
            __syncthreads();
            const u64 pre = s_prefix, mask = s_mask;
            for (int i = threadIdx.x; i < total; i += blockDim.x) {
                const u64 key = key_at(i);
                if ((key & mask) == pre) atomicAdd(&hist[(unsigned)(key >> shift) & 0xffu], 1u);
            }
            __syncthreads();
            if (threadIdx.x < 32) {
                int d;
                unsigned nw;
                warp_pick_digit(hist, s_want, lane, &d, &nw);
                __syncwarp();
                if (lane == 0) {
                    s_want = nw;
                    s_prefix = pre | ((u64)(unsigned)d << shift);
                    s_mask = mask | ((u64)0xffu << shift);
                }
            }
            __syncthreads();
        }
        thr = s_prefix;
    }
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const u64 key = key_at(i);
        if (key >= thr) {
            const int pos = atomicAdd(&s_fill, 1);
            if (pos < kTqMaxK) sel[pos] = key;
        }
    }
    __syncthreads();
    if (warp == 0) {
        for (int size = 2; size <= kTqMaxK; size <<= 1) {
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                for (int tt = lane; tt < kTqMaxK / 2; tt += 32) {
                    const int i = 2 * tt - (tt & (stride - 1));
                    const int j = i + stride;
                    const bool desc = (i & size) == 0;
                    const u64 x = sel[i], y = sel[j];
                    if ((x < y) == desc) {
                        sel[i] = y;
                        sel[j] = x;
                    }
                }
                __syncwarp();
            }
        }
        for (int i = lane; i < k; i += 32) {
            const u64 key = i < kk ? sel[i] : 0;
            if (out_keys != nullptr) out_keys[(long long)qi * k + i] = key;
            if (out_ids != nullptr) {
                out_ids[(long long)qi * k + i] = key != 0 ? (long long)(0xffffffffu - (uint32_t)(key & 0xffffffffu)) : -1;
                out_scores[(long long)qi * k + i] = key != 0 ? ordered_to_float((uint32_t)(key >> 32)) : -INFINITY;
            }
        }
    }
}

// Pruning thresholds from the scores of a sample: scores is [queries][total] fp32 (every sample document's score,
// written by the batch kernels in their seed mode).  Only the upper 16 of the 32 order-preserving score bits are
// kept (rounded down, so that up to kSeedCapScores documents take 80 KB of shared memory and two radix passes
// select): tau[q] = (k-th best truncated score, as a key whose other bits are 0) - 1.  At least k documents of
// the sample have a key above it, so the k-th best key of the whole shard does too; the truncation (2^-7 of
// the score) only lets a few more candidates pass.  0 when the sample holds fewer than k documents.  The radix
// select counts into one histogram per warp (the scores of a query share their leading digits, and a single
// histogram would serialise every warp on one counter).
__global__ void __launch_bounds__(kListThreads)
tq_seed_tau_scores_kernel(const float* __restrict__ scores, long long query_stride, int total, int k,
                          unsigned long long* __restrict__ tau) {
    extern __shared__ __align__(16) uint8_t lsm[];
    uint16_t* buf = reinterpret_cast<uint16_t*>(lsm);                     // [kSeedCapScores]
    unsigned* whist = reinterpret_cast<unsigned*>(buf + kSeedCapScores);  // [warps][256]
    __shared__ unsigned hist[256];
    __shared__ uint32_t s_prefix, s_mask;
    __shared__ unsigned s_want;
    const int qi = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const float* src = scores + (long long)qi * query_stride;
    if (total > kSeedCapScores) total = kSeedCapScores;
    auto ordered = [](float v) { return v == v ? float_to_ordered(v) >> 16 : 0u; };  // NaN (no document) sorts last
    if ((query_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(scores) & 15u) == 0) {
        const float4* src4 = reinterpret_cast<const float4*>(src);
        const int n4 = total >> 2;
        for (int i0 = threadIdx.x; i0 < n4; i0 += 4 * kListThreads) {  // four independent 16-byte loads in flight
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (i0 + u * kListThreads < n4) v[u] = src4[i0 + u * kListThreads];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * kListThreads;
                if (i < n4)
                    reinterpret_cast<uint2*>(buf)[i] = make_uint2(ordered(v[u].x) | (ordered(v[u].y) << 16),
                                                                  ordered(v[u].z) | (ordered(v[u].w) << 16));
            }
        }
        for (int i = (n4 << 2) + threadIdx.x; i < total; i += blockDim.x) buf[i] = (uint16_t)ordered(src[i]);
    } else {
        for (int i = threadIdx.x; i < total; i += blockDim.x) buf[i] = (uint16_t)ordered(src[i]);
    }
    if (threadIdx.x == 0) {
        s_prefix = 0;
        s_mask = 0;
        s_want = (unsigned)k;
    }
    __syncthreads();
    if (total < k) {
        if (threadIdx.x == 0) tau[qi] = 0;
        return;
    }
    for (int shift = 8; shift >= 0; shift -= 8) {
        for (int i = lane; i < 256; i += 32) whist[warp * 256 + i] = 0;
        __syncwarp();
        const uint32_t pre = s_prefix, mask = s_mask;
        for (int i = threadIdx.x; i < total; i += blockDim.x) {
            const uint32_t key = buf[i];
            if ((key & mask) == pre) atomicAdd(&whist[warp * 256 + ((key >> shift) & 0xffu)], 1u);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < 256; i += blockDim.x) {
            unsigned sum = 0;
            for (int w = 0; w < nwarps; ++w) sum += whist[w * 256 + i];
            hist[i] = sum;
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            int d;
            unsigned nw;
            warp_pick_digit(hist, s_want, lane, &d, &nw);
            __syncwarp();
            if (lane == 0) {
                s_want = nw;
                s_prefix = pre | ((uint32_t)d << shift);
                s_mask = mask | (0xffu << shift);
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) tau[qi] = s_prefix != 0 ? ((u64)s_prefix << 48) - 1 : 0;
}

// ------------------------------------------------------------------------------------------
// merge: one CTA per query; block-wide radix select of the k-th largest key over all candidate
// segments (read from global / L2), gather of the survivors, bitonic sort by one warp.
// ------------------------------------------------------------------------------------------
constexpr int kMergeThreads = 512;

__global__ void __launch_bounds__(kMergeThreads)
tq_merge_kernel(const u64* __restrict__ cand, long long query_stride, long long seg_stride, int n_segs, int seg_len,
                const int* __restrict__ counts, int k, long long id_base, long long* __restrict__ out_ids,
                float* __restrict__ out_scores, u64* __restrict__ out_keys) {
    __shared__ unsigned hist[256];
    __shared__ u64 s_prefix, s_mask;
    __shared__ unsigned s_want;
    __shared__ int s_total, s_fill;
    __shared__ u64 sel[kTqWideK];
    const int qi = blockIdx.x;
    const u64* base = cand + (long long)qi * query_stride;
    const int* cnts = counts != nullptr ? counts + (long long)qi * n_segs : nullptr;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    // visits every stored key: a warp per segment, a lane per entry (only the entries in use when counts are given);
    // the whole warp calls f together (key 0 for the lanes past the end), so f may use full-warp primitives
    auto for_each_key = [&](auto&& f) {
        for (int seg = warp; seg < n_segs; seg += nwarps) {
            const int c = cnts != nullptr ? min(cnts[seg], seg_len) : seg_len;
            const u64* sp = base + (long long)seg * seg_stride;
            for (int off0 = 0; off0 < c; off0 += 32) f(off0 + lane < c ? sp[off0 + lane] : 0ull);
        }
    };

    // number of non-empty candidates
    if (threadIdx.x == 0) {
        s_total = 0;
        s_fill = 0;
    }
    for (int i = threadIdx.x; i < kTqWideK; i += blockDim.x) sel[i] = 0;
    __syncthreads();
    int local = 0;
    for_each_key([&](u64 key) { local += key != 0; });
    for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    if (lane == 0 && local) atomicAdd(&s_total, local);
    __syncthreads();
    const int total = s_total;
    const int kk = total < k ? total : k;
    u64 thr = 1;  // keep every non-empty key
    if (total > k) {
        if (threadIdx.x == 0) {
            s_prefix = 0;
            s_mask = 0;
            s_want = (unsigned)k;
        }
        for (int shift = 56; shift >= 0; shift -= 8) {
            for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
            __syncthreads();
            const u64 prefix = s_prefix, mask = s_mask;
            for_each_key([&](u64 key) {
                if (key != 0 && (key & mask) == prefix) atomicAdd(&hist[(unsigned)(key >> shift) & 0xffu], 1u);
            });
            __syncthreads();
            if (threadIdx.x < 32) {
                int d;
                unsigned nw;
                warp_pick_digit(hist, s_want, lane, &d, &nw);
                __syncwarp();
                if (lane == 0) {
                    s_want = nw;
                    s_prefix = prefix | ((u64)(unsigned)d << shift);
                    s_mask = mask | ((u64)0xffu << shift);
                }
            }
            __syncthreads();
        }
        thr = s_prefix;
    }
    for_each_key([&](u64 key) {
        if (key != 0 && key >= thr) {
            const int pos = atomicAdd(&s_fill, 1);
            if (pos < kTqWideK) sel[pos] = key;
        }
    });
    __syncthreads();
    if (warp == 0) {
        // bitonic sort of the selected keys, descending; empty slots (0) sink to the end
        for (int size = 2; size <= kTqWideK; size <<= 1) {
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                for (int tt = lane; tt < kTqWideK / 2; tt += 32) {
                    const int i = 2 * tt - (tt & (stride - 1));
                    const int j = i + stride;
                    const bool desc = (i & size) == 0;
                    const u64 x = sel[i], y = sel[j];
                    if ((x < y) == desc) {
                        sel[i] = y;
                        sel[j] = x;
                    }
                }
                __syncwarp();
            }
        }
        for (int i = lane; i < k; i += 32) {
            const u64 key = i < kk ? sel[i] : 0;
            if (out_keys != nullptr) out_keys[(long long)qi * k + i] = key;
            if (out_ids != nullptr) {
                out_ids[(long long)qi * k + i] =
                    key != 0 ? id_base + (long long)(0xffffffffu - (uint32_t)(key & 0xffffffffu)) : -1;
                out_scores[(long long)qi * k + i] = key != 0 ? ordered_to_float((uint32_t)(key >> 32)) : -INFINITY;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// multi-vector parents (runtime/retrieval_multivector_turboquant.go:746-810): per (row, parent)
// the 5 best child scores in descending order, then the aggregate.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
parent_agg_kernel(const float* __restrict__ scores, long long stride, int rows, const int* __restrict__ child_order,
                  const int* __restrict__ offsets, int parents, int top_n, double penalty, float* __restrict__ agg) {
    const long long total = (long long)rows * parents;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int row = (int)(i / parents), p = (int)(i % parents);
        const int c0 = offsets[p], c1 = offsets[p + 1];
        float top[5];
        int kept = 0;
        const float* sr = scores + (long long)row * stride;
        for (int c = c0; c < c1; ++c) {
            const float sc = sr[child_order[c]];
            if (kept < 5) {
                top[kept++] = sc;
            } else if (sc > top[4]) {
                top[4] = sc;
            } else {
                continue;
            }
            for (int j = kept - 1; j > 0 && top[j] > top[j - 1]; --j) {
                const float t = top[j];
                top[j] = top[j - 1];
                top[j - 1] = t;
            }
        }
        float out = 0.f;
        if (kept > 0) {
            int avail = top_n <= 0 ? 1 : top_n;
            if (avail > kept) avail = kept;
            double sum = 0.0;
            for (int j = 0; j < avail; ++j) sum += (double)top[j];
            double sc = sum / (double)avail;
            if (penalty != 0.0) sc -= penalty * log1p((double)(c1 - c0));
            out = (float)sc;
        }
        agg[i] = out;
    }
}

__global__ void __launch_bounds__(256)
parent_key_kernel(const float* __restrict__ agg, int rows, const int* __restrict__ offsets, int parents,
                  u64* __restrict__ keys) {
    for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < parents; p += gridDim.x * blockDim.x) {
        if (offsets[p + 1] == offsets[p]) {
            keys[p] = 0;
            continue;
        }
        float sum = agg[p];
        for (int r = 1; r < rows; ++r) sum += agg[(long long)r * parents + p];
        keys[p] = make_key(sum, (uint32_t)p);
    }
}

}  // namespace

// SMs of the current device (set by tq_scan_init; grids of the grid-stride kernels are multiples of it)
static int g_sm_count = 148;

// ------------------------------------------------------------------------------------------
// wide path: every score of a query chunk is materialised (scan kernels with all_scores), optionally corrected by
// the sign stage of the inner-product quantiser, turned into sortable keys and selected by tq_merge_kernel.  It
// serves k in (128, 256] (over-fetch before a rerank, runtime/retrieval_turboquant.go:1610-1662) and the rows bound
// as turboquant.IPQuantized{MSE, Signs, ResNorm, Norm} (runtime/turboquant_quantized_vector.go:43-49).
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
tq_score_keys_kernel(const float* __restrict__ scores, long long score_stride, int queries, long long n,
                     long long key_stride, u64* __restrict__ keys) {
    const long long total = (long long)queries * key_stride;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long q = i / key_stride, r = i - q * key_stride;
        keys[i] = r < n ? make_key(scores[q * score_stride + r], (uint32_t)r) : 0ull;
    }
}

constexpr int kIpQueryGroup = 4;

// scores[q, row] += norm[row] * resnorm[row] * qjl_scale * sum_i sketch[q, i] * (sign bit i of row ? +1 : -1).
// One warp per row; the sketches of kIpQueryGroup queries sit in shared memory bit-major ([q][bit][word]) so that the
// 32 lanes, one sign word each, read consecutive addresses.  sum = 2 * (sum over set bits) - (sum of the sketch).
__global__ void __launch_bounds__(256)
tq_ip_sign_stage_kernel(const uint32_t* __restrict__ signs, int words, const float* __restrict__ resnorms,
                        const float* __restrict__ norms, long long n, const float* __restrict__ sketch, int queries,
                        int dim, float qjl_scale, float* __restrict__ scores, long long score_stride) {
    extern __shared__ float ip_smem[];
    float* sq = ip_smem;                                       // [kIpQueryGroup][32][words]
    float* tot = ip_smem + (size_t)kIpQueryGroup * 32 * words;  // [kIpQueryGroup]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int q0 = 0; q0 < queries; q0 += kIpQueryGroup) {
        const int qn = min(kIpQueryGroup, queries - q0);
        __syncthreads();
        for (int i = threadIdx.x; i < kIpQueryGroup * 32 * words; i += blockDim.x) {
            const int q = i / (32 * words), rem = i - q * 32 * words;
            const int coord = rem;                              // coordinate = word * 32 + bit
            const int w = coord >> 5, b = coord & 31;
            sq[((size_t)q * 32 + b) * words + w] = (q < qn && coord < dim) ? sketch[(size_t)(q0 + q) * dim + coord] : 0.f;
        }
        __syncthreads();
        if (warp < kIpQueryGroup) {
            float t = 0.f;
            for (int i = lane; i < 32 * words; i += 32) t += sq[(size_t)warp * 32 * words + i];
            t = warp_sum(t);
            if (lane == 0) tot[warp] = t;
        }
        __syncthreads();
        for (long long row = (long long)blockIdx.x * 8 + warp; row < n; row += (long long)gridDim.x * 8) {
            float acc[kIpQueryGroup];
#pragma unroll
            for (int q = 0; q < kIpQueryGroup; ++q) acc[q] = 0.f;
            for (int w = lane; w < words; w += 32) {
                const uint32_t bits = __ldg(signs + row * words + w);
#pragma unroll 8
                for (int b = 0; b < 32; ++b) {
                    const bool on = (bits >> b) & 1u;
#pragma unroll
                    for (int q = 0; q < kIpQueryGroup; ++q) {
                        const float v = sq[((size_t)q * 32 + b) * words + w];
                        acc[q] += on ? v : 0.f;
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < kIpQueryGroup; ++q) acc[q] = warp_sum(acc[q]);
            const float scale = __ldg(norms + row) * __ldg(resnorms + row) * qjl_scale;
            if (lane < qn) {
                float mine = acc[0];
#pragma unroll
                for (int q = 1; q < kIpQueryGroup; ++q) mine = lane == q ? acc[q] : mine;
                float* dst = scores + (long long)(q0 + lane) * score_stride + row;
                *dst = *dst + scale * (2.f * mine - tot[lane]);
            }
        }
    }
}

void launch_parent_keys(const float* scores, long long stride, int rows, const int* child_order, const int* offsets,
                        int parents, int top_n, double penalty, float* agg_scratch, uint64_t* keys,
                        cudaStream_t stream) {
    parent_agg_kernel<<<g_sm_count * 8, 256, 0, stream>>>(scores, stride, rows, child_order, offsets, parents, top_n, penalty,
                                                   agg_scratch);
    parent_key_kernel<<<(parents + 255) / 256, 256, 0, stream>>>(agg_scratch, rows, offsets, parents,
                                                                 reinterpret_cast<u64*>(keys));
}

void launch_tq_pack(const float* x, int64_t n, const TqSpec& spec, uint8_t* codes, float* norms,
                    cudaStream_t stream) {
    if (n <= 0) return;
    // 2 float rows per warp within the default 48 KB of dynamic shared memory: 8 warps up to dim 768
    int warps = 6144 / spec.dim;
    warps = warps > 8 ? 8 : (warps < 1 ? 1 : warps);
    const size_t smem = (size_t)warps * 2 * spec.dim * sizeof(float);
    long long blocks = (n + warps - 1) / warps;
    if (blocks > (long long)g_sm_count * 8) blocks = (long long)g_sm_count * 8;
    tq_norms_kernel<<<(int)((n + 255) / 256), 256, 0, stream>>>(x, (long long)n, spec.dim, norms);
    tq_pack_kernel<<<(int)blocks, warps * 32, smem, stream>>>(x, (long long)n, spec, codes, norms);
}

void launch_tq_transcode(const uint8_t* codes, int64_t n, int dim, int bits, uint8_t* tiles, cudaStream_t stream) {
    if (n <= 0) return;
    tq_transcode_kernel<<<g_sm_count * 8, 256, 0, stream>>>(codes, (long long)n, dim, bits,
                                                     reinterpret_cast<uint32_t*>(tiles));
}

void launch_tq_prepare(const float* queries, int q, int q_fill, const TqSpec& spec, uint2* bfrag, float* rotated_out,
                       __half* qperm, cudaStream_t stream) {
    if (q <= 0) return;
    const int warps = 4;
    const size_t smem = (size_t)warps * 3 * spec.dim * sizeof(float);
    const int q_padded = q_fill;
    int blocks = (q_padded + warps - 1) / warps;
    if (blocks > (long long)g_sm_count * 4) blocks = (long long)g_sm_count * 4;
    tq_prepare_kernel<<<blocks, warps * 32, smem, stream>>>(queries, q, q_fill, spec, tq_ksteps(spec.dim), bfrag,
                                                            rotated_out, qperm);
}

// Empty when every kernel of the scoring path can be launched for vectors of this dimension, else the reason:
// the widest users of shared memory are the prepare kernel (3 float rows per warp) and the 32-query scan (the
// query fragments of four tiles), both limited to the 200 KB the kernels ask for.
std::string tq_check_dim(int dim) {
    const size_t limit = 200 * 1024;
    const size_t prepare = (size_t)4 * 3 * dim * sizeof(float);
    const size_t scan = tq_scan_smem_bytes(4, dim);
    if (prepare > limit || scan > limit || dim > 6144)
        return "dim " + std::to_string(dim) + " is too wide for the scoring kernels (shared memory: prepare " +
               std::to_string(prepare) + " B, scan " + std::to_string(scan) + " B, limit " + std::to_string(limit) + " B)";
    return "";
}

size_t tq_scan_smem_bytes(int query_tiles, int dim) {
    if (query_tiles != 1 && query_tiles != 2 && query_tiles != 4) return 0;
    const int qb = 8 * query_tiles;
    return (size_t)query_tiles * tq_ksteps(dim) * 32 * 8 + (size_t)qb * kScanCap * 8 + (size_t)qb * 8 +
           (size_t)qb * 4 + (size_t)kTqScanWarps * 256 * 4;
}

cudaError_t tq_scan_init() {
    {
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0)
            g_sm_count = sms;
    }
    const int max_smem = 200 * 1024;
    cudaError_t e = cudaFuncSetAttribute(tq_scan_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(tq_scan_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(tq_scan_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(tq_scan_stream_kernel<48>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(tq_scan_stream_kernel<24>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(tq_scan_stream_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(tq_scan_stream_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(tq_pack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(tq_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    return e;
}

void launch_tq_scan(const TqScanArgs& a, cudaStream_t stream) {
    if (a.query_tiles == 1) {
        const int ks = tq_ksteps(a.dim);
        const int threads = kStreamWarps * 32;
        if (ks == 48) { tq_scan_stream_kernel<48><<<a.grid, threads, tq_stream_smem<48>(), stream>>>(a); return; }
        if (ks == 24) { tq_scan_stream_kernel<24><<<a.grid, threads, tq_stream_smem<24>(), stream>>>(a); return; }
        if (ks == 16) { tq_scan_stream_kernel<16><<<a.grid, threads, tq_stream_smem<16>(), stream>>>(a); return; }
        if (ks == 8) { tq_scan_stream_kernel<8><<<a.grid, threads, tq_stream_smem<8>(), stream>>>(a); return; }
    }
    const size_t smem = tq_scan_smem_bytes(a.query_tiles, a.dim);
    const int threads = kTqScanWarps * 32;
    if (a.query_tiles == 1) tq_scan_kernel<1><<<a.grid, threads, smem, stream>>>(a);
    else if (a.query_tiles == 2) tq_scan_kernel<2><<<a.grid, threads, smem, stream>>>(a);
    else tq_scan_kernel<4><<<a.grid, threads, smem, stream>>>(a);
}

cudaError_t tq_merge_init() {
    cudaError_t e = cudaFuncSetAttribute(tq_merge_lists_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kListCapKeys * 8 + (kListMaxSegs + 1) * 4);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(tq_seed_tau_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kSeedCapScores * 2 + (kListThreads / 32) * 256 * 4);
    return e;
}

void launch_tq_merge_lists(const uint64_t* cand, int64_t query_stride, int64_t seg_stride, int n_segs, int seg_len,
                           const int* counts, int queries, int k, int64_t* out_ids, float* out_scores, uint64_t* out_keys,
                           cudaStream_t stream) {
    if (queries <= 0) return;
    if (n_segs > kListMaxSegs) {  // more lists than the prefix table holds: the general merge
        launch_tq_merge(cand, query_stride, seg_stride, n_segs, seg_len, counts, queries, k, 0, out_ids, out_scores,
                        out_keys, stream);
        return;
    }
    tq_merge_lists_kernel<<<queries, kListThreads, kListCapKeys * 8 + (n_segs + 1) * 4, stream>>>(
        reinterpret_cast<const u64*>(cand), (long long)query_stride, (long long)seg_stride, n_segs, seg_len, counts, k,
        reinterpret_cast<long long*>(out_ids), out_scores, reinterpret_cast<u64*>(out_keys));
}

void launch_tq_seed_tau_scores(const float* scores, int64_t query_stride, int total, int queries, int k,
                               unsigned long long* tau, cudaStream_t stream) {
    if (queries <= 0) return;
    tq_seed_tau_scores_kernel<<<queries, kListThreads, kSeedCapScores * 2 + (kListThreads / 32) * 256 * 4, stream>>>(
        scores, (long long)query_stride, total, k, tau);
}

void launch_tq_merge(const uint64_t* cand, int64_t query_stride, int64_t seg_stride, int n_segs, int seg_len,
                     const int* counts, int queries, int k, int64_t id_base, int64_t* out_ids, float* out_scores,
                     uint64_t* out_keys, cudaStream_t stream) {
    if (queries <= 0) return;
    tq_merge_kernel<<<queries, kMergeThreads, 0, stream>>>(
        reinterpret_cast<const u64*>(cand), (long long)query_stride, (long long)seg_stride, n_segs, seg_len, counts,
        k, (long long)id_base, reinterpret_cast<long long*>(out_ids), out_scores, reinterpret_cast<u64*>(out_keys));
}

void launch_dense_keys(const void* docs, bool docs_f16, int64_t n_rows, int dim, const float* queries, int nq,
                       const int64_t* cand_ids, int64_t cand, int metric, uint64_t* keys, int sm_count,
                       cudaStream_t stream) {
    if (nq <= 0 || cand <= 0) return;
    const int grid = sm_count * 8;
    if (docs_f16)
        dense_keys_kernel<true><<<grid, 256, 0, stream>>>(docs, (long long)n_rows, dim, queries, nq,
                                                          reinterpret_cast<const long long*>(cand_ids), (long long)cand,
                                                          metric, reinterpret_cast<u64*>(keys));
    else
        dense_keys_kernel<false><<<grid, 256, 0, stream>>>(docs, (long long)n_rows, dim, queries, nq,
                                                           reinterpret_cast<const long long*>(cand_ids), (long long)cand,
                                                           metric, reinterpret_cast<u64*>(keys));
}

void launch_tq_score_keys(const float* scores, int64_t score_stride, int queries, int64_t n, int64_t key_stride,
                          uint64_t* keys, int sm_count, cudaStream_t stream) {
    if (queries <= 0 || key_stride <= 0) return;
    tq_score_keys_kernel<<<sm_count * 8, 256, 0, stream>>>(scores, (long long)score_stride, queries, (long long)n,
                                                          (long long)key_stride, reinterpret_cast<u64*>(keys));
}

size_t tq_ip_sign_stage_smem(int dim) {
    const int words = (dim + 31) / 32;
    return ((size_t)kIpQueryGroup * 32 * words + kIpQueryGroup) * sizeof(float);
}

cudaError_t tq_ip_init() {
    return cudaFuncSetAttribute(tq_ip_sign_stage_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
}

void launch_tq_ip_sign_stage(const uint32_t* signs, const float* resnorms, const float* norms, int64_t n,
                             const float* sketch, int queries, int dim, float qjl_scale, float* scores,
                             int64_t score_stride, int sm_count, cudaStream_t stream) {
    if (n <= 0 || queries <= 0) return;
    const int words = (dim + 31) / 32;
    long long blocks = (n + 7) / 8;
    if (blocks > (long long)sm_count * 4) blocks = (long long)sm_count * 4;
    tq_ip_sign_stage_kernel<<<(int)blocks, 256, tq_ip_sign_stage_smem(dim), stream>>>(
        signs, words, resnorms, norms, (long long)n, sketch, queries, dim, qjl_scale, scores, (long long)score_stride);
}

}  // namespace eosb
