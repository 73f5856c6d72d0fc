// Device helpers shared by the TurboQuant scoring kernels: the scan-tile layout, the sortable candidate keys, the
// warp sort that cuts a candidate list and the register expansion of 4-bit codes to f16.
#pragma once
#include <stdint.h>

#include "turboquant.cuh"

namespace eosb {

typedef unsigned long long u64;

// ------------------------------------------------------------------------------------------
// scan layout.  A tile = 16 documents.  For chunk c (128 coordinates = 8 MMA k-steps), lane
// (g = lane/4, t = lane%4) owns 32 bytes at tile + c*1024 + lane*32: a uint4 for document g and
// a uint4 for document g+8.  Word i of a uint4 covers k-steps 8c+2i and 8c+2i+1; its element
// e = 2q+h (q = 0..3, h = 0,1) is coordinate 16*(8c+2i+(q>>1)) + 2t + 8*(q&1) + h, magnitude
// index in bits [4e, 4e+3), sign (1 = negative) in bit 8e+7 for e < 4 and bit 8(e-4)+3 for e >= 4: the
// signs of elements 0..3 (4..7) sit on (4 bits below) the top bit of the byte that the high-byte
// lookup of their magnitudes yields, so one AND-XOR applies four of them.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ int scan_coord(int c, int i, int t, int e) {
    const int q = e >> 1, h = e & 1;
    return 16 * (8 * c + 2 * i + (q >> 1)) + 2 * t + 8 * (q & 1) + h;
}


// ------------------------------------------------------------------------------------------
// keys: (order-preserving score bits << 32) | (0xffffffff - doc index): larger key = better
// candidate under "score descending, then id ascending"; 0 = empty.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t float_to_ordered(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ordered_to_float(uint32_t o) {
    return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
}
__device__ __forceinline__ u64 make_key(float score, uint32_t doc) {
    return ((u64)float_to_ordered(score) << 32) | (u64)(0xffffffffu - doc);
}

// Radix-select the k-th largest of keys[0..n) (distinct, n > k >= 1) with one warp.
// hist: 256 counters of shared memory owned by the warp.
__device__ inline u64 warp_kth_largest(const u64* keys, int n, int k, unsigned* hist, int lane) {
    u64 prefix = 0, mask = 0;
    unsigned want = (unsigned)k;
    for (int shift = 56; shift >= 0; shift -= 8) {
        for (int i = lane; i < 256; i += 32) hist[i] = 0;
        __syncwarp();
        for (int i = lane; i < n; i += 32) {
            const u64 key = keys[i];
            if ((key & mask) == prefix) atomicAdd(&hist[(unsigned)(key >> shift) & 0xffu], 1u);
        }
        __syncwarp();
        unsigned c[8], s = 0;
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            c[b] = hist[lane * 8 + b];
            s += c[b];
        }
        unsigned incl = s;  // sum over lanes >= this one (higher lanes own higher digits)
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned tmp = __shfl_down_sync(0xffffffffu, incl, o);
            if (lane + o < 32) incl += tmp;
        }
        const unsigned above = incl - s;
        const bool mine = (above < want) && (want <= incl);
        int d = 0;
        unsigned next_want = 0;
        if (mine) {
            unsigned run = above;
#pragma unroll
            for (int b = 7; b >= 0; --b) {
                if (next_want == 0) {
                    if (run + c[b] >= want) {
                        d = lane * 8 + b;
                        next_want = want - run;
                    } else {
                        run += c[b];
                    }
                }
            }
        }
        const unsigned bal = __ballot_sync(0xffffffffu, mine);
        const int src = bal ? (__ffs(bal) - 1) : 0;
        d = __shfl_sync(0xffffffffu, d, src);
        want = __shfl_sync(0xffffffffu, next_want, src);
        prefix |= (u64)(unsigned)d << shift;
        mask |= (u64)0xffu << shift;
        __syncwarp();
    }
    return prefix;
}


// Bitonic sort of the kSortCap = 256 slots of a list in shared memory by one warp, descending; slots from n on are
// cleared first (empty = 0 sinks to the end).  Measured faster here than the 8-pass radix select for a few hundred
// keys, and faster than the same network held in registers (whose unrolled code is long and rarely executed).
constexpr int kSortCap = 256;
__device__ __forceinline__ void warp_sort_desc(u64* keys, int n, int lane) {
    for (int i = n + lane; i < kSortCap; i += 32) keys[i] = 0;
    __syncwarp();
    for (int size = 2; size <= kSortCap; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
#pragma unroll
            for (int tt = lane; tt < kSortCap / 2; tt += 32) {
                const int i = 2 * tt - (tt & (stride - 1));
                const int j = i + stride;
                const bool desc = (i & size) == 0;
                const u64 x = keys[i], y = keys[j];
                if ((x < y) == desc) {
                    keys[i] = y;
                    keys[j] = x;
                }
            }
            __syncwarp();
        }
    }
}


// 8 sign-magnitude nibbles -> 4 half2 (elements 0/1, 2/3, 4/5, 6/7)
__device__ __forceinline__ void dequant8(uint32_t w, uint32_t hi_a, uint32_t hi_b, uint32_t lo_a, uint32_t lo_b,
                                         uint32_t (&v)[4]) {
    const uint32_t m = w & 0x77777777u;
    const uint32_t mh = m >> 16;
    const uint32_t h0 = __byte_perm(hi_a, hi_b, m) ^ (w & 0x80808080u), l0 = __byte_perm(lo_a, lo_b, m);
    const uint32_t h1 = __byte_perm(hi_a, hi_b, mh) ^ ((w << 4) & 0x80808080u), l1 = __byte_perm(lo_a, lo_b, mh);
    v[0] = __byte_perm(l0, h0, 0x5140);
    v[1] = __byte_perm(l0, h0, 0x7362);
    v[2] = __byte_perm(l1, h1, 0x5140);
    v[3] = __byte_perm(l1, h1, 0x7362);
}


// ---------------------------------------------------------------- blocked Hadamard transform (packing, decoding)
__device__ __forceinline__ int highest_pow2_le(int v) {
    int p = 1;
    while ((p << 1) <= v) p <<= 1;
    return p;
}

// G consecutive butterfly stages (the first has distance 2^lg) of a block of `size` floats in shared memory, by one
// warp: a lane takes the 2^G elements that these stages combine among themselves, runs the stages in registers and
// writes them back, scaled by `scale` (1 except after the last stage).  Every butterfly is the a + b / a - b of the
// sequential form on the same pair, so the result is that form's bit for bit.
template <int G>
__device__ __forceinline__ void warp_fwht_stages(float* v, int size, int lg, float scale, int lane) {
    constexpr int E = 1 << G;
    const int stride = 1 << lg;
    const bool wide = G == 3 && lg == 0 && (reinterpret_cast<uintptr_t>(v) & 15u) == 0;   // 8 neighbours: two 16-byte accesses
    for (int p = lane; p < (size >> G); p += 32) {
        const int low = p & (stride - 1), high = p >> lg;
        float* b = v + ((high << (lg + G)) | low);
        float e[E];
        if (wide) {
            const float4 lo4 = reinterpret_cast<const float4*>(b)[0], hi4 = reinterpret_cast<const float4*>(b)[E > 4 ? 1 : 0];
            e[0] = lo4.x, e[1] = lo4.y;
            if (E > 2) e[2] = lo4.z, e[3] = lo4.w;
            if (E > 4) e[4] = hi4.x, e[5] = hi4.y, e[6] = hi4.z, e[7] = hi4.w;
        } else {
#pragma unroll
            for (int k = 0; k < E; ++k) e[k] = b[k * stride];
        }
#pragma unroll
        for (int st = 0; st < G; ++st) {
#pragma unroll
            for (int k = 0; k < E; ++k) {
                if ((k & (1 << st)) == 0) {
                    const float a = e[k], c = e[k | (1 << st)];
                    e[k] = __fadd_rn(a, c);
                    e[k | (1 << st)] = __fsub_rn(a, c);
                }
            }
        }
        if (scale != 1.0f) {
#pragma unroll
            for (int k = 0; k < E; ++k) e[k] = __fmul_rn(e[k], scale);
        }
        if (wide) {
            reinterpret_cast<float4*>(b)[0] = make_float4(e[0], e[1], e[E > 2 ? 2 : 0], e[E > 2 ? 3 : 0]);
            if (E > 4) reinterpret_cast<float4*>(b)[1] = make_float4(e[E > 4 ? 4 : 0], e[E > 4 ? 5 : 0], e[E > 4 ? 6 : 0], e[E > 4 ? 7 : 0]);
        } else {
#pragma unroll
            for (int k = 0; k < E; ++k) b[k * stride] = e[k];
        }
    }
    __syncwarp();
}

// In-place blocked normalised FWHT of `work` (shared memory) by one warp: blocks of the largest power of two that
// still fits, each transformed and multiplied by 1 / sqrt(size) (the reference's apply_blocks).  Stages run three at
// a time in registers; the scaling rides on the last group.
__device__ __forceinline__ void warp_fwht_blocks(float* work, int dim, int lane) {
    int offset = 0, remaining = dim;
    while (remaining > 0) {
        const int size = highest_pow2_le(remaining);
        float* v = work + offset;
        const int stages = 31 - __clz(size);
        const float scale = size > 1 ? __fdiv_rn(1.0f, __fsqrt_rn((float)size)) : 1.0f;
        int lg = 0;
        while (stages - lg > 3) {
            warp_fwht_stages<3>(v, size, lg, 1.0f, lane);
            lg += 3;
        }
        if (stages - lg == 3) warp_fwht_stages<3>(v, size, lg, scale, lane);
        else if (stages - lg == 2) warp_fwht_stages<2>(v, size, lg, scale, lane);
        else if (stages - lg == 1) warp_fwht_stages<1>(v, size, lg, scale, lane);
        offset += size;
        remaining -= size;
    }
}


}  // namespace eosb
