// Host-side interface of the tcgen05 GEMM (gemm_tc.cu).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace eosb {

// Epilogue applied to acc[m,n] * scale[n] + bias[n] before the f16 store.
enum GemmEpilogue : int {
    kEpiBias = 0,          // plain projection
    kEpiBiasGeluErf = 1,   // FFN up-projection, erf GELU
    kEpiBiasResidual = 2,  // projection + residual (input of a post-LayerNorm)
    kEpiBiasGeluTanh = 3   // FFN up-projection, tanh GELU (compact encoder profile)
};

struct GemmParams {
    const int* m_ptr;       // device scalar: rows actually in use (clamped to m_alloc); may be null
    int m_alloc;            // rows covered by the A / out allocations
    int n;                  // output features
    int k;                  // input features
    const float* scale;     // [n] per-output-channel dequant scale, or null (= 1)
    const float* bias;      // [n] or null (= 0)
    const __half* residual; // [m, ldr] for kEpiBiasResidual
    int ldr;
    __half* out;            // [m, ldo]
    int ldo;
    int mode;               // GemmEpilogue
    int* status;            // device status word (receives kStatusPipelineTimeout on a bounded-wait failure)
};

struct GemmPlan {
    CUtensorMap tm_a;
    CUtensorMap tm_b;
    CUtensorMap tm_out;   // output rows, boxes of 32 rows x 32 columns (the epilogue's staging slabs, 64-byte swizzle)
    GemmParams p;
    int grid;
    bool b_int8;
    bool pair;  // two CTAs of a cluster per 256x256 tile (f16 weights)
};

// Builds the TMA descriptors for out[m, n] = A[m, k] (f16, row stride lda elements) x W[n, k]^T.
// W is either biased-uint8 codes (value + 128, row stride ldw bytes) when b_int8, or f16 (row
// stride ldw elements).  k, lda (and ldw) must keep every row start 16-byte aligned.
// Returns an empty string on success, else the error text.
std::string gemm_make_plan(GemmPlan* plan, const __half* a, int lda, const void* w, int ldw, bool b_int8,
                           const GemmParams& params, int sm_count);

void gemm_launch(const GemmPlan& plan, cudaStream_t stream);

// One-time per process: raises the dynamic shared memory limit of the kernels and asks the driver how
// many CTA pairs fit on the device for the CTA-pair kernel, which serves deep or wide f16-weight projections
// (K >= 2048, or N >= 2048 with K >= 768; environment EOS_B200_GEMM_CTA_PAIR=1: every f16-weight projection, =0: none).
std::string gemm_global_init();

}  // namespace eosb
