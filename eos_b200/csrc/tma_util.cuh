// Host helper: 2-D tiled TMA descriptors through cuTensorMapEncodeTiled, resolved at run time with
// cudaGetDriverEntryPoint so the library has no link-time dependency on libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace eosb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn(std::string* err) {
    static EncodeTiledFn fn = nullptr;
    if (fn != nullptr) return fn;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
    if (e != cudaSuccess || sym == nullptr || qres != cudaDriverEntryPointSuccess) {
        *err = std::string("cuTensorMapEncodeTiled is not available: ") + cudaGetErrorString(e);
        return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(sym);
    return fn;
}

inline std::string encode_2d(CUtensorMap* tm, CUtensorMapDataType dt, const void* ptr, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw) {
    std::string err;
    EncodeTiledFn fn = get_encode_fn(&err);
    if (fn == nullptr) return err;
    if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0) return "tensor map base address is not 16-byte aligned";
    if ((row_stride_bytes & 15u) != 0) return "tensor map row stride is not a multiple of 16 bytes";
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(tm, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r);
    return "";
}


}  // namespace eosb
