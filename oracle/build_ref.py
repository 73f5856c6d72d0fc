"""Builds oracle/_ref/libturboq_ref.so from the reference's OWN TurboQuant encode / decode code.

TEST INFRASTRUCTURE ONLY (the checker's checker): nothing in the shipped library uses it.

The reference (Go) cannot be built here, but its device restatement of the TurboQuant Hadamard/MSE encode and
decode is plain C inside a Go raw string: `turboQKernelSource`,
runtime/backends/cuda/native_linux.go:1812-2003 (manta_turboq_encode / manta_turboq_decode, one thread per
vector).  This script reads that string from the reference tree where it lies, at build time, prepends a few
host shims (empty __device__ / __global__, a settable blockIdx / blockDim / threadIdx, rsqrtf as 1/sqrtf) and
a C driver that runs the "kernel" once per vector, and pipes the result to g++ through stdin: no reference
source text is written into this repository, only the compiled library under oracle/_ref/ (git-ignored).

Flags match oracle/Makefile (-ffp-contract=off, no -march): float expressions evaluate as written.
The one deliberate difference from the device build of the same string is rsqrtf: the GPU's is an approximation,
the shim's is the correctly rounded 1/sqrtf (the same choice the C restatement in eos_oracle.c states).
"""
from __future__ import annotations

import os
import re
import subprocess
from typing import Optional

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libturboq_ref.so")
REF_FILE = os.path.join("runtime", "backends", "cuda", "native_linux.go")

_SHIMS = r"""
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#define __device__
#define __global__
namespace { struct Idx3 { int x, y, z; }; }
static thread_local Idx3 blockIdx = {0, 0, 0}, blockDim = {1, 1, 1}, threadIdx = {0, 0, 0};
static inline float rsqrtf(float v) { return 1.0f / sqrtf(v); }
"""

_DRIVER = r"""
extern "C" __attribute__((visibility("default")))
void ref_turboq_encode(const float* input, float* coords, float* norms, const float* perm, const float* signs1,
                       const float* signs2, const float* centroids, const float* boundaries, int vectors,
                       int channels, int levels) {
    float* work = (float*)malloc(sizeof(float) * (size_t)vectors * channels);
    float* rot = (float*)malloc(sizeof(float) * (size_t)vectors * channels);
    blockDim.x = 1;
    threadIdx.x = 0;
    /* [N, C, H, W] with C = channels, H = 1, W = 1: vector v is n = v, its channels contiguous */
    for (int v = 0; v < vectors; ++v) {
        blockIdx.x = v;
        manta_turboq_encode(input, coords, norms, work, rot, perm, signs1, signs2, centroids, boundaries, vectors,
                            channels, 1, 1, levels);
    }
    free(work);
    free(rot);
}
extern "C" __attribute__((visibility("default")))
void ref_turboq_decode(const float* coords, const float* norms, float* out, const float* perm, const float* signs1,
                       const float* signs2, const float* centroids, int vectors, int channels, int levels) {
    float* work = (float*)malloc(sizeof(float) * (size_t)vectors * channels);
    float* rot = (float*)malloc(sizeof(float) * (size_t)vectors * channels);
    blockDim.x = 1;
    threadIdx.x = 0;
    for (int v = 0; v < vectors; ++v) {
        blockIdx.x = v;
        manta_turboq_decode(coords, norms, out, work, rot, perm, signs1, signs2, centroids, vectors, channels, 1, 1,
                            levels);
    }
    free(work);
    free(rot);
}
extern "C" __attribute__((visibility("default")))
int ref_turboq_norm_code(float norm) { return manta_tq_quantize_norm(norm); }
extern "C" __attribute__((visibility("default")))
float ref_turboq_norm_value(int code) { return manta_tq_dequantize_norm(code); }
"""


def _extract(ref_root: str) -> str:
    text = open(os.path.join(ref_root, REF_FILE), encoding="utf-8").read()
    m = re.search(r"const turboQKernelSource = `(.*?)`", text, re.S)
    if m is None:
        raise RuntimeError("turboQKernelSource not found in " + REF_FILE)
    return m.group(1)


def build(ref_root: str = "/root/reference", force: bool = False) -> Optional[str]:
    """Returns the library path, or None when neither the reference tree nor a prebuilt library is present."""
    src_path = os.path.join(ref_root, REF_FILE)
    if not os.path.exists(src_path):
        return LIB if os.path.exists(LIB) else None
    if os.path.exists(LIB) and not force and os.path.getmtime(LIB) >= max(os.path.getmtime(src_path),
                                                                           os.path.getmtime(__file__)):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    program = _SHIMS + _extract(ref_root) + _DRIVER
    cmd = ["g++", "-x", "c++", "-O2", "-fPIC", "-ffp-contract=off", "-fvisibility=hidden", "-shared", "-o", LIB, "-",
           "-lm"]
    subprocess.run(cmd, input=program.encode("utf-8"), check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
