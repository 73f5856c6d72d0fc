// C ABI of libeos_b200.so (declarations and reference citations: include/eos_b200.h).
// Host-side orchestration only: argument validation, device memory, kernel sequencing.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <dlfcn.h>

#include <algorithm>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/eos_b200.h"
#include "common.cuh"
#include "attention_tc.cuh"
#include "encoder_kernels.cuh"
#include "gemm_tc.cuh"
#include "sparse_attention.cuh"
#include "token_pool.cuh"
#include "turboquant.cuh"

using namespace eosb;

// ------------------------------------------------------------------------------------------------
// helpers
// ------------------------------------------------------------------------------------------------
namespace {

char* dup_cstring(const std::string& s) {
    char* p = static_cast<char*>(std::malloc(s.size() + 1));
    if (p != nullptr) std::memcpy(p, s.c_str(), s.size() + 1);
    return p;
}

int fail(char** err, const std::string& msg, int code = EOS_B200_ERROR) {
    if (err != nullptr) *err = dup_cstring(msg);
    return code;
}

#define CUDA_TRY(expr)                                                                              \
    do {                                                                                            \
        cudaError_t e__ = (expr);                                                                   \
        if (e__ != cudaSuccess) {                                                                   \
            cudaGetLastError();                                                                     \
            return fail(err, std::string(#expr) + ": " + cudaGetErrorString(e__));                  \
        }                                                                                           \
    } while (0)

template <typename T>
cudaError_t dev_alloc(T** p, size_t count) {
    *p = nullptr;
    if (count == 0) count = 1;
    return cudaMalloc(reinterpret_cast<void**>(p), count * sizeof(T));
}

template <typename T>
void dev_free(T*& p) {
    if (p != nullptr) cudaFree(p);
    p = nullptr;
}

std::vector<__half> to_half(const float* src, size_t n) {
    std::vector<__half> out(n);
    for (size_t i = 0; i < n; ++i) out[i] = __float2half_rn(src[i]);
    return out;
}

cudaStream_t pick_stream(EosB200Runtime* rt, void* stream);

}  // namespace

struct EosB200Runtime {
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaDeviceProp prop{};
    int sm_count = 0;
    int* d_status = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
};

namespace {
cudaStream_t pick_stream(EosB200Runtime* rt, void* stream) {
    return stream != nullptr ? static_cast<cudaStream_t>(stream) : rt->stream;
}

// One warp waits on an mbarrier nobody ever arrives on, with the given limit; the wait gives up, and the kernel
// reports it through the status word exactly as the pipelines do.
__global__ void bounded_wait_probe_kernel(long long limit_cycles, int* status) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        mbar_fence_init();
    }
    __syncwarp();
    const bool ok = mbar_wait_limit(smem_u32(&bar), 0, &abort_flag, limit_cycles);
    __syncwarp();
    if (threadIdx.x == 0 && (!ok || abort_flag != 0)) atomicExch(status, kStatusPipelineTimeout);
}

int read_status(EosB200Runtime* rt, cudaStream_t s, char** err) {
    int st = 0;
    CUDA_TRY(cudaMemcpyAsync(&st, rt->d_status, sizeof(int), cudaMemcpyDeviceToHost, s));
    CUDA_TRY(cudaStreamSynchronize(s));
    if (st == kStatusOk) return EOS_B200_OK;
    cudaMemsetAsync(rt->d_status, 0, sizeof(int), s);  // reported once
    const char* what = "unknown device status";
    if (st == kStatusBadTokenId) what = "input_ids value out of range [0, vocab)";
    else if (st == kStatusBadTypeId) what = "token_type_ids value out of range";
    else if (st == kStatusBadPosition) what = "sequence longer than max_positions";
    else if (st == kStatusPipelineTimeout) what = "a bounded wait inside a kernel ran out (pipeline timeout)";
    return fail(err, std::string("device status ") + std::to_string(st) + ": " + what, EOS_B200_DEVICE_STATUS);
}
}  // namespace

extern "C" {

const char* eos_b200_version(void) { return "eos_b200 0.1 (sm_100a)"; }

void eos_b200_free_cstring(char* s) { std::free(s); }

int eos_b200_runtime_create(int device, EosB200Runtime** out, char** err) {
    if (out == nullptr) return fail(err, "runtime_create: out is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count <= 0) {
        cudaGetLastError();
        return fail(err, std::string("no CUDA device available (no CPU fallback): ") + cudaGetErrorString(e));
    }
    if (device < 0 || device >= count) return fail(err, "runtime_create: device index out of range");
    CUDA_TRY(cudaSetDevice(device));
    EosB200Runtime* rt = new EosB200Runtime();
    rt->device = device;
    e = cudaGetDeviceProperties(&rt->prop, device);
    if (e != cudaSuccess) {
        delete rt;
        return fail(err, std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(e));
    }
    if (rt->prop.major != 10) {
        std::string msg = "device '" + std::string(rt->prop.name) + "' is compute capability " +
                          std::to_string(rt->prop.major) + "." + std::to_string(rt->prop.minor) +
                          "; this library only contains sm_100a code (no fallback)";
        delete rt;
        return fail(err, msg);
    }
    rt->sm_count = rt->prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&rt->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreate(&rt->ev0) != cudaSuccess || cudaEventCreate(&rt->ev1) != cudaSuccess ||
        dev_alloc(&rt->d_status, 1) != cudaSuccess || cudaMemset(rt->d_status, 0, sizeof(int)) != cudaSuccess) {
        std::string msg = std::string("runtime_create: ") + cudaGetErrorString(cudaGetLastError());
        eos_b200_runtime_destroy(rt);
        return fail(err, msg);
    }
    std::string ge = gemm_global_init();
    if (ge.empty()) ge = attn_tc_global_init();
    if (ge.empty()) {
        cudaError_t se = tq_scan_init();
        if (se != cudaSuccess) ge = std::string("tq_scan_init: ") + cudaGetErrorString(se);
        if (se == cudaSuccess && (se = tq_tc_init()) != cudaSuccess) ge = std::string("tq_tc_init: ") + cudaGetErrorString(se);
        if (se == cudaSuccess && (se = tq_tc256_init()) != cudaSuccess) ge = std::string("tq_tc256_init: ") + cudaGetErrorString(se);
        if (se == cudaSuccess && (se = tq_merge_init()) != cudaSuccess) ge = std::string("tq_merge_init: ") + cudaGetErrorString(se);
        if (se == cudaSuccess && (se = tq_ip_init()) != cudaSuccess) ge = std::string("tq_ip_init: ") + cudaGetErrorString(se);
        if (se == cudaSuccess && (se = sparse_attention_init()) != cudaSuccess) ge = std::string("sparse_attention_init: ") + cudaGetErrorString(se);
    }
    if (!ge.empty()) {
        eos_b200_runtime_destroy(rt);
        return fail(err, ge);
    }
    *out = rt;
    return EOS_B200_OK;
}

void eos_b200_runtime_destroy(EosB200Runtime* rt) {
    if (rt == nullptr) return;
    cudaSetDevice(rt->device);
    if (rt->stream) cudaStreamSynchronize(rt->stream);
    if (rt->ev0) cudaEventDestroy(rt->ev0);
    if (rt->ev1) cudaEventDestroy(rt->ev1);
    dev_free(rt->d_status);
    if (rt->stream) cudaStreamDestroy(rt->stream);
    delete rt;
}

int eos_b200_selftest_bounded_wait(EosB200Runtime* rt, int64_t limit_cycles, char** err) {
    if (rt == nullptr) return fail(err, "selftest_bounded_wait: null runtime");
    if (limit_cycles <= 0 || limit_cycles > 200000000LL)
        return fail(err, "selftest_bounded_wait: limit_cycles must be in [1, 2e8] (about 0.1 s)");
    CUDA_TRY(cudaSetDevice(rt->device));
    CUDA_TRY(cudaMemsetAsync(rt->d_status, 0, sizeof(int), rt->stream));
    bounded_wait_probe_kernel<<<1, 32, 0, rt->stream>>>(limit_cycles, rt->d_status);
    CUDA_TRY(cudaGetLastError());
    return read_status(rt, rt->stream, err);
}

int eos_b200_runtime_info(EosB200Runtime* rt, EosB200DeviceInfo* out, char** err) {
    if (rt == nullptr || out == nullptr) return fail(err, "runtime_info: null argument");
    std::memset(out, 0, sizeof(*out));
    out->device = rt->device;
    out->cc_major = rt->prop.major;
    out->cc_minor = rt->prop.minor;
    out->sm_count = rt->sm_count;
    out->total_memory_bytes = (int64_t)rt->prop.totalGlobalMem;
    std::strncpy(out->name, rt->prop.name, sizeof(out->name) - 1);
    return EOS_B200_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// dense weights
// ------------------------------------------------------------------------------------------------
namespace {

struct DenseW {
    void* w = nullptr;      // biased uint8 codes [n, ldw] or f16 [n, ldw]
    bool int8 = false;
    int ldw = 0;
    float* scale = nullptr; // [n] or null
    float* bias = nullptr;  // [n] or null
    int n = 0, k = 0;
};

void free_dense(DenseW& d) {
    if (d.w) cudaFree(d.w);
    d.w = nullptr;
    dev_free(d.scale);
    dev_free(d.bias);
}

std::string check_matrix(const EosB200Matrix& m, int rows, int cols, const char* name) {
    if (m.rows != rows || m.cols != cols)
        return std::string(name) + " weight shape [" + std::to_string(m.rows) + "," + std::to_string(m.cols) +
               "] does not match [out,in]=[" + std::to_string(rows) + "," + std::to_string(cols) + "]";
    if (m.q8_codes != nullptr) {
        if (m.q8_scales == nullptr) return std::string(name) + ": q8 weight without scales";
        if (m.n_scales != 1 && m.n_scales != rows)
            return std::string(name) + ": n_scales must be 1 (per tensor) or rows (per output channel)";
    } else if (m.dense == nullptr) {
        return std::string(name) + ": weight has neither q8 codes nor dense values";
    }
    return "";
}

// Uploads the vertical concatenation of `parts` (same cols) as one dense weight.
std::string upload_dense(const std::vector<const EosB200Matrix*>& parts, const std::vector<const float*>& biases,
                         int weight_mode, DenseW* out) {
    const int k = parts[0]->cols;
    int n = 0;
    const bool q8 = parts[0]->q8_codes != nullptr;
    for (auto* p : parts) {
        if ((p->q8_codes != nullptr) != q8) return "mixed q8 / dense tensors inside one fused projection";
        if (p->cols != k) return "fused projection parts disagree on the input width";
        n += p->rows;
    }
    if (k % 16 != 0) return "dense input width must be a multiple of 16 (16-byte aligned rows of 8-bit codes)";
    out->n = n;
    out->k = k;
    out->ldw = k;
    out->int8 = q8 && weight_mode == EOS_B200_WEIGHTS_Q8_SMEM_DEQUANT;
    std::vector<float> scale;
    std::vector<float> bias((size_t)n, 0.0f);
    bool any_bias = false;
    size_t row0 = 0;
    if (q8) scale.resize((size_t)n);
    std::vector<uint8_t> codes8;
    std::vector<__half> w16;
    if (out->int8) codes8.resize((size_t)n * k);
    else w16.resize((size_t)n * k);
    for (size_t pi = 0; pi < parts.size(); ++pi) {
        const EosB200Matrix* p = parts[pi];
        const size_t cnt = (size_t)p->rows * k;
        if (q8) {
            for (int r = 0; r < p->rows; ++r) scale[row0 + r] = p->q8_scales[p->n_scales == 1 ? 0 : r];
            if (out->int8) {
                for (size_t i = 0; i < cnt; ++i) codes8[row0 * k + i] = (uint8_t)((int)p->q8_codes[i] + 128);
            } else {
                for (size_t i = 0; i < cnt; ++i) w16[row0 * k + i] = __float2half_rn((float)p->q8_codes[i]);
            }
        } else {
            for (size_t i = 0; i < cnt; ++i) w16[row0 * k + i] = __float2half_rn(p->dense[i]);
        }
        if (biases[pi] != nullptr) {
            any_bias = true;
            for (int r = 0; r < p->rows; ++r) bias[row0 + r] = biases[pi][r];
        }
        row0 += p->rows;
    }
    cudaError_t e;
    if (out->int8) {
        e = cudaMalloc(&out->w, codes8.size());
        if (e == cudaSuccess) e = cudaMemcpy(out->w, codes8.data(), codes8.size(), cudaMemcpyHostToDevice);
    } else {
        e = cudaMalloc(&out->w, w16.size() * sizeof(__half));
        if (e == cudaSuccess) e = cudaMemcpy(out->w, w16.data(), w16.size() * sizeof(__half), cudaMemcpyHostToDevice);
    }
    if (e == cudaSuccess && q8) {
        e = dev_alloc(&out->scale, (size_t)n);
        if (e == cudaSuccess) e = cudaMemcpy(out->scale, scale.data(), (size_t)n * 4, cudaMemcpyHostToDevice);
    }
    if (e == cudaSuccess && any_bias) {
        e = dev_alloc(&out->bias, (size_t)n);
        if (e == cudaSuccess) e = cudaMemcpy(out->bias, bias.data(), (size_t)n * 4, cudaMemcpyHostToDevice);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        return std::string("weight upload: ") + cudaGetErrorString(e);
    }
    return "";
}

std::string upload_f32(const float* src, size_t n, float** dst) {
    cudaError_t e = dev_alloc(dst, n);
    if (e == cudaSuccess) e = cudaMemcpy(*dst, src, n * 4, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return std::string("vector upload: ") + cudaGetErrorString(e);
    }
    return "";
}

std::string upload_f16(const float* src, size_t n, __half** dst) {
    std::vector<__half> h = to_half(src, n);
    cudaError_t e = dev_alloc(dst, n);
    if (e == cudaSuccess) e = cudaMemcpy(*dst, h.data(), n * sizeof(__half), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return std::string("table upload: ") + cudaGetErrorString(e);
    }
    return "";
}

struct LayerW {
    DenseW qkv, ao, inter, out;
    float *g1 = nullptr, *b1 = nullptr, *g2 = nullptr, *b2 = nullptr;
};

// CUDA-event pairs around individual launches, tagged with a kernel class.
enum KernelClass : int {
    kClsLayout = 0, kClsEmbed, kClsGemm, kClsAttention, kClsLayerNorm, kClsPool, kClsScan,
    kClsGemmKind0 = 16  // + 0..3: QKV, attention output, FFN up, FFN down
};

struct Profiler {
    std::vector<cudaEvent_t> ev;  // 2 per slot
    std::vector<int> cls;
    int used = 0;
    bool on = false;

    void reset() {
        for (cudaEvent_t e : ev) cudaEventDestroy(e);
        ev.clear();
        cls.clear();
        used = 0;
        on = false;
    }
    bool begin(int slots) {
        reset();
        ev.resize((size_t)slots * 2);
        cls.assign((size_t)slots, 0);
        for (auto& e : ev)
            if (cudaEventCreate(&e) != cudaSuccess) return false;
        on = true;
        return true;
    }
    template <typename F>
    void launch(int c, cudaStream_t s, F&& f) {
        const bool rec = on && (size_t)used < cls.size();
        if (rec) cudaEventRecord(ev[(size_t)used * 2], s);
        f();
        if (rec) {
            cudaEventRecord(ev[(size_t)used * 2 + 1], s);
            cls[used++] = c;
        }
    }
};

}  // namespace

struct EosB200Encoder {
    EosB200Runtime* rt = nullptr;
    int layers = 0, hidden = 0, heads = 0, inter = 0, vocab = 0, max_pos = 0, type_vocab = 0;
    int activation = 0, pooling = 0, window = 0, head_out = 0;
    float eps = 1e-12f;
    __half *tok = nullptr, *pos = nullptr, *typ = nullptr;
    float *eg = nullptr, *eb = nullptr, *head_w = nullptr;
    std::vector<LayerW> lw;
    // workspace
    int cap_batch = 0;
    long long cap_elems = 0;
    int m_alloc = 0;
    int32_t *d_ids = nullptr, *d_mask = nullptr, *d_types = nullptr;
    SeqLayout lay{};
    __half *h0 = nullptr, *h1 = nullptr, *qkv = nullptr, *ctx = nullptr, *pre = nullptr, *ffn = nullptr;
    float *pooled = nullptr, *d_out = nullptr;
    std::vector<GemmPlan> plans;  // 4 per layer: qkv, attn-out, inter, out
    AttnTcPlan attn_plan{};
    bool attn_tc = false;        // tensor-memory attention kernel usable (head_dim 64)
    Profiler prof;
    int launches_per_forward = 0;
    // forwards of the host-buffer calls, captured once per [batch, tokens] shape and replayed as one graph launch
    struct ForwardGraph {
        int batch, tokens;
        bool types;
        int launches;
        cudaGraphExec_t exec;
    };
    std::vector<ForwardGraph> graphs;
    bool graphs_off = false;
    int submitted_launches = 0;          // of the batches submitted since the last wait
    int64_t submitted_up = 0, submitted_down = 0;
    // compact profile (models/default_embedding.go:461-505): role table instead of position / type tables,
    // rotary positions, no biases, non-affine LayerNorm, per-token normalize + masked mean at the end
    bool compact = false;
    int role_vocab = 0;
    __half* role = nullptr;
    DenseW outp;                 // optional output projection [output_dim, hidden]
    float2* rope_cs = nullptr;   // [rope_tokens, hidden / 2] (cos, sin), workspace
    int rope_tokens = 0;
    GemmPlan outp_plan{};
    // per-token output head (long-context multi-vector documents): [token_dim, hidden] dense, no bias
    DenseW tokp;
    int token_dim = 0;
    __half* tok_f16 = nullptr;   // [m_alloc, token_dim] workspace
    GemmPlan tokp_plan{};
};

namespace {

void free_workspace(EosB200Encoder* e) {
    if (!e->graphs.empty()) {   // they hold the workspace's pointers; none may be in flight when it goes
        cudaStreamSynchronize(e->rt->stream);
        for (auto& g : e->graphs) cudaGraphExecDestroy(g.exec);
        e->graphs.clear();
    }
    dev_free(e->d_ids);
    dev_free(e->d_mask);
    dev_free(e->d_types);
    dev_free(e->lay.key_count);
    dev_free(e->lay.row_count);
    dev_free(e->lay.cu_rows);
    dev_free(e->lay.cls_row);
    dev_free(e->lay.row_src);
    dev_free(e->lay.total_rows);
    dev_free(e->lay.cu_qtiles);
    dev_free(e->lay.qtile_info);
    dev_free(e->lay.qtile_win);
    dev_free(e->lay.qtile_info_seq);
    dev_free(e->lay.qtile_win_seq);
    dev_free(e->h0);
    dev_free(e->h1);
    dev_free(e->qkv);
    dev_free(e->ctx);
    dev_free(e->pre);
    dev_free(e->ffn);
    dev_free(e->pooled);
    dev_free(e->d_out);
    dev_free(e->tok_f16);
    e->plans.clear();
    e->cap_batch = 0;
    e->cap_elems = 0;
    e->m_alloc = 0;
}

int ensure_workspace(EosB200Encoder* e, int batch, int tokens, char** err) {
    if (e->compact && tokens > e->rope_tokens) {
        // rotary table for positions 0 .. tokens-1: the angle in double, cosine and sine rounded to float, as
        // ropeRows computes them (runtime/backend/tensor_ops.go:1936-1965)
        const int D = e->hidden;
        std::vector<float2> cs((size_t)tokens * (D / 2));
        for (int t = 0; t < tokens; ++t)
            for (int c = 0; c + 1 < D; c += 2) {
                const double theta = (double)t / std::pow(10000.0, (double)c / (double)D);
                cs[(size_t)t * (D / 2) + c / 2] = make_float2((float)std::cos(theta), (float)std::sin(theta));
            }
        CUDA_TRY(cudaStreamSynchronize(e->rt->stream));
        dev_free(e->rope_cs);
        e->rope_tokens = 0;
        CUDA_TRY(dev_alloc(&e->rope_cs, cs.size()));
        CUDA_TRY(cudaMemcpy(e->rope_cs, cs.data(), cs.size() * sizeof(float2), cudaMemcpyHostToDevice));
        e->rope_tokens = tokens;
    }
    const long long elems = (long long)batch * tokens;
    if (batch <= e->cap_batch && elems <= e->cap_elems) return EOS_B200_OK;
    const int nb = batch > e->cap_batch ? batch : e->cap_batch;
    const long long ne = elems > e->cap_elems ? elems : e->cap_elems;
    if (ne + nb > 0x7fffffffLL / 4) return fail(err, "encoder: batch*tokens too large for 32-bit row indexing");
    free_workspace(e);
    const int m = (int)(ne + nb);
    const int D = e->hidden, F = e->inter;
    const int E = e->head_out > 0 ? e->head_out : D;
    CUDA_TRY(dev_alloc(&e->d_ids, (size_t)ne));
    CUDA_TRY(dev_alloc(&e->d_mask, (size_t)ne));
    CUDA_TRY(dev_alloc(&e->d_types, (size_t)ne));
    CUDA_TRY(dev_alloc(&e->lay.key_count, (size_t)nb));
    CUDA_TRY(dev_alloc(&e->lay.row_count, (size_t)nb));
    CUDA_TRY(dev_alloc(&e->lay.cu_rows, (size_t)nb + 1));
    CUDA_TRY(dev_alloc(&e->lay.cls_row, (size_t)nb));
    CUDA_TRY(dev_alloc(&e->lay.row_src, (size_t)m));
    CUDA_TRY(dev_alloc(&e->lay.total_rows, 1));
    CUDA_TRY(dev_alloc(&e->lay.cu_qtiles, (size_t)nb + 1));
    CUDA_TRY(dev_alloc(&e->lay.qtile_info, (size_t)(m / 128 + nb + 1)));
    CUDA_TRY(dev_alloc(&e->lay.qtile_win, (size_t)(m / 128 + nb + 1)));
    CUDA_TRY(dev_alloc(&e->lay.qtile_info_seq, (size_t)(m / 128 + nb + 1)));
    CUDA_TRY(dev_alloc(&e->lay.qtile_win_seq, (size_t)(m / 128 + nb + 1)));
    CUDA_TRY(dev_alloc(&e->h0, (size_t)m * D));
    CUDA_TRY(dev_alloc(&e->h1, (size_t)m * D));
    CUDA_TRY(dev_alloc(&e->qkv, (size_t)m * 3 * D));
    CUDA_TRY(dev_alloc(&e->ctx, (size_t)m * D));
    CUDA_TRY(dev_alloc(&e->pre, (size_t)m * D));
    CUDA_TRY(dev_alloc(&e->ffn, (size_t)m * F));
    CUDA_TRY(dev_alloc(&e->pooled, (size_t)nb * D));
    CUDA_TRY(dev_alloc(&e->d_out, (size_t)nb * E));
    // activations start as zeros so that rows no kernel writes are finite
    CUDA_TRY(cudaMemset(e->qkv, 0, (size_t)m * 3 * D * sizeof(__half)));
    CUDA_TRY(cudaMemset(e->ctx, 0, (size_t)m * D * sizeof(__half)));
    CUDA_TRY(cudaMemset(e->h0, 0, (size_t)m * D * sizeof(__half)));
    CUDA_TRY(cudaMemset(e->h1, 0, (size_t)m * D * sizeof(__half)));
    CUDA_TRY(cudaMemset(e->ffn, 0, (size_t)m * F * sizeof(__half)));
    e->cap_batch = nb;
    e->cap_elems = ne;
    e->m_alloc = m;
    e->attn_tc = false;
    if (e->hidden / e->heads == 64 && std::getenv("EOS_B200_LEGACY_ATTENTION") == nullptr) {
        std::string ae = attn_tc_make_plan(&e->attn_plan, e->qkv, m, D);
        if (!ae.empty()) return fail(err, "attention plan: " + ae);
        e->attn_tc = true;
    }
    e->plans.resize((size_t)e->layers * 4);
    const int act_mode = e->activation == EOS_B200_ACT_GELU_TANH ? kEpiBiasGeluTanh : kEpiBiasGeluErf;
    for (int l = 0; l < e->layers; ++l) {
        LayerW& w = e->lw[l];
        struct Spec {
            DenseW* d;
            const __half* a;
            int lda;
            __half* out;
            int ldo;
            int mode;
            const __half* res;
        } specs[4] = {
            {&w.qkv, e->h0, D, e->qkv, 3 * D, kEpiBias, nullptr},
            {&w.ao, e->ctx, D, e->pre, D, kEpiBiasResidual, e->h0},
            {&w.inter, e->h1, D, e->ffn, F, act_mode, nullptr},
            {&w.out, e->ffn, F, e->pre, D, kEpiBiasResidual, e->h1},
        };
        for (int i = 0; i < 4; ++i) {
            GemmParams p{};
            p.m_ptr = e->lay.total_rows;
            p.m_alloc = m;
            p.n = specs[i].d->n;
            p.k = specs[i].d->k;
            p.scale = specs[i].d->scale;
            p.bias = specs[i].d->bias;
            p.residual = specs[i].res;
            p.ldr = D;
            p.out = specs[i].out;
            p.ldo = specs[i].ldo;
            p.mode = specs[i].mode;
            p.status = e->rt->d_status;
            std::string ge = gemm_make_plan(&e->plans[(size_t)l * 4 + i], specs[i].a, specs[i].lda, specs[i].d->w,
                                            specs[i].d->ldw, specs[i].d->int8, p, e->rt->sm_count);
            if (!ge.empty()) return fail(err, "encoder layer " + std::to_string(l) + ": " + ge);
        }
    }
    if (e->token_dim > 0) {
        CUDA_TRY(dev_alloc(&e->tok_f16, (size_t)m * e->token_dim));
        GemmParams p{};
        p.m_ptr = e->lay.total_rows;
        p.m_alloc = m;
        p.n = e->tokp.n;
        p.k = e->tokp.k;
        p.scale = e->tokp.scale;
        p.bias = nullptr;
        p.out = e->tok_f16;
        p.ldo = e->token_dim;
        p.mode = kEpiBias;
        p.status = e->rt->d_status;
        std::string ge = gemm_make_plan(&e->tokp_plan, e->h0, D, e->tokp.w, e->tokp.ldw, e->tokp.int8, p, e->rt->sm_count);
        if (!ge.empty()) return fail(err, "token head: " + ge);
    }
    if (e->compact) {
        if (e->outp.w != nullptr) {
            GemmParams p{};
            p.m_ptr = e->lay.total_rows;
            p.m_alloc = m;
            p.n = e->outp.n;
            p.k = e->outp.k;
            p.scale = e->outp.scale;
            p.bias = nullptr;
            p.out = e->qkv;  // free at that point of the forward; row stride = output_dim
            p.ldo = e->outp.n;
            p.mode = kEpiBias;
            p.status = e->rt->d_status;
            std::string ge = gemm_make_plan(&e->outp_plan, e->h0, D, e->outp.w, e->outp.ldw, e->outp.int8, p, e->rt->sm_count);
            if (!ge.empty()) return fail(err, "output projection: " + ge);
        }
    }
    return EOS_B200_OK;
}

// Enqueues the whole forward on `s`; returns the number of kernels launched.
// d_out == nullptr: stop after the last layer (the final hidden states stay in e->h0).
int enqueue_forward(EosB200Encoder* e, const int32_t* d_ids, const int32_t* d_mask, const int32_t* d_types, int batch,
                    int tokens, float* d_out, cudaStream_t s) {
    EosB200Runtime* rt = e->rt;
    const int D = e->hidden;
    const int cls = e->pooling == EOS_B200_POOL_CLS ? 1 : 0;
    int launches = 0;
    Profiler& pf = e->prof;
    pf.launch(kClsLayout, s, [&] { launch_seq_layout(d_mask, batch, tokens, cls, e->window, e->lay, s); });
    launches += 5;
    pf.launch(kClsEmbed, s, [&] {
        if (e->compact)
            launch_embed_rope(d_ids, d_types, e->lay, tokens, e->tok, e->vocab, e->role, e->role_vocab, e->rope_cs,
                              e->rope_tokens, D, e->m_alloc, e->h0, rt->d_status, rt->sm_count, s);
        else
            launch_embed_ln(d_ids, d_types, e->lay, tokens, e->tok, e->vocab, e->pos, e->max_pos, e->typ, e->type_vocab,
                            e->eg, e->eb, e->eps, D, e->m_alloc, e->h0, rt->d_status, rt->sm_count, s);
    });
    launches += 1;
    for (int l = 0; l < e->layers; ++l) {
        LayerW& w = e->lw[l];
        pf.launch(kClsGemmKind0 + 0, s, [&] { gemm_launch(e->plans[(size_t)l * 4 + 0], s); });
        pf.launch(kClsAttention, s, [&] {
            if (e->attn_tc)
                attn_tc_launch(e->attn_plan, e->lay, batch, tokens, D, e->heads, e->window, e->ctx, rt->d_status,
                               rt->sm_count, s);
            else
                launch_attention(e->qkv, e->lay, batch, tokens, D, e->heads, e->window, e->ctx, s);
        });
        pf.launch(kClsGemmKind0 + 1, s, [&] { gemm_launch(e->plans[(size_t)l * 4 + 1], s); });
        pf.launch(kClsLayerNorm, s, [&] {
            launch_layernorm(e->pre, w.g1, w.b1, e->eps, D, e->m_alloc, e->lay.total_rows, e->h1, rt->sm_count, s);
        });
        pf.launch(kClsGemmKind0 + 2, s, [&] { gemm_launch(e->plans[(size_t)l * 4 + 2], s); });
        pf.launch(kClsGemmKind0 + 3, s, [&] { gemm_launch(e->plans[(size_t)l * 4 + 3], s); });
        pf.launch(kClsLayerNorm, s, [&] {
            launch_layernorm(e->pre, w.g2, w.b2, e->eps, D, e->m_alloc, e->lay.total_rows, e->h0, rt->sm_count, s);
        });
        launches += 7;
    }
    if (d_out == nullptr) {
        e->launches_per_forward = launches;
        return launches;
    }
    if (e->compact) {
        if (e->outp.w != nullptr) {
            pf.launch(kClsPool, s, [&] { launch_token_normalize(e->h0, e->lay, D, e->m_alloc, rt->sm_count, s); });
            pf.launch(kClsGemm, s, [&] { gemm_launch(e->outp_plan, s); });
            pf.launch(kClsPool, s, [&] { launch_compact_pool(e->qkv, e->lay, batch, tokens, e->outp.n, 0, d_out, s); });
            launches += 3;
        } else {
            pf.launch(kClsPool, s, [&] { launch_compact_pool(e->h0, e->lay, batch, tokens, D, 1, d_out, s); });
            launches += 1;
        }
    } else {
        pf.launch(kClsPool, s, [&] {
            launch_pool_head(e->h0, e->lay, batch, D, cls, e->head_w, e->head_out, e->pooled, d_out, s);
        });
        launches += e->head_w != nullptr ? 2 : 1;
    }
    e->launches_per_forward = launches;
    return launches;
}

// The forward of a host-buffer call (inputs in e->d_ids / d_mask / d_types, result in e->d_out): captured into a CUDA
// graph the first time a [batch, tokens] shape is seen and replayed afterwards.  A 12-layer forward is 92 launches;
// for a single query or a small batch the host's launch calls, not the kernels, set the latency.  Every pointer and
// size the kernels receive is fixed per shape (row counts are read from device memory), so a replay is the same work.
// Falls back to plain launches while a profile is being recorded, when EOS_B200_NO_GRAPHS is set, or if a capture fails.
int forward_host_call(EosB200Encoder* e, bool types, int batch, int tokens, cudaStream_t s) {
    static const bool env_off = [] {
        const char* v = getenv("EOS_B200_NO_GRAPHS");
        return v != nullptr && v[0] != '\0' && v[0] != '0';
    }();
    const int32_t* d_types = types ? e->d_types : nullptr;
    if (env_off || e->graphs_off || e->prof.on)
        return enqueue_forward(e, e->d_ids, e->d_mask, d_types, batch, tokens, e->d_out, s);
    for (const auto& g : e->graphs)
        if (g.batch == batch && g.tokens == tokens && g.types == types) {
            if (cudaGraphLaunch(g.exec, s) == cudaSuccess) return g.launches;
            cudaGetLastError();   // a replay that cannot be launched: plain launches from here on
            e->graphs_off = true;
            return enqueue_forward(e, e->d_ids, e->d_mask, d_types, batch, tokens, e->d_out, s);
        }
    if (e->graphs.size() >= 16) {   // a host cycling through many shapes: start over rather than grow without bound
        cudaStreamSynchronize(s);
        for (auto& g : e->graphs) cudaGraphExecDestroy(g.exec);
        e->graphs.clear();
    }
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int launches = 0;
    bool ok = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
    if (ok) {
        launches = enqueue_forward(e, e->d_ids, e->d_mask, d_types, batch, tokens, e->d_out, s);
        ok = cudaStreamEndCapture(s, &graph) == cudaSuccess && graph != nullptr;
    }
    if (ok) ok = cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess;
    if (graph != nullptr) cudaGraphDestroy(graph);
    if (ok) ok = cudaGraphLaunch(exec, s) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();   // the failed capture's error is not this call's
        if (exec != nullptr) cudaGraphExecDestroy(exec);
        e->graphs_off = true;
        return enqueue_forward(e, e->d_ids, e->d_mask, d_types, batch, tokens, e->d_out, s);
    }
    e->graphs.push_back({batch, tokens, types, launches, exec});
    return launches;
}

}  // namespace

extern "C" {

void eos_b200_encoder_destroy(EosB200Encoder* enc) {
    if (enc == nullptr) return;
    cudaSetDevice(enc->rt->device);
    cudaStreamSynchronize(enc->rt->stream);
    free_workspace(enc);
    enc->prof.reset();
    dev_free(enc->tok);
    dev_free(enc->pos);
    dev_free(enc->typ);
    dev_free(enc->eg);
    dev_free(enc->eb);
    dev_free(enc->head_w);
    dev_free(enc->role);
    dev_free(enc->rope_cs);
    free_dense(enc->outp);
    free_dense(enc->tokp);
    for (auto& w : enc->lw) {
        free_dense(w.qkv);
        free_dense(w.ao);
        free_dense(w.inter);
        free_dense(w.out);
        dev_free(w.g1);
        dev_free(w.b1);
        dev_free(w.g2);
        dev_free(w.b2);
    }
    delete enc;
}

int eos_b200_encoder_bind(EosB200Runtime* rt, const EosB200EncoderDesc* d, EosB200Encoder** out, char** err) {
    if (rt == nullptr || d == nullptr || out == nullptr) return fail(err, "encoder_bind: null argument");
    *out = nullptr;
    if (d->layers <= 0) return fail(err, "bert_embedder num_hidden_layers must be positive");
    if (d->heads <= 0) return fail(err, "bert_encoder_layer num_attention_heads must be positive");
    if (d->hidden <= 0 || d->intermediate <= 0 || d->vocab <= 0 || d->max_positions <= 0 || d->type_vocab <= 0)
        return fail(err, "encoder_bind: dimensions must be positive");
    if (d->hidden % d->heads != 0) return fail(err, "hidden size must be divisible by num_attention_heads");
    if (d->hidden % 16 != 0 || d->intermediate % 16 != 0)
        return fail(err, "hidden and intermediate sizes must be multiples of 16");
    const int hd = d->hidden / d->heads;
    if (hd > 64 || hd % 2 != 0) return fail(err, "head dimension must be even and at most 64");
    if (d->hidden > 2048) return fail(err, "hidden size above 2048 is not supported");
    if (d->epsilon < 0) return fail(err, "epsilon must be non-negative");
    if (d->activation != EOS_B200_ACT_GELU_ERF && d->activation != EOS_B200_ACT_GELU_TANH)
        return fail(err, "unsupported hidden_act; only gelu (erf) and gelu_tanh are supported");
    if (d->pooling != EOS_B200_POOL_MASKED_MEAN && d->pooling != EOS_B200_POOL_CLS)
        return fail(err, "unsupported pooling; supported values are masked_mean and cls");
    if (!d->token_embeddings || !d->position_embeddings || !d->type_embeddings || !d->embedding_ln_gamma ||
        !d->embedding_ln_beta || !d->layer)
        return fail(err, "encoder_bind: missing tensor");
    if (d->head_out < 0 || (d->head_out > 0 && d->head_weights == nullptr))
        return fail(err, "encoder_bind: projection head without weights");
    CUDA_TRY(cudaSetDevice(rt->device));
    EosB200Encoder* e = new EosB200Encoder();
    e->rt = rt;
    e->layers = d->layers;
    e->hidden = d->hidden;
    e->heads = d->heads;
    e->inter = d->intermediate;
    e->vocab = d->vocab;
    e->max_pos = d->max_positions;
    e->type_vocab = d->type_vocab;
    e->activation = d->activation;
    e->pooling = d->pooling;
    e->window = d->attention_window;
    e->head_out = d->head_out;
    e->eps = (float)d->epsilon;
    const int D = d->hidden, F = d->intermediate;
    std::string msg;
    auto step = [&](const std::string& m) {
        if (msg.empty() && !m.empty()) msg = m;
    };
    step(upload_f16(d->token_embeddings, (size_t)d->vocab * D, &e->tok));
    step(upload_f16(d->position_embeddings, (size_t)d->max_positions * D, &e->pos));
    step(upload_f16(d->type_embeddings, (size_t)d->type_vocab * D, &e->typ));
    step(upload_f32(d->embedding_ln_gamma, D, &e->eg));
    step(upload_f32(d->embedding_ln_beta, D, &e->eb));
    if (d->head_out > 0) step(upload_f32(d->head_weights, (size_t)D * d->head_out, &e->head_w));
    e->lw.resize(d->layers);
    for (int l = 0; l < d->layers && msg.empty(); ++l) {
        const EosB200EncoderLayer& s = d->layer[l];
        const std::string pre = "encoder layer " + std::to_string(l) + " ";
        step(check_matrix(s.query, D, D, "attention query"));
        step(check_matrix(s.key, D, D, "attention key"));
        step(check_matrix(s.value, D, D, "attention value"));
        step(check_matrix(s.attn_out, D, D, "attention output"));
        step(check_matrix(s.inter, F, D, "intermediate"));
        step(check_matrix(s.out, D, F, "output"));
        if (!s.attn_ln_gamma || !s.attn_ln_beta || !s.out_ln_gamma || !s.out_ln_beta) step("missing LayerNorm tensor");
        if (!s.query_bias || !s.key_bias || !s.value_bias || !s.attn_out_bias || !s.inter_bias || !s.out_bias)
            step("dense expects non-nil weight and bias");
        if (!msg.empty()) {
            msg = pre + msg;
            break;
        }
        LayerW& w = e->lw[l];
        step(upload_dense({&s.query, &s.key, &s.value}, {s.query_bias, s.key_bias, s.value_bias}, d->weight_mode,
                          &w.qkv));
        step(upload_dense({&s.attn_out}, {s.attn_out_bias}, d->weight_mode, &w.ao));
        step(upload_dense({&s.inter}, {s.inter_bias}, d->weight_mode, &w.inter));
        step(upload_dense({&s.out}, {s.out_bias}, d->weight_mode, &w.out));
        step(upload_f32(s.attn_ln_gamma, D, &w.g1));
        step(upload_f32(s.attn_ln_beta, D, &w.b1));
        step(upload_f32(s.out_ln_gamma, D, &w.g2));
        step(upload_f32(s.out_ln_beta, D, &w.b2));
        if (!msg.empty()) msg = pre + msg;
    }
    if (!msg.empty()) {
        eos_b200_encoder_destroy(e);
        return fail(err, msg);
    }
    *out = e;
    return EOS_B200_OK;
}

namespace {
// An Eos [in, out] matrix as the [out, in] EosB200Matrix the uploader takes (storage in `keep`).
struct TransposedMatrix {
    std::vector<int8_t> codes;
    std::vector<float> dense;
    EosB200Matrix m{};
};
std::string transpose_in_out(const EosB200Matrix& src, int in, int out, const char* name, TransposedMatrix* t) {
    if (src.rows != in || src.cols != out)
        return std::string(name) + " weight shape [" + std::to_string(src.rows) + "," + std::to_string(src.cols) +
               "] does not match [in,out]=[" + std::to_string(in) + "," + std::to_string(out) + "]";
    t->m = src;
    t->m.rows = out;
    t->m.cols = in;
    if (src.q8_codes != nullptr) {
        if (src.q8_scales == nullptr) return std::string(name) + ": q8 weight without scales";
        if (src.n_scales != 1 && src.n_scales != out)
            return std::string(name) + ": n_scales must be 1 (per tensor) or cols (per output channel)";
        t->codes.resize((size_t)in * out);
        for (int i = 0; i < in; ++i)
            for (int o = 0; o < out; ++o) t->codes[(size_t)o * in + i] = src.q8_codes[(size_t)i * out + o];
        t->m.q8_codes = t->codes.data();
    } else if (src.dense != nullptr) {
        t->dense.resize((size_t)in * out);
        for (int i = 0; i < in; ++i)
            for (int o = 0; o < out; ++o) t->dense[(size_t)o * in + i] = src.dense[(size_t)i * out + o];
        t->m.dense = t->dense.data();
    } else {
        return std::string(name) + ": weight has neither q8 codes nor dense values";
    }
    return "";
}
}  // namespace

int eos_b200_compact_encoder_bind(EosB200Runtime* rt, const EosB200CompactEncoderDesc* d, EosB200Encoder** out,
                                  char** err) {
    if (rt == nullptr || d == nullptr || out == nullptr) return fail(err, "compact_encoder_bind: null argument");
    *out = nullptr;
    if (d->layers <= 0 || d->heads <= 0 || d->hidden <= 0 || d->intermediate <= 0 || d->vocab <= 0 || d->role_vocab <= 0)
        return fail(err, "compact_encoder_bind: dimensions must be positive");
    if (d->hidden % d->heads != 0) return fail(err, "hidden size must be divisible by num_attention_heads");
    if (d->hidden % 16 != 0 || d->intermediate % 16 != 0)
        return fail(err, "hidden and intermediate sizes must be multiples of 16");
    const int hd = d->hidden / d->heads;
    if (hd > 64 || hd % 2 != 0) return fail(err, "head dimension must be even and at most 64");
    if (d->hidden > 2048) return fail(err, "hidden size above 2048 is not supported");
    if (!d->token_embedding || !d->role_embedding || !d->layer) return fail(err, "compact_encoder_bind: missing tensor");
    const bool project = d->output_dim > 0 && d->output_dim != d->hidden;
    if (d->output_dim < 0 || (project && d->output_dim % 8 != 0))
        return fail(err, "compact_encoder_bind: output_dim must be a non-negative multiple of 8");
    CUDA_TRY(cudaSetDevice(rt->device));
    EosB200Encoder* e = new EosB200Encoder();
    e->rt = rt;
    e->compact = true;
    e->layers = d->layers;
    e->hidden = d->hidden;
    e->heads = d->heads;
    e->inter = d->intermediate;
    e->vocab = d->vocab;
    e->role_vocab = d->role_vocab;
    e->activation = EOS_B200_ACT_GELU_TANH;
    e->pooling = EOS_B200_POOL_MASKED_MEAN;
    e->head_out = project ? d->output_dim : 0;  // sizes the output buffer; there is no BERT-style head
    e->eps = 1e-5f;
    const int D = d->hidden, F = d->intermediate;
    std::string msg;
    auto step = [&](const std::string& m) {
        if (msg.empty() && !m.empty()) msg = m;
    };
    step(upload_f16(d->token_embedding, (size_t)d->vocab * D, &e->tok));
    step(upload_f16(d->role_embedding, (size_t)d->role_vocab * D, &e->role));
    const std::vector<float> ones((size_t)D, 1.0f), zeros((size_t)D, 0.0f);
    e->lw.resize(d->layers);
    for (int l = 0; l < d->layers && msg.empty(); ++l) {
        const EosB200CompactLayer& s = d->layer[l];
        TransposedMatrix q, k, v, o, up, down;
        step(transpose_in_out(s.attn_q, D, D, "attention query", &q));
        step(transpose_in_out(s.attn_k, D, D, "attention key", &k));
        step(transpose_in_out(s.attn_v, D, D, "attention value", &v));
        step(transpose_in_out(s.attn_o, D, D, "attention output", &o));
        step(transpose_in_out(s.ffn_up, D, F, "ffn up", &up));
        step(transpose_in_out(s.ffn_down, F, D, "ffn down", &down));
        if (!msg.empty()) {
            msg = "encoder layer " + std::to_string(l) + " " + msg;
            break;
        }
        LayerW& w = e->lw[l];
        step(upload_dense({&q.m, &k.m, &v.m}, {nullptr, nullptr, nullptr}, d->weight_mode, &w.qkv));
        step(upload_dense({&o.m}, {nullptr}, d->weight_mode, &w.ao));
        step(upload_dense({&up.m}, {nullptr}, d->weight_mode, &w.inter));
        step(upload_dense({&down.m}, {nullptr}, d->weight_mode, &w.out));
        step(upload_f32(ones.data(), D, &w.g1));
        step(upload_f32(zeros.data(), D, &w.b1));
        step(upload_f32(ones.data(), D, &w.g2));
        step(upload_f32(zeros.data(), D, &w.b2));
        if (!msg.empty()) msg = "encoder layer " + std::to_string(l) + " " + msg;
    }
    if (msg.empty() && project) {
        TransposedMatrix p;
        step(transpose_in_out(d->output_projection, D, d->output_dim, "output projection", &p));
        if (msg.empty()) step(upload_dense({&p.m}, {nullptr}, d->weight_mode, &e->outp));
    }
    if (!msg.empty()) {
        eos_b200_encoder_destroy(e);
        return fail(err, msg);
    }
    *out = e;
    return EOS_B200_OK;
}

int eos_b200_encoder_reserve(EosB200Encoder* enc, int batch, int tokens, char** err) {
    if (enc == nullptr) return fail(err, "encoder_reserve: null encoder");
    if (batch <= 0 || tokens <= 0) return fail(err, "encoder_reserve: batch and tokens must be positive");
    CUDA_TRY(cudaSetDevice(enc->rt->device));
    return ensure_workspace(enc, batch, tokens, err);
}

int eos_b200_encoder_run_device(EosB200Encoder* enc, const int32_t* d_ids, const int32_t* d_mask,
                                const int32_t* d_types, int batch, int tokens, float* d_out, void* stream,
                                EosB200Stats* stats, char** err) {
    if (enc == nullptr || d_ids == nullptr || d_mask == nullptr || d_out == nullptr)
        return fail(err, "bert_embedder expects non-nil input_ids, attention_mask and output");
    if (batch <= 0 || tokens <= 0) return fail(err, "bert_embedder input_ids must be a non-empty [B,T] tensor");
    if (!enc->compact && tokens > enc->max_pos)
        return fail(err, "bert_embeddings position_ids value out of range (tokens > max_positions)");
    CUDA_TRY(cudaSetDevice(enc->rt->device));
    int rc = ensure_workspace(enc, batch, tokens, err);
    if (rc != EOS_B200_OK) return rc;
    cudaStream_t s = pick_stream(enc->rt, stream);
    CUDA_TRY(cudaMemsetAsync(enc->rt->d_status, 0, sizeof(int), s));
    const int launches = enqueue_forward(enc, d_ids, d_mask, d_types, batch, tokens, d_out, s);
    CUDA_TRY(cudaGetLastError());
    if (stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = launches;
    }
    return EOS_B200_OK;
}

int eos_b200_encoder_set_token_head(EosB200Encoder* enc, const float* h_weights, int token_dim, char** err) {
    if (enc == nullptr || h_weights == nullptr) return fail(err, "encoder_set_token_head: null argument");
    if (token_dim <= 0 || token_dim % 8 != 0 || token_dim > 1024)
        return fail(err, "encoder_set_token_head: token_dim must be a multiple of 8 in [8, 1024]");
    CUDA_TRY(cudaSetDevice(enc->rt->device));
    CUDA_TRY(cudaStreamSynchronize(enc->rt->stream));
    const int D = enc->hidden;
    // [hidden, token_dim] in-major (as a projection head is stored) -> [token_dim, hidden] for the projection kernel
    std::vector<float> wt((size_t)token_dim * D);
    for (int i = 0; i < D; ++i)
        for (int j = 0; j < token_dim; ++j) wt[(size_t)j * D + i] = h_weights[(size_t)i * token_dim + j];
    EosB200Matrix m{};
    m.rows = token_dim;
    m.cols = D;
    m.dense = wt.data();
    free_dense(enc->tokp);
    std::string msg = upload_dense({&m}, {nullptr}, EOS_B200_WEIGHTS_F16_RESIDENT, &enc->tokp);
    if (!msg.empty()) return fail(err, "encoder_set_token_head: " + msg);
    enc->token_dim = token_dim;
    free_workspace(enc);   // the next run re-plans with the head's buffers
    return EOS_B200_OK;
}

int eos_b200_encoder_token_vectors_device(EosB200Encoder* enc, const int32_t* d_ids, const int32_t* d_mask,
                                          const int32_t* d_types, int batch, int tokens, float* d_vectors,
                                          int32_t* d_row_count, void* stream, EosB200Stats* stats, char** err) {
    if (enc == nullptr || d_ids == nullptr || d_mask == nullptr || d_vectors == nullptr)
        return fail(err, "encoder_token_vectors: null argument");
    if (enc->token_dim <= 0) return fail(err, "encoder_token_vectors: no token head set (eos_b200_encoder_set_token_head)");
    if (enc->compact) return fail(err, "encoder_token_vectors: not available for the compact profile");
    if (batch <= 0 || tokens <= 0) return fail(err, "bert_embedder input_ids must be a non-empty [B,T] tensor");
    if (tokens > enc->max_pos) return fail(err, "bert_embeddings position_ids value out of range (tokens > max_positions)");
    CUDA_TRY(cudaSetDevice(enc->rt->device));
    int rc = ensure_workspace(enc, batch, tokens, err);
    if (rc != EOS_B200_OK) return rc;
    cudaStream_t s = pick_stream(enc->rt, stream);
    CUDA_TRY(cudaMemsetAsync(enc->rt->d_status, 0, sizeof(int), s));
    int launches = enqueue_forward(enc, d_ids, d_mask, d_types, batch, tokens, nullptr, s);
    gemm_launch(enc->tokp_plan, s);
    launch_rows_normalize_f32(enc->tok_f16, enc->lay, enc->token_dim, enc->m_alloc, d_vectors, enc->rt->sm_count, s);
    launches += 2;
    if (d_row_count != nullptr)
        CUDA_TRY(cudaMemcpyAsync(d_row_count, enc->lay.total_rows, sizeof(int32_t), cudaMemcpyDeviceToDevice, s));
    CUDA_TRY(cudaGetLastError());
    if (stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = launches;
    }
    return EOS_B200_OK;
}

int eos_b200_encoder_profile_begin(EosB200Encoder* enc, int max_steps, char** err) {
    if (enc == nullptr || max_steps <= 0) return fail(err, "encoder_profile_begin: bad argument");
    CUDA_TRY(cudaSetDevice(enc->rt->device));
    const int per_forward = 3 + enc->layers * 7;  // event pairs per forward (one per launcher call)
    if (!enc->prof.begin(per_forward * max_steps)) return fail(err, "encoder_profile_begin: cudaEventCreate failed");
    return EOS_B200_OK;
}

int eos_b200_encoder_profile_end(EosB200Encoder* enc, void* stream, EosB200EncoderTimes* out, char** err) {
    if (enc == nullptr || out == nullptr) return fail(err, "encoder_profile_end: null argument");
    CUDA_TRY(cudaSetDevice(enc->rt->device));
    CUDA_TRY(cudaStreamSynchronize(pick_stream(enc->rt, stream)));
    std::memset(out, 0, sizeof(*out));
    const int per_forward = 3 + enc->layers * 7;
    out->steps = enc->prof.used / per_forward;
    for (int i = 0; i < enc->prof.used; ++i) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, enc->prof.ev[(size_t)i * 2], enc->prof.ev[(size_t)i * 2 + 1]);
        const int cls = enc->prof.cls[i];
        if (cls >= kClsGemmKind0 && cls < kClsGemmKind0 + 4) {
            out->gemm_ms += ms;
            out->gemm_launches++;
            out->gemm_kind_ms[cls - kClsGemmKind0] += ms;
            continue;
        }
        switch (cls) {
            case kClsGemm: out->gemm_ms += ms; out->gemm_launches++; break;
            case kClsAttention: out->attention_ms += ms; out->attention_launches++; break;
            case kClsLayerNorm: out->layernorm_ms += ms; out->layernorm_launches++; break;
            case kClsEmbed: out->embed_ms += ms; out->other_launches++; break;
            case kClsPool: out->pool_ms += ms; out->other_launches += enc->head_w != nullptr ? 2 : 1; break;
            default: out->layout_ms += ms; out->other_launches += 5; break;
        }
    }
    enc->prof.reset();
    return EOS_B200_OK;
}

int eos_b200_encoder_sync(EosB200Encoder* enc, void* stream, char** err) {
    if (enc == nullptr) return fail(err, "encoder_sync: null encoder");
    CUDA_TRY(cudaSetDevice(enc->rt->device));
    return read_status(enc->rt, pick_stream(enc->rt, stream), err);
}

int eos_b200_encoder_run(EosB200Encoder* enc, const int32_t* h_ids, const int32_t* h_mask, const int32_t* h_types,
                         int batch, int tokens, float* h_out, EosB200Stats* stats, char** err) {
    if (enc == nullptr || h_ids == nullptr || h_mask == nullptr || h_out == nullptr)
        return fail(err, "bert_embedder expects non-nil input_ids, attention_mask and output");
    if (batch <= 0 || tokens <= 0) return fail(err, "bert_embedder input_ids must be a non-empty [B,T] tensor");
    if (!enc->compact && tokens > enc->max_pos)
        return fail(err, "bert_embeddings position_ids value out of range (tokens > max_positions)");
    EosB200Runtime* rt = enc->rt;
    CUDA_TRY(cudaSetDevice(rt->device));
    int rc = ensure_workspace(enc, batch, tokens, err);
    if (rc != EOS_B200_OK) return rc;
    cudaStream_t s = rt->stream;
    const size_t n = (size_t)batch * tokens;
    const int E = enc->head_out > 0 ? enc->head_out : enc->hidden;
    CUDA_TRY(cudaEventRecord(rt->ev0, s));
    CUDA_TRY(cudaMemsetAsync(rt->d_status, 0, sizeof(int), s));
    CUDA_TRY(cudaMemcpyAsync(enc->d_ids, h_ids, n * 4, cudaMemcpyHostToDevice, s));
    CUDA_TRY(cudaMemcpyAsync(enc->d_mask, h_mask, n * 4, cudaMemcpyHostToDevice, s));
    if (h_types != nullptr) CUDA_TRY(cudaMemcpyAsync(enc->d_types, h_types, n * 4, cudaMemcpyHostToDevice, s));
    const int launches = forward_host_call(enc, h_types != nullptr, batch, tokens, s);
    CUDA_TRY(cudaGetLastError());
    CUDA_TRY(cudaMemcpyAsync(h_out, enc->d_out, (size_t)batch * E * 4, cudaMemcpyDeviceToHost, s));
    int rows = 0;
    CUDA_TRY(cudaMemcpyAsync(&rows, enc->lay.total_rows, 4, cudaMemcpyDeviceToHost, s));
    CUDA_TRY(cudaEventRecord(rt->ev1, s));
    rc = read_status(rt, s, err);
    if (stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = launches;
        stats->uploaded_bytes = (int64_t)n * 4 * (h_types != nullptr ? 3 : 2);
        stats->downloaded_bytes = (int64_t)batch * E * 4 + 8;
        stats->valid_tokens = rows;
        cudaEventElapsedTime(&stats->device_ms, rt->ev0, rt->ev1);
    }
    return rc;
}

int eos_b200_encoder_submit(EosB200Encoder* enc, const int32_t* h_ids, const int32_t* h_mask, const int32_t* h_types,
                            int batch, int tokens, float* h_out, char** err) {
    if (enc == nullptr || h_ids == nullptr || h_mask == nullptr || h_out == nullptr)
        return fail(err, "bert_embedder expects non-nil input_ids, attention_mask and output");
    if (batch <= 0 || tokens <= 0) return fail(err, "bert_embedder input_ids must be a non-empty [B,T] tensor");
    if (!enc->compact && tokens > enc->max_pos)
        return fail(err, "bert_embeddings position_ids value out of range (tokens > max_positions)");
    EosB200Runtime* rt = enc->rt;
    CUDA_TRY(cudaSetDevice(rt->device));
    // growing the workspace frees the buffers batches in flight still use: they are waited for first
    const long long elems = (long long)batch * tokens;
    if (batch > enc->cap_batch || elems > enc->cap_elems) CUDA_TRY(cudaStreamSynchronize(rt->stream));
    int rc = ensure_workspace(enc, batch, tokens, err);
    if (rc != EOS_B200_OK) return rc;
    cudaStream_t s = rt->stream;
    const size_t n = (size_t)batch * tokens;
    const int E = enc->head_out > 0 ? enc->head_out : enc->hidden;
    // stream order does the rest: this batch's uploads follow the previous batch's kernels, its kernels the previous
    // batch's download.  The status word is not reset here: an error of any batch in flight stays until the wait.
    CUDA_TRY(cudaMemcpyAsync(enc->d_ids, h_ids, n * 4, cudaMemcpyHostToDevice, s));
    CUDA_TRY(cudaMemcpyAsync(enc->d_mask, h_mask, n * 4, cudaMemcpyHostToDevice, s));
    if (h_types != nullptr) CUDA_TRY(cudaMemcpyAsync(enc->d_types, h_types, n * 4, cudaMemcpyHostToDevice, s));
    const int launches = forward_host_call(enc, h_types != nullptr, batch, tokens, s);
    CUDA_TRY(cudaGetLastError());
    CUDA_TRY(cudaMemcpyAsync(h_out, enc->d_out, (size_t)batch * E * 4, cudaMemcpyDeviceToHost, s));
    enc->submitted_launches += launches;
    enc->submitted_up += (int64_t)n * 4 * (h_types != nullptr ? 3 : 2);
    enc->submitted_down += (int64_t)batch * E * 4;
    return EOS_B200_OK;
}

int eos_b200_encoder_wait(EosB200Encoder* enc, EosB200Stats* stats, char** err) {
    if (enc == nullptr) return fail(err, "encoder_wait: null encoder");
    EosB200Runtime* rt = enc->rt;
    CUDA_TRY(cudaSetDevice(rt->device));
    const int rc = read_status(rt, rt->stream, err);   // synchronises the stream
    if (stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = enc->submitted_launches;
        stats->uploaded_bytes = enc->submitted_up;
        stats->downloaded_bytes = enc->submitted_down;
    }
    enc->submitted_launches = 0;
    enc->submitted_up = enc->submitted_down = 0;
    return rc;
}

int eos_b200_linear(EosB200Runtime* rt, const float* h_x, int64_t rows, const EosB200Matrix* w, const float* h_bias,
                    int epilogue, const float* h_residual, int weight_mode, float* h_y, EosB200Stats* stats,
                    char** err) {
    if (rt == nullptr || h_x == nullptr || w == nullptr || h_y == nullptr) return fail(err, "linear: null argument");
    if (rows <= 0 || rows > 0x7fffffff / 2) return fail(err, "linear: rows must be positive and fit 31 bits");
    if (epilogue < 0 || epilogue > 3) return fail(err, "linear: unknown epilogue");
    if (epilogue == kEpiBiasResidual && h_residual == nullptr) return fail(err, "linear: residual epilogue without residual");
    std::string cm = check_matrix(*w, w->rows, w->cols, "linear");
    if (!cm.empty()) return fail(err, cm);
    CUDA_TRY(cudaSetDevice(rt->device));
    const int n = w->rows, k = w->cols;
    const int ldo = (n + 7) / 8 * 8;
    DenseW dw;
    std::string ue = upload_dense({w}, {h_bias}, weight_mode, &dw);
    if (!ue.empty()) {
        free_dense(dw);
        return fail(err, ue);
    }
    __half *d_x = nullptr, *d_y = nullptr, *d_r = nullptr;
    int rc = EOS_B200_OK;
    std::string msg;
    do {
        std::vector<__half> hx = to_half(h_x, (size_t)rows * k);
        if (dev_alloc(&d_x, (size_t)rows * k) != cudaSuccess || dev_alloc(&d_y, (size_t)rows * ldo) != cudaSuccess) {
            msg = "linear: device allocation failed";
            break;
        }
        cudaMemcpyAsync(d_x, hx.data(), hx.size() * 2, cudaMemcpyHostToDevice, rt->stream);
        if (h_residual != nullptr) {
            std::vector<__half> hr((size_t)rows * ldo, __float2half_rn(0.f));
            for (int64_t r = 0; r < rows; ++r)
                for (int c = 0; c < n; ++c) hr[(size_t)r * ldo + c] = __float2half_rn(h_residual[(size_t)r * n + c]);
            if (dev_alloc(&d_r, (size_t)rows * ldo) != cudaSuccess) {
                msg = "linear: device allocation failed";
                break;
            }
            cudaMemcpy(d_r, hr.data(), hr.size() * 2, cudaMemcpyHostToDevice);
        }
        GemmParams p{};
        p.m_ptr = nullptr;
        p.m_alloc = (int)rows;
        p.n = n;
        p.k = k;
        p.scale = dw.scale;
        p.bias = dw.bias;
        p.residual = d_r;
        p.ldr = ldo;
        p.out = d_y;
        p.ldo = ldo;
        p.mode = epilogue;
        p.status = rt->d_status;
        GemmPlan plan;
        msg = gemm_make_plan(&plan, d_x, k, dw.w, dw.ldw, dw.int8, p, rt->sm_count);
        if (!msg.empty()) break;
        cudaMemsetAsync(rt->d_status, 0, sizeof(int), rt->stream);
        cudaEventRecord(rt->ev0, rt->stream);
        gemm_launch(plan, rt->stream);
        cudaEventRecord(rt->ev1, rt->stream);
        cudaError_t le = cudaGetLastError();
        if (le != cudaSuccess) {
            msg = std::string("linear launch: ") + cudaGetErrorString(le);
            break;
        }
        std::vector<__half> hy((size_t)rows * ldo);
        cudaError_t ce = cudaMemcpyAsync(hy.data(), d_y, hy.size() * 2, cudaMemcpyDeviceToHost, rt->stream);
        if (ce != cudaSuccess) {
            msg = std::string("linear download: ") + cudaGetErrorString(ce);
            break;
        }
        rc = read_status(rt, rt->stream, err);
        if (rc != EOS_B200_OK) break;
        for (int64_t r = 0; r < rows; ++r)
            for (int c = 0; c < n; ++c) h_y[(size_t)r * n + c] = __half2float(hy[(size_t)r * ldo + c]);
        if (stats != nullptr) {
            std::memset(stats, 0, sizeof(*stats));
            stats->kernel_launches = 1;
            stats->uploaded_bytes = (int64_t)rows * k * 2;
            stats->downloaded_bytes = (int64_t)rows * ldo * 2;
            cudaEventElapsedTime(&stats->device_ms, rt->ev0, rt->ev1);
        }
    } while (false);
    cudaStreamSynchronize(rt->stream);
    dev_free(d_x);
    dev_free(d_y);
    dev_free(d_r);
    free_dense(dw);
    if (!msg.empty()) return fail(err, msg);
    return rc;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// compiled pipeline
// ------------------------------------------------------------------------------------------------
struct EosB200EmbedPooled {
    EosB200Runtime* rt = nullptr;
    int vocab = 0, dim = 0, out_dim = 0;
    __half *table = nullptr, *proj = nullptr;
    int32_t *d_tokens = nullptr, *d_mask = nullptr;
    float* d_out = nullptr;
    float* d_partial = nullptr;   // [batch][ceil(tokens / 8)][out_dim] group sums
    int* d_counts = nullptr;      // [batch] valid tokens
    long long cap_elems = 0;
    int cap_batch = 0;
    float matmul_scale = 1.0f;    // the matmul step's `scale` attribute, resolved to a number by the caller
};

extern "C" {

int eos_b200_embed_pooled_set_matmul_scale(EosB200EmbedPooled* ep, float scale, char** err) {
    if (ep == nullptr) return fail(err, "embed_pooled_set_matmul_scale: null pipeline");
    if (std::isnan(scale) || std::isinf(scale)) return fail(err, "matmul scale must be finite");
    ep->matmul_scale = scale;
    return EOS_B200_OK;
}

void eos_b200_embed_pooled_destroy(EosB200EmbedPooled* ep) {
    if (ep == nullptr) return;
    cudaSetDevice(ep->rt->device);
    cudaStreamSynchronize(ep->rt->stream);
    dev_free(ep->table);
    dev_free(ep->proj);
    dev_free(ep->d_tokens);
    dev_free(ep->d_mask);
    dev_free(ep->d_out);
    dev_free(ep->d_partial);
    dev_free(ep->d_counts);
    delete ep;
}

int eos_b200_embed_pooled_bind(EosB200Runtime* rt, const float* h_table, int vocab, int dim,
                               const float* h_projection, int out_dim, EosB200EmbedPooled** out, char** err) {
    if (rt == nullptr || h_table == nullptr || h_projection == nullptr || out == nullptr)
        return fail(err, "embed_pooled_bind: null argument");
    *out = nullptr;
    if (vocab <= 0 || dim <= 0 || out_dim <= 0) return fail(err, "embed_pooled_bind: dimensions must be positive");
    if (out_dim > 1024) return fail(err, "embed_pooled_bind: out_dim above 1024 is not supported");
    if (dim > 1536) return fail(err, "embed_pooled_bind: dim above 1536 is not supported");
    CUDA_TRY(cudaSetDevice(rt->device));
    EosB200EmbedPooled* ep = new EosB200EmbedPooled();
    ep->rt = rt;
    ep->vocab = vocab;
    ep->dim = dim;
    ep->out_dim = out_dim;
    std::string msg = upload_f16(h_table, (size_t)vocab * dim, &ep->table);
    if (msg.empty()) msg = upload_f16(h_projection, (size_t)dim * out_dim, &ep->proj);
    if (!msg.empty()) {
        eos_b200_embed_pooled_destroy(ep);
        return fail(err, msg);
    }
    *out = ep;
    return EOS_B200_OK;
}

int eos_b200_embed_pooled_run(EosB200EmbedPooled* ep, const int32_t* h_tokens, const int32_t* h_mask, int batch,
                              int tokens, int pool_then_l2, float* h_out, EosB200Stats* stats, char** err) {
    if (ep == nullptr || h_tokens == nullptr || h_mask == nullptr || h_out == nullptr)
        return fail(err, "embed_pooled_run: null argument");
    if (batch <= 0 || tokens <= 0) return fail(err, "embed_pooled_run: empty token batch");
    EosB200Runtime* rt = ep->rt;
    CUDA_TRY(cudaSetDevice(rt->device));
    const long long n = (long long)batch * tokens;
    if (n > ep->cap_elems || batch > ep->cap_batch) {
        dev_free(ep->d_tokens);
        dev_free(ep->d_mask);
        dev_free(ep->d_out);
        dev_free(ep->d_partial);
        dev_free(ep->d_counts);
        CUDA_TRY(dev_alloc(&ep->d_tokens, (size_t)n));
        CUDA_TRY(dev_alloc(&ep->d_mask, (size_t)n));
        CUDA_TRY(dev_alloc(&ep->d_out, (size_t)batch * ep->out_dim));
        CUDA_TRY(dev_alloc(&ep->d_partial, (size_t)(n / 8 + batch) * ep->out_dim));
        CUDA_TRY(dev_alloc(&ep->d_counts, (size_t)batch));
        ep->cap_elems = n;
        ep->cap_batch = batch;
    }
    cudaStream_t s = rt->stream;
    CUDA_TRY(cudaEventRecord(rt->ev0, s));
    CUDA_TRY(cudaMemsetAsync(rt->d_status, 0, sizeof(int), s));
    CUDA_TRY(cudaMemcpyAsync(ep->d_tokens, h_tokens, (size_t)n * 4, cudaMemcpyHostToDevice, s));
    CUDA_TRY(cudaMemcpyAsync(ep->d_mask, h_mask, (size_t)n * 4, cudaMemcpyHostToDevice, s));
    launch_embed_pooled(ep->d_tokens, ep->d_mask, batch, tokens, ep->table, ep->vocab, ep->dim, ep->proj, ep->out_dim,
                        ep->matmul_scale, pool_then_l2 ? 1 : 0, ep->d_partial, ep->d_counts, ep->d_out, rt->d_status, s);
    CUDA_TRY(cudaGetLastError());
    CUDA_TRY(cudaMemcpyAsync(h_out, ep->d_out, (size_t)batch * ep->out_dim * 4, cudaMemcpyDeviceToHost, s));
    CUDA_TRY(cudaEventRecord(rt->ev1, s));
    int rc = read_status(rt, s, err);
    if (stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = 2;
        stats->uploaded_bytes = n * 8;
        stats->downloaded_bytes = (int64_t)batch * ep->out_dim * 4;
        cudaEventElapsedTime(&stats->device_ms, rt->ev0, rt->ev1);
    }
    return rc;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// TurboQuant
// ------------------------------------------------------------------------------------------------
struct EosB200Quantizer {
    EosB200Runtime* rt = nullptr;
    int dim = 0, bits = 0;
    int* perm = nullptr;
    float *signs1 = nullptr, *signs2 = nullptr, *centroids = nullptr, *boundaries = nullptr;
    uint32_t mag_hi[2] = {0, 0}, mag_lo[2] = {0, 0};
    TqSpec spec() const { return TqSpec{dim, bits, perm, signs1, signs2, centroids, boundaries}; }
};

struct EosB200Corpus {
    EosB200Quantizer* qz = nullptr;
    int64_t n = 0, id_base = 0;
    uint8_t* tiles = nullptr;
    float* norms = nullptr;
    // scoring workspace
    int cap_queries = 0;       // padded query capacity
    float* d_queries = nullptr;
    uint2* bfrag = nullptr;
    uint64_t* cand = nullptr;  // [group][grid][kTqMaxK]
    int* cand_count = nullptr;
    unsigned long long* shared_tau = nullptr;  // [cap_queries] pruning thresholds shared by the CTAs of a pass
    uint64_t* seed_keys = nullptr;             // [cap_queries][kTqMaxK] top-k keys of the sample that seeds them
    int64_t* d_ids = nullptr;
    float* d_scores = nullptr;
    int grid = 0;
    // tensor-core batch paths, allocated on first use: plan 0 = 128 queries per launch (queries are the MMA rows),
    // plan 1 = 256 queries per launch (128-document tiles are the MMA rows)
    struct TcPlan {
        int queries = 0;          // queries per launch
        int tile_docs = 0;        // documents per tile
        int segs_per_cta = 0;     // candidate lists a CTA keeps per query
        int grid = 0;
        bool q_in_tmem = false;   // plan 0 only: opt-in variant with the queries resident in tensor memory
        int map_queries = 0;      // query rows the tensor map covers (0 = not built)
        int slots = 1;            // launches whose candidate lists are held before one merge launch
        uint64_t* cand = nullptr;     // [slots][queries][segs_per_cta * grid][kTqTcSegLen]
        int* count = nullptr;         // [slots][queries][segs_per_cta * grid]
        float* seed_scores = nullptr; // [slots][queries][grid * 256] scores of the sample that seeds the thresholds
        CUtensorMap tm;
    } tcp[2];
    int qperm_queries = 0;
    __half* qperm = nullptr;        // [qperm_queries][padded dim] rotated queries, coordinates in code-word order
    Profiler prof;
};

namespace {
constexpr int kTqGroupQueries = 256;  // queries whose per-CTA candidates are held before one merge launch
constexpr int kTqTcMergeSlots = 16;   // launches of the 256-query batch kernel whose lists one launch merges

__global__ void synth_gaussian_kernel(unsigned long long seed, long long row_offset, long long n, int dim, int normalize,
                                      float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long r = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < n; r += warps) {
        const unsigned long long rowkey = seed * 0x9E3779B97F4A7C15ull + (unsigned long long)(row_offset + r);
        float sq = 0.f;
        for (int pass = 0; pass < (normalize ? 2 : 1); ++pass) {
            float inv = 1.0f;
            if (pass == 1) {
                float tot = sq;
                for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
                inv = tot > 0.f ? rsqrtf(tot) : 1.0f;
            }
            for (int p = lane; p < (dim + 1) / 2; p += 32) {
                unsigned long long z = rowkey * 0xD1342543DE82EF95ull + (unsigned long long)p * 0x9E3779B97F4A7C15ull;
                z ^= z >> 30;
                z *= 0xBF58476D1CE4E5B9ull;
                z ^= z >> 27;
                z *= 0x94D049BB133111EBull;
                z ^= z >> 31;
                const float u1 = ((float)(unsigned)(z >> 40) + 0.5f) * (1.0f / 16777216.0f);
                const float u2 = ((float)(unsigned)((z >> 8) & 0xffffffu) + 0.5f) * (1.0f / 16777216.0f);
                const float rad = sqrtf(-2.0f * logf(u1));
                float s, c;
                sincosf(6.283185307179586f * u2, &s, &c);
                const float a = rad * c, b = rad * s;
                if (normalize && pass == 0) {
                    sq += a * a;
                    if (2 * p + 1 < dim) sq += b * b;
                } else {
                    out[r * dim + 2 * p] = a * inv;
                    if (2 * p + 1 < dim) out[r * dim + 2 * p + 1] = b * inv;
                }
            }
        }
    }
}

int corpus_finish_bind(EosB200Quantizer* qz, const uint8_t* d_codes, const float* d_norms, int64_t n, int64_t id_base,
                       EosB200Corpus** out, char** err) {
    EosB200Corpus* c = new EosB200Corpus();
    c->qz = qz;
    c->n = n;
    c->id_base = id_base;
    const int64_t n_tiles = (n + kTqDocsPerTile - 1) / kTqDocsPerTile;
    const size_t tile_bytes = tq_tile_bytes(qz->dim);
    cudaError_t e = dev_alloc(&c->tiles, (size_t)(n_tiles > 0 ? n_tiles : 1) * tile_bytes);
    if (e == cudaSuccess) e = dev_alloc(&c->norms, (size_t)(n > 0 ? n : 1));
    if (e == cudaSuccess && n > 0) {
        e = cudaMemcpyAsync(c->norms, d_norms, (size_t)n * 4, cudaMemcpyDeviceToDevice, qz->rt->stream);
        launch_tq_transcode(d_codes, n, qz->dim, qz->bits, c->tiles, qz->rt->stream);
        if (e == cudaSuccess) e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaStreamSynchronize(qz->rt->stream);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        std::string msg = std::string("corpus_bind: ") + cudaGetErrorString(e);
        eos_b200_corpus_destroy(c);
        return fail(err, msg);
    }
    int64_t tiles_per_cta = (n_tiles + kTqScanWarps - 1) / kTqScanWarps;
    c->grid = (int)(tiles_per_cta < qz->rt->sm_count ? (tiles_per_cta > 0 ? tiles_per_cta : 1) : qz->rt->sm_count);
    *out = c;
    return EOS_B200_OK;
}

int ensure_score_workspace(EosB200Corpus* c, int q_count, char** err) {
    const int q_pad = (q_count + kTqTc256Queries - 1) / kTqTc256Queries * kTqTc256Queries;
    if (q_pad <= c->cap_queries) return EOS_B200_OK;
    dev_free(c->d_queries);
    dev_free(c->bfrag);
    dev_free(c->cand);
    dev_free(c->cand_count);
    dev_free(c->shared_tau);
    dev_free(c->seed_keys);
    dev_free(c->d_ids);
    dev_free(c->d_scores);
    dev_free(c->qperm);
    c->qperm_queries = 0;
    c->cap_queries = 0;
    const int ksteps = tq_ksteps(c->qz->dim);
    CUDA_TRY(dev_alloc(&c->d_queries, (size_t)q_pad * c->qz->dim));
    CUDA_TRY(dev_alloc(&c->bfrag, (size_t)(q_pad / 8) * ksteps * 32));
    CUDA_TRY(dev_alloc(&c->cand, (size_t)kTqGroupQueries * c->grid * kTqMaxK));
    CUDA_TRY(dev_alloc(&c->cand_count, (size_t)kTqGroupQueries * c->grid));
    CUDA_TRY(dev_alloc(&c->shared_tau, (size_t)q_pad));
    CUDA_TRY(dev_alloc(&c->seed_keys, (size_t)q_pad * kTqMaxK));
    CUDA_TRY(dev_alloc(&c->d_ids, (size_t)q_pad * kTqMaxK));
    CUDA_TRY(dev_alloc(&c->d_scores, (size_t)q_pad * kTqMaxK));
    c->cap_queries = q_pad;
    return EOS_B200_OK;
}

// Buffers of a tensor-core batch plan; the query capacity follows ensure_score_workspace.
int ensure_tc_workspace(EosB200Corpus* c, int plan, char** err) {
    EosB200Corpus::TcPlan& p = c->tcp[plan];
    const int dimp = tq_ksteps(c->qz->dim) * 16;
    if (c->qperm_queries != c->cap_queries || c->qperm == nullptr) {
        dev_free(c->qperm);
        c->qperm_queries = 0;
        CUDA_TRY(dev_alloc(&c->qperm, (size_t)c->cap_queries * dimp));
        c->qperm_queries = c->cap_queries;
        c->tcp[0].map_queries = c->tcp[1].map_queries = 0;
    }
    if (p.grid == 0) {
        p.queries = plan == 1 ? kTqTc256Queries : kTqTcQueries;
        // The variant of plan 0 with the queries resident in tensor memory is correct but measured slower (0.42 ms against
        // 0.26 ms per launch over 1.25 M rows), so it is opt-in.
        const char* in_tmem = getenv("EOS_B200_TQ_QUERIES_IN_TMEM");
        p.q_in_tmem = plan == 0 && tq_tc_queries_fit_tmem(c->qz->dim) && in_tmem != nullptr && in_tmem[0] != '\0' &&
                      in_tmem[0] != '0';
        p.tile_docs = plan == 1 ? kTqTc256Docs : (p.q_in_tmem ? kTqTcDocsQ : kTqTcDocs);
        p.segs_per_cta = plan == 1 ? 1 : 2;
        const int64_t tiles = (c->n + p.tile_docs - 1) / p.tile_docs;
        const int grid = (int)(tiles < c->qz->rt->sm_count ? (tiles > 0 ? tiles : 1) : c->qz->rt->sm_count);
        // the 256-query plan keeps the lists of up to 16 launches (16 x 77.6 MB on a full grid) and merges them with
        // one launch: a merge of 256 queries is a 40 us launch of 256 blocks, one of 4096 queries fills the GPU
        p.slots = plan == 1 ? kTqTcMergeSlots : 1;
        CUDA_TRY(dev_alloc(&p.cand, (size_t)p.slots * p.queries * p.segs_per_cta * grid * kTqTcSegLen));
        CUDA_TRY(dev_alloc(&p.count, (size_t)p.slots * p.queries * p.segs_per_cta * grid));
        CUDA_TRY(dev_alloc(&p.seed_scores, (size_t)p.slots * p.queries * grid * 256));
        p.grid = grid;
    }
    if (p.map_queries != c->cap_queries) {
        const std::string m = plan == 1 ? tq_tc256_make_query_map(&p.tm, c->qperm, dimp, c->cap_queries)
                                        : tq_tc_make_query_map(&p.tm, c->qperm, dimp, c->cap_queries);
        if (!m.empty()) return fail(err, "score_topk: " + m);
        p.map_queries = c->cap_queries;
    }
    return EOS_B200_OK;
}

// shared_tau[q] = (k-th best key of the sample) - 1, so that the sample's own k-th document still passes; 0 when the
// sample holds fewer than k documents.
__global__ void seed_tau_kernel(const uint64_t* __restrict__ keys, int q_count, int k, unsigned long long* __restrict__ tau) {
    const int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= q_count) return;
    const uint64_t kth = keys[(size_t)q * k + (k - 1)];
    const unsigned long long t = kth != 0 ? kth - 1 : 0;
    if (t > tau[q]) tau[q] = t;  // never below a threshold that is already there
}

// Scan passes of `per_pass` queries over the first n_docs rows + one merge per group of queries.
int enqueue_scan_passes(EosB200Corpus* c, int64_t n_docs, int q_count, int k, int per_pass, bool use_shared_tau,
                        bool profile, int64_t* d_ids, float* d_scores, uint64_t* d_keys, cudaStream_t s) {
    EosB200Quantizer* qz = c->qz;
    const int ksteps = tq_ksteps(qz->dim);
    int launches = 0;
    const int j = per_pass / 8;
    for (int g0 = 0; g0 < q_count; g0 += kTqGroupQueries) {
        const int g_queries = (q_count - g0) < kTqGroupQueries ? (q_count - g0) : kTqGroupQueries;
        const int g_tiles = (g_queries + 7) / 8;
        for (int t0 = 0; t0 < g_tiles; t0 += j) {
            TqScanArgs a{};
            a.tiles = c->tiles;
            a.norms = c->norms;
            a.n_docs = n_docs;
            a.id_base = (uint32_t)c->id_base;
            a.dim = qz->dim;
            a.bfrag = c->bfrag + (size_t)(g0 / 8 + t0) * ksteps * 32;
            a.query_tiles = j;
            a.k = k;
            a.mag_hi[0] = qz->mag_hi[0];
            a.mag_hi[1] = qz->mag_hi[1];
            a.mag_lo[0] = qz->mag_lo[0];
            a.mag_lo[1] = qz->mag_lo[1];
            a.cand_keys = c->cand + (size_t)t0 * 8 * c->grid * kTqMaxK;
            a.cand_count = c->cand_count + (size_t)t0 * 8 * c->grid;
            a.grid = c->grid;
            a.shared_tau = (use_shared_tau && j == 1) ? c->shared_tau + (size_t)g0 + (size_t)t0 * 8 : nullptr;
            a.all_scores = nullptr;
            a.status = qz->rt->d_status;
            a.all_stride = 0;
            if (profile) c->prof.launch(kClsScan, s, [&] { launch_tq_scan(a, s); });
            else launch_tq_scan(a, s);
            launches++;
        }
        launch_tq_merge(c->cand, (int64_t)c->grid * kTqMaxK, kTqMaxK, c->grid, kTqMaxK, c->cand_count, g_queries, k,
                        0, d_ids != nullptr ? d_ids + (size_t)g0 * k : nullptr,
                        d_scores != nullptr ? d_scores + (size_t)g0 * k : nullptr,
                        d_keys != nullptr ? d_keys + (size_t)g0 * k : nullptr, s);
        launches++;
    }
    return launches;
}

// Tensor-core launches of one plan over the first n_docs rows.  seed = true: the scores of each launch become the
// pruning thresholds of its queries (shared_tau); otherwise the lists are merged into the top-k outputs.
int enqueue_tc_passes(EosB200Corpus* c, int plan, int64_t n_docs, int q_count, int k, bool seed, bool profile,
                      int64_t* d_ids, float* d_scores, uint64_t* d_keys, cudaStream_t s) {
    EosB200Quantizer* qz = c->qz;
    EosB200Corpus::TcPlan& p = c->tcp[plan];
    const int64_t tiles = (n_docs + p.tile_docs - 1) / p.tile_docs;
    const int grid = (int)(tiles < p.grid ? tiles : p.grid);
    const int n_segs = p.segs_per_cta * grid;
    int launches = 0;
    // lists (or, in seed mode, sample scores) of the launches since the last merge: launch i of them writes slot i of
    // the workspace; what belongs to all their queries is then contiguous ([slot][query][...]) and one launch -- the
    // list merge, or the threshold select of the seed mode -- serves them all
    const size_t slot_lists = (size_t)p.queries * n_segs;
    int pending = 0, pending_q0 = 0, slot = 0;
    auto merge = [&] {
        if (pending == 0) return;
        if (seed)   // the sample's scores of all pending queries -> their thresholds
            launch_tq_seed_tau_scores(p.seed_scores, n_docs, (int)n_docs, pending, k, c->shared_tau + pending_q0, s);
        else
            launch_tq_merge_lists(p.cand, (int64_t)n_segs * kTqTcSegLen, kTqTcSegLen, n_segs, kTqTcSegLen, p.count, pending,
                                  k, d_ids != nullptr ? d_ids + (size_t)pending_q0 * k : nullptr,
                                  d_scores != nullptr ? d_scores + (size_t)pending_q0 * k : nullptr,
                                  d_keys != nullptr ? d_keys + (size_t)pending_q0 * k : nullptr, s);
        ++launches;
        pending_q0 += pending;
        pending = 0;
        slot = 0;
    };
    for (int q0 = 0; q0 < q_count; q0 += p.queries) {
        const int q_here = (q_count - q0) < p.queries ? (q_count - q0) : p.queries;
        TqTcArgs a{};
        a.tiles = c->tiles;
        a.norms = c->norms;
        a.n_docs = n_docs;
        a.id_base = (uint32_t)c->id_base;
        a.dim = qz->dim;
        a.q_row0 = q0;
        a.q_valid = q_here;
        a.k = k;
        a.mag_hi[0] = qz->mag_hi[0];
        a.mag_hi[1] = qz->mag_hi[1];
        a.mag_lo[0] = qz->mag_lo[0];
        a.mag_lo[1] = qz->mag_lo[1];
        a.cand_keys = p.cand + (seed ? 0 : (size_t)slot * slot_lists * kTqTcSegLen);
        a.cand_count = p.count + (seed ? 0 : (size_t)slot * slot_lists);
        a.shared_tau = c->shared_tau + q0;
        // seed mode: n_docs = grid * 256 scores per query, a multiple of the tile; slot i holds launch i's queries
        a.seed_scores = seed ? p.seed_scores + (size_t)slot * p.queries * n_docs : nullptr;
        a.seed_stride = n_docs;
        a.qperm = c->qperm;
        a.status = qz->rt->d_status;
        auto launch = [&] {
            if (plan == 1) launch_tq_score_tc256(p.tm, a, grid, s);
            else launch_tq_score_tc(p.tm, a, p.q_in_tmem, grid, s);
        };
        if (profile) c->prof.launch(kClsScan, s, launch);
        else launch();
        ++launches;
        pending += q_here;
        if (++slot == p.slots) merge();
    }
    merge();
    return launches;
}

// Late-interaction launches (plan 0: 128 query vectors per launch = 128 / group queries): every launch walks the whole
// shard and keeps per-query candidate lists of parent keys; the lists of up to 128 queries (several launches) are
// merged by one launch.
int enqueue_maxsim_passes(EosB200Corpus* c, int q_vectors, int group, int children, int k, int64_t* d_ids, float* d_scores,
                          uint64_t* d_keys, cudaStream_t s) {
    EosB200Quantizer* qz = c->qz;
    EosB200Corpus::TcPlan& p = c->tcp[0];
    const int64_t tiles = (c->n + p.tile_docs - 1) / p.tile_docs;
    const int grid = (int)(tiles < p.grid ? tiles : p.grid);
    const int n_segs = p.segs_per_cta * grid;
    const int per_launch = p.queries / group;   // queries of one launch
    int launches = 0;
    int pending = 0;        // queries whose lists wait for the merge
    int first_pending = 0;  // index of the first of them
    auto merge = [&] {
        if (pending == 0) return;
        const size_t out0 = (size_t)first_pending * k;
        launch_tq_merge_lists(p.cand, (int64_t)n_segs * kTqTcSegLen, kTqTcSegLen, n_segs, kTqTcSegLen, p.count, pending, k,
                              d_ids != nullptr ? d_ids + out0 : nullptr, d_scores != nullptr ? d_scores + out0 : nullptr,
                              d_keys != nullptr ? d_keys + out0 : nullptr, s);
        ++launches;
        first_pending += pending;
        pending = 0;
    };
    for (int q0 = 0; q0 < q_vectors; q0 += p.queries) {
        const int q_here = (q_vectors - q0) < p.queries ? (q_vectors - q0) : p.queries;
        if (pending + per_launch > p.queries) merge();
        TqTcArgs a{};
        a.tiles = c->tiles;
        a.norms = c->norms;
        a.n_docs = c->n;
        a.id_base = (uint32_t)c->id_base;
        a.dim = qz->dim;
        a.q_row0 = q0;
        a.q_valid = q_here;
        a.k = k;
        a.mag_hi[0] = qz->mag_hi[0];
        a.mag_hi[1] = qz->mag_hi[1];
        a.mag_lo[0] = qz->mag_lo[0];
        a.mag_lo[1] = qz->mag_lo[1];
        a.cand_keys = p.cand;
        a.cand_count = p.count;
        a.shared_tau = c->shared_tau + q0 / group;
        a.seed_scores = nullptr;
        a.seed_stride = 0;
        a.qperm = c->qperm;
        a.status = qz->rt->d_status;
        a.maxsim_children = children;
        a.maxsim_group = group;
        a.maxsim_list_base = pending;
        c->prof.launch(kClsScan, s, [&] { launch_tq_score_tc(p.tm, a, p.q_in_tmem, grid, s); });
        ++launches;
        pending += q_here / group;
    }
    merge();
    return launches;
}

// Rows of the second threshold sample (0 = none).  A threshold that is the k-th best score of s rows lets about
// k n / s of a shard's n rows into each query's candidate lists, and handling those costs the batch kernel about 42 ns
// per candidate and query of a launch (measured at 768 dimensions: 0.14 ms per launch of 256 queries at 3300
// candidates each, whatever the shard's size).  Scoring a sample of f n rows costs f of a launch per group of
// queries a rank seeds; with `sharing` ranks splitting the seeding of a batch, total time is least at
// f = sqrt(sharing * 108 k (768 / padded dim) / n): 1/30 for one GPU at 10 M rows, 1/4 for eight GPUs at 1.25 M each.
// A sample under four times the first one (grid * 256 rows) tightens too little to pay for its launches.
int64_t second_sample_rows(const EosB200Corpus* c, int64_t seed_docs, int k, int sharing) {
    if (c->n <= 0) return 0;
    const double dimp = (double)tq_ksteps(c->qz->dim) * 16.0;
    double f = std::sqrt((double)(sharing > 0 ? sharing : 1) * 108.0 * (double)k * (768.0 / dimp) / (double)c->n);
    if (f < 1.0 / 32.0) f = 1.0 / 32.0;
    if (f > 0.5) f = 0.5;
    const int64_t rows = (int64_t)(f * (double)c->n) / 256 * 256;
    return rows >= 4 * seed_docs ? rows : 0;
}

// The batch paths.  Thresholds are seeded from the first grid * 256 rows (every score written out, k-th best per
// query); on a large shard a second sample of 1/32 of the rows, scored with those thresholds and merged like the real
// pass, tightens them further, so that the lists of the full pass stay short (no list is cut, and the merge gathers a
// few thousand keys per query).  Then the whole shard.
// d_tau_in, when non-null, holds one threshold per query supplied by the caller (for instance seeded on other shards
// and gathered): it replaces the seeding passes.  With thresholds that are lower bounds of the k-th best key of the
// whole sharded corpus, the result is the shard's part of the global top-k rather than the shard's own top-k.
int enqueue_score_tc(EosB200Corpus* c, int plan, const float* d_queries, int q_count, int k, int64_t* d_ids,
                     float* d_scores, uint64_t* d_keys, const uint64_t* d_tau_in, cudaStream_t s) {
    const EosB200Corpus::TcPlan& p = c->tcp[plan];
    const int q_pad = (q_count + p.queries - 1) / p.queries * p.queries;
    int launches = 1;
    launch_tq_prepare(d_queries, q_count, q_pad, c->qz->spec(), nullptr, nullptr, c->qperm, s);
    cudaMemsetAsync(c->shared_tau, 0, (size_t)q_pad * sizeof(unsigned long long), s);
    const int64_t seed_docs = (int64_t)p.grid * 256;
    if (d_tau_in != nullptr) {
        cudaMemcpyAsync(c->shared_tau, d_tau_in, (size_t)q_count * sizeof(unsigned long long), cudaMemcpyDeviceToDevice, s);
    } else if (c->n >= 8 * seed_docs && k <= seed_docs) {
        launches += enqueue_tc_passes(c, plan, seed_docs, q_count, k, true, false, nullptr, nullptr, nullptr, s);
        const int64_t second = second_sample_rows(c, seed_docs, k, 1);
        if (second > 0) {
            launches += enqueue_tc_passes(c, plan, second, q_count, k, false, false, nullptr, nullptr, c->seed_keys, s);
            seed_tau_kernel<<<(q_count + 255) / 256, 256, 0, s>>>(c->seed_keys, q_count, k, c->shared_tau);
            launches++;
        }
    }
    launches += enqueue_tc_passes(c, plan, c->n, q_count, k, false, true, d_ids, d_scores, d_keys, s);
    return launches;
}

// valid[q] = 1 when the lists of query q hold its exact top-k for a k above the kernel's own list size: no CTA cut a
// list (the shared threshold still is the seeded one: a cut always publishes a higher one), no list ran over, and at
// least k candidates exist, i.e. every document above the seeded threshold is in a list and the k-th best is among them.
__global__ void wide_check_kernel(const int* __restrict__ counts, int n_segs, int seg_len, const unsigned long long* __restrict__ tau_now,
                                  const unsigned long long* __restrict__ tau_seed, int q_count, int k, int* __restrict__ valid) {
    const int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= q_count) return;
    long long total = 0;
    bool over = false;
    for (int i = 0; i < n_segs; ++i) {
        const int cnt = counts[(size_t)q * n_segs + i];
        over |= cnt > seg_len;
        total += cnt;
    }
    valid[q] = (!over && tau_now[q] == tau_seed[q] && total >= k) ? 1 : 0;
}

// The 256-query batch kernel for k above its list size (128 < k <= 256): one pass with the kernel's own k = 128, then
// a merge of the per-CTA lists for the caller's k and a validity flag per query (wide_check_kernel).  Queries whose
// flag is 0 have to be answered by the all-scores path.
int enqueue_score_tc_wide(EosB200Corpus* c, const float* d_queries, int q_count, int k, int64_t* d_ids, float* d_scores,
                          int* d_valid, cudaStream_t s) {
    const int plan = 1;
    EosB200Corpus::TcPlan& p = c->tcp[plan];
    EosB200Quantizer* qz = c->qz;
    const int q_pad = (q_count + p.queries - 1) / p.queries * p.queries;
    int launches = 1;
    launch_tq_prepare(d_queries, q_count, q_pad, qz->spec(), nullptr, nullptr, c->qperm, s);
    cudaMemsetAsync(c->shared_tau, 0, (size_t)q_pad * sizeof(unsigned long long), s);
    const int64_t seed_docs = (int64_t)p.grid * 256;
    launches += enqueue_tc_passes(c, plan, seed_docs, q_count, kTqMaxK, true, false, nullptr, nullptr, nullptr, s);
    if (c->n >= 64 * seed_docs) {
        const int64_t second = c->n / 32 / 256 * 256;
        launches += enqueue_tc_passes(c, plan, second, q_count, kTqMaxK, false, false, nullptr, nullptr, c->seed_keys, s);
        seed_tau_kernel<<<(q_count + 255) / 256, 256, 0, s>>>(c->seed_keys, q_count, kTqMaxK, c->shared_tau);
        launches++;
    }
    // the seeded thresholds, kept for the check (seed_keys is free once the thresholds are made)
    unsigned long long* tau_seed = reinterpret_cast<unsigned long long*>(c->seed_keys);
    cudaMemcpyAsync(tau_seed, c->shared_tau, (size_t)q_pad * sizeof(unsigned long long), cudaMemcpyDeviceToDevice, s);
    const int64_t tiles = (c->n + p.tile_docs - 1) / p.tile_docs;
    const int grid = (int)(tiles < p.grid ? tiles : p.grid);
    const int n_segs = p.segs_per_cta * grid;
    for (int q0 = 0; q0 < q_count; q0 += p.queries) {
        const int q_here = (q_count - q0) < p.queries ? (q_count - q0) : p.queries;
        TqTcArgs a{};
        a.tiles = c->tiles;
        a.norms = c->norms;
        a.n_docs = c->n;
        a.id_base = (uint32_t)c->id_base;
        a.dim = qz->dim;
        a.q_row0 = q0;
        a.q_valid = q_here;
        a.k = kTqMaxK;
        a.mag_hi[0] = qz->mag_hi[0];
        a.mag_hi[1] = qz->mag_hi[1];
        a.mag_lo[0] = qz->mag_lo[0];
        a.mag_lo[1] = qz->mag_lo[1];
        a.cand_keys = p.cand;
        a.cand_count = p.count;
        a.shared_tau = c->shared_tau + q0;
        a.seed_scores = nullptr;
        a.seed_stride = c->n;
        a.qperm = c->qperm;
        a.status = qz->rt->d_status;
        launch_tq_score_tc256(p.tm, a, grid, s);
        wide_check_kernel<<<(q_here + 255) / 256, 256, 0, s>>>(p.count, n_segs, kTqTcSegLen, c->shared_tau + q0, tau_seed + q0,
                                                               q_here, k, d_valid + q0);
        launch_tq_merge(p.cand, (int64_t)n_segs * kTqTcSegLen, kTqTcSegLen, n_segs, kTqTcSegLen, p.count, q_here, k, 0,
                        d_ids + (size_t)q0 * k, d_scores + (size_t)q0 * k, nullptr, s);
        launches += 3;
    }
    return launches;
}

// Enqueues prepare + scan passes + merges; returns launches (or -1 with *err set).
int enqueue_score(EosB200Corpus* c, const float* d_queries, int q_count, int k, int per_pass, int64_t* d_ids,
                  float* d_scores, uint64_t* d_keys, cudaStream_t s) {
    EosB200Quantizer* qz = c->qz;
    if (per_pass == kTqTcQueries || per_pass == kTqTc256Queries)
        return enqueue_score_tc(c, per_pass == kTqTc256Queries ? 1 : 0, d_queries, q_count, k, d_ids, d_scores, d_keys,
                                nullptr, s);
    int launches = 0;
    launch_tq_prepare(d_queries, q_count, (q_count + 31) / 32 * 32, qz->spec(), c->bfrag, nullptr, nullptr, s);
    launches++;
    // One pruning threshold per query, shared by the CTAs of the pass that scores it (streaming kernel, 8 queries per
    // pass).  It starts from a sample: the k-th best key among the first kSeedDocs rows is a lower bound of the k-th best
    // key of the whole shard, costs a fraction of a percent of the scan (32 queries per pass over 6 MB of codes), and
    // spares every CTA of every pass the phase in which nearly every document is still a candidate.
    constexpr int64_t kSeedDocs = 16384;
    const bool seeded = per_pass == 8 && c->n >= 8 * kSeedDocs && k <= kSeedDocs;
    if (per_pass == 8)
        cudaMemsetAsync(c->shared_tau, 0, (size_t)((q_count + 31) / 32 * 32) * sizeof(unsigned long long), s);
    if (seeded) {
        launches += enqueue_scan_passes(c, kSeedDocs, q_count, k, 32, false, false, nullptr, nullptr, c->seed_keys, s);
        seed_tau_kernel<<<(q_count + 255) / 256, 256, 0, s>>>(c->seed_keys, q_count, k, c->shared_tau);
        launches++;
    }
    launches += enqueue_scan_passes(c, c->n, q_count, k, per_pass, true, true, d_ids, d_scores, d_keys, s);
    return launches;
}

// queries_per_pass = 0 lets the library choose: the streaming scan for one pass' worth of queries, the batch kernels
// above (4 M rows x 768, 4 bits: 8 queries 0.65 ms by the scan; 12 and 16 queries 1.1 ms by two passes of the scan,
// 0.95 ms by one launch of the 128-query kernel, whose time hardly depends on how many of its queries exist).
int resolve_per_pass(int per_pass, int q_count) {
    if (per_pass != 0) return per_pass;
    if (q_count <= 8) return 8;
    return q_count <= kTqTcQueries ? kTqTcQueries : kTqTc256Queries;
}

int wide_topk(EosB200Corpus* c, const struct ::EosB200IpCorpus* ip, const float* h_queries, const float* h_sketch,
              float qjl_scale, int q_count, int k, int64_t* h_ids, float* h_scores, EosB200Stats* stats, const char* what,
              char** err);

std::string check_score_args(const EosB200Corpus* c, int q_count, int k, int per_pass) {
    if (q_count <= 0) return "score_topk: no queries";
    if (k <= 0 || k > kTqMaxK) return "score_topk: k must be in [1, 128] (the host call eos_b200_score_topk takes up to 256)";
    if (per_pass != 8 && per_pass != 16 && per_pass != 32 && per_pass != kTqTcQueries && per_pass != kTqTc256Queries)
        return "score_topk: queries_per_pass must be 0 (automatic), 8, 16, 32, 128 or 256";
    if (c->n + c->id_base > 0xffffffffLL || c->id_base < 0) return "score_topk: document ids must fit 32 bits";
    return "";
}

}  // namespace

extern "C" {

void eos_b200_quantizer_destroy(EosB200Quantizer* qz) {
    if (qz == nullptr) return;
    cudaSetDevice(qz->rt->device);
    dev_free(qz->perm);
    dev_free(qz->signs1);
    dev_free(qz->signs2);
    dev_free(qz->centroids);
    dev_free(qz->boundaries);
    delete qz;
}

int eos_b200_quantizer_create(EosB200Runtime* rt, int dim, int bits, const int32_t* perm, const float* signs1,
                              const float* signs2, const float* centroids, const float* boundaries,
                              EosB200Quantizer** out, char** err) {
    if (rt == nullptr || perm == nullptr || signs1 == nullptr || signs2 == nullptr || centroids == nullptr ||
        boundaries == nullptr || out == nullptr)
        return fail(err, "quantizer_create: null argument");
    *out = nullptr;
    if (dim <= 0) return fail(err, "quantizer_create: dim must be positive");
    {
        const std::string why = tq_check_dim(dim);
        if (!why.empty()) return fail(err, "quantizer_create: " + why);
    }
    if (bits != 2 && bits != 4) return fail(err, "quantizer_create: bits must be 2 or 4");
    const int levels = 1 << bits;
    std::vector<char> seen((size_t)dim, 0);
    for (int i = 0; i < dim; ++i) {
        if (perm[i] < 0 || perm[i] >= dim || seen[perm[i]]) return fail(err, "quantizer_create: perm is not a permutation");
        seen[perm[i]] = 1;
    }
    for (int i = 0; i + 1 < levels; ++i)
        if (!(centroids[i] < centroids[i + 1])) return fail(err, "quantizer_create: centroids must be ascending");
    uint16_t mag[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int m = 0; m < levels / 2; ++m) {
        const __half pos = __float2half_rn(centroids[levels / 2 + m]);
        const __half neg = __float2half_rn(centroids[levels / 2 - 1 - m]);
        const uint16_t pb = *reinterpret_cast<const uint16_t*>(&pos), nb = *reinterpret_cast<const uint16_t*>(&neg);
        if ((pb ^ 0x8000u) != nb || (pb & 0x8000u))
            return fail(err, "quantizer_create: the centroid table must be symmetric (c[L-1-i] == -c[i])");
        mag[m] = pb;
    }
    CUDA_TRY(cudaSetDevice(rt->device));
    EosB200Quantizer* qz = new EosB200Quantizer();
    qz->rt = rt;
    qz->dim = dim;
    qz->bits = bits;
    for (int m = 0; m < 8; ++m) {
        qz->mag_hi[m / 4] |= (uint32_t)(mag[m] >> 8) << (8 * (m % 4));
        qz->mag_lo[m / 4] |= (uint32_t)(mag[m] & 0xff) << (8 * (m % 4));
    }
    cudaError_t e = dev_alloc(&qz->perm, (size_t)dim);
    if (e == cudaSuccess) e = cudaMemcpy(qz->perm, perm, (size_t)dim * 4, cudaMemcpyHostToDevice);
    std::string msg;
    if (e != cudaSuccess) msg = std::string("quantizer_create: ") + cudaGetErrorString(e);
    if (msg.empty()) msg = upload_f32(signs1, dim, &qz->signs1);
    if (msg.empty()) msg = upload_f32(signs2, dim, &qz->signs2);
    if (msg.empty()) msg = upload_f32(centroids, levels, &qz->centroids);
    if (msg.empty()) msg = upload_f32(boundaries, levels - 1, &qz->boundaries);
    if (!msg.empty()) {
        eos_b200_quantizer_destroy(qz);
        return fail(err, msg);
    }
    *out = qz;
    return EOS_B200_OK;
}

int eos_b200_quantize_device(EosB200Quantizer* qz, const float* d_x, int64_t n, uint8_t* d_codes, float* d_norms,
                             void* stream, char** err) {
    if (qz == nullptr || d_x == nullptr || d_codes == nullptr || d_norms == nullptr)
        return fail(err, "quantize: null argument");
    if (n < 0) return fail(err, "quantize: negative row count");
    CUDA_TRY(cudaSetDevice(qz->rt->device));
    launch_tq_pack(d_x, n, qz->spec(), d_codes, d_norms, pick_stream(qz->rt, stream));
    CUDA_TRY(cudaGetLastError());
    return EOS_B200_OK;
}

int eos_b200_quantize(EosB200Quantizer* qz, const float* h_x, int64_t n, uint8_t* h_codes, float* h_norms,
                      EosB200Stats* stats, char** err) {
    if (qz == nullptr || h_x == nullptr || h_codes == nullptr || h_norms == nullptr)
        return fail(err, "quantize: null argument");
    if (n <= 0) return fail(err, "quantize: no vectors");
    EosB200Runtime* rt = qz->rt;
    CUDA_TRY(cudaSetDevice(rt->device));
    const size_t cb = ((size_t)qz->dim * qz->bits + 7) / 8;
    float *d_x = nullptr, *d_norms = nullptr;
    uint8_t* d_codes = nullptr;
    cudaError_t e = dev_alloc(&d_x, (size_t)n * qz->dim);
    if (e == cudaSuccess) e = dev_alloc(&d_codes, (size_t)n * cb);
    if (e == cudaSuccess) e = dev_alloc(&d_norms, (size_t)n);
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev0, rt->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_x, h_x, (size_t)n * qz->dim * 4, cudaMemcpyHostToDevice, rt->stream);
    if (e == cudaSuccess) {
        launch_tq_pack(d_x, n, qz->spec(), d_codes, d_norms, rt->stream);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_codes, d_codes, (size_t)n * cb, cudaMemcpyDeviceToHost, rt->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_norms, d_norms, (size_t)n * 4, cudaMemcpyDeviceToHost, rt->stream);
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev1, rt->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(rt->stream);
    if (e == cudaSuccess && stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = 2;
        stats->uploaded_bytes = (int64_t)n * qz->dim * 4;
        stats->downloaded_bytes = (int64_t)n * (cb + 4);
        cudaEventElapsedTime(&stats->device_ms, rt->ev0, rt->ev1);
    }
    dev_free(d_x);
    dev_free(d_codes);
    dev_free(d_norms);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(err, std::string("quantize: ") + cudaGetErrorString(e));
    }
    return EOS_B200_OK;
}

void eos_b200_corpus_destroy(EosB200Corpus* c) {
    if (c == nullptr) return;
    cudaSetDevice(c->qz->rt->device);
    cudaStreamSynchronize(c->qz->rt->stream);
    dev_free(c->tiles);
    dev_free(c->norms);
    dev_free(c->d_queries);
    dev_free(c->bfrag);
    dev_free(c->cand);
    dev_free(c->cand_count);
    dev_free(c->shared_tau);
    dev_free(c->seed_keys);
    dev_free(c->d_ids);
    dev_free(c->d_scores);
    dev_free(c->qperm);
    for (auto& p : c->tcp) {
        dev_free(p.cand);
        dev_free(p.count);
        dev_free(p.seed_scores);
    }
    c->prof.reset();
    delete c;
}

int eos_b200_corpus_profile_begin(EosB200Corpus* c, int max_launches, char** err) {
    if (c == nullptr || max_launches <= 0) return fail(err, "corpus_profile_begin: bad argument");
    CUDA_TRY(cudaSetDevice(c->qz->rt->device));
    if (!c->prof.begin(max_launches)) return fail(err, "corpus_profile_begin: cudaEventCreate failed");
    return EOS_B200_OK;
}

int eos_b200_corpus_profile_end(EosB200Corpus* c, void* stream, float* out_ms, int* out_launches, char** err) {
    if (c == nullptr || out_ms == nullptr || out_launches == nullptr) return fail(err, "corpus_profile_end: null argument");
    CUDA_TRY(cudaSetDevice(c->qz->rt->device));
    CUDA_TRY(cudaStreamSynchronize(pick_stream(c->qz->rt, stream)));
    float total = 0.f;
    for (int i = 0; i < c->prof.used; ++i) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, c->prof.ev[(size_t)i * 2], c->prof.ev[(size_t)i * 2 + 1]);
        total += ms;
    }
    *out_ms = total;
    *out_launches = c->prof.used;
    c->prof.reset();
    return EOS_B200_OK;
}

int64_t eos_b200_corpus_vector_bytes(const EosB200Corpus* c) {
    if (c == nullptr) return 0;
    return ((int64_t)c->qz->dim * c->qz->bits + 7) / 8 + 4;
}

int eos_b200_corpus_bind_device(EosB200Quantizer* qz, const uint8_t* d_codes, const float* d_norms, int64_t n,
                                int64_t id_base, EosB200Corpus** out, char** err) {
    if (qz == nullptr || out == nullptr || (n > 0 && (d_codes == nullptr || d_norms == nullptr)))
        return fail(err, "corpus_bind: null argument");
    *out = nullptr;
    if (n < 0 || id_base < 0 || n + id_base > 0xffffffffLL) return fail(err, "corpus_bind: row ids must fit 32 bits");
    CUDA_TRY(cudaSetDevice(qz->rt->device));
    return corpus_finish_bind(qz, d_codes, d_norms, n, id_base, out, err);
}

int eos_b200_corpus_bind(EosB200Quantizer* qz, const uint8_t* h_codes, const float* h_norms, int64_t n,
                         int64_t id_base, int allow_zero_norm, EosB200Corpus** out, char** err) {
    if (qz == nullptr || out == nullptr || (n > 0 && (h_codes == nullptr || h_norms == nullptr)))
        return fail(err, "corpus_bind: null argument");
    *out = nullptr;
    if (n < 0 || id_base < 0 || n + id_base > 0xffffffffLL) return fail(err, "corpus_bind: row ids must fit 32 bits");
    for (int64_t i = 0; i < n; ++i) {
        const float v = h_norms[i];
        if (std::isnan(v) || std::isinf(v) || v < 0 || (v == 0 && !allow_zero_norm))
            return fail(err, "corpus_bind: quantized vector norm must be positive and finite (row " +
                                 std::to_string(i) + "); pass allow_zero_norm for confirmed zero vectors");
    }
    CUDA_TRY(cudaSetDevice(qz->rt->device));
    const size_t cb = ((size_t)qz->dim * qz->bits + 7) / 8;
    uint8_t* d_codes = nullptr;
    float* d_norms = nullptr;
    cudaError_t e = dev_alloc(&d_codes, (size_t)n * cb);
    if (e == cudaSuccess) e = dev_alloc(&d_norms, (size_t)n);
    if (e == cudaSuccess && n > 0) e = cudaMemcpy(d_codes, h_codes, (size_t)n * cb, cudaMemcpyHostToDevice);
    if (e == cudaSuccess && n > 0) e = cudaMemcpy(d_norms, h_norms, (size_t)n * 4, cudaMemcpyHostToDevice);
    int rc;
    if (e != cudaSuccess) {
        cudaGetLastError();
        rc = fail(err, std::string("corpus_bind: ") + cudaGetErrorString(e));
    } else {
        rc = corpus_finish_bind(qz, d_codes, d_norms, n, id_base, out, err);
    }
    dev_free(d_codes);
    dev_free(d_norms);
    return rc;
}

int eos_b200_score_topk_device(EosB200Corpus* c, const float* d_queries, int q_count, int k, int per_pass,
                               int64_t* d_ids, float* d_scores, uint64_t* d_keys, void* stream, EosB200Stats* stats,
                               char** err) {
    if (c == nullptr || d_queries == nullptr) return fail(err, "score_topk: null argument");
    if ((d_ids == nullptr) != (d_scores == nullptr))
        return fail(err, "score_topk: d_ids and d_scores must be given together or both be null");
    if (d_ids == nullptr && d_keys == nullptr) return fail(err, "score_topk: no output requested");
    per_pass = resolve_per_pass(per_pass, q_count);
    std::string m = check_score_args(c, q_count, k, per_pass);
    if (!m.empty()) return fail(err, m);
    if (c->n == 0) return fail(err, "score_topk: empty corpus");
    CUDA_TRY(cudaSetDevice(c->qz->rt->device));
    int rc = ensure_score_workspace(c, q_count, err);
    if (rc == EOS_B200_OK && (per_pass == kTqTcQueries || per_pass == kTqTc256Queries))
        rc = ensure_tc_workspace(c, per_pass == kTqTc256Queries ? 1 : 0, err);
    if (rc != EOS_B200_OK) return rc;
    const int launches =
        enqueue_score(c, d_queries, q_count, k, per_pass, d_ids, d_scores, d_keys, pick_stream(c->qz->rt, stream));
    CUDA_TRY(cudaGetLastError());
    if (stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = launches;
    }
    return EOS_B200_OK;
}

// Thresholds of q_count queries from samples of this shard.  sharing = ranks that split the seeding of one batch
// between them (each calls this for its slice): the more they are, the larger the second sample that pays.
static int score_seed_shared(EosB200Corpus* c, const float* d_queries, int q_count, int k, uint64_t* d_tau_out, int sharing,
                      void* stream, int* launches_out, char** err) {
    if (c == nullptr || d_queries == nullptr || d_tau_out == nullptr) return fail(err, "score_seed: null argument");
    std::string m = check_score_args(c, q_count, k, kTqTc256Queries);
    if (!m.empty()) return fail(err, m);
    CUDA_TRY(cudaSetDevice(c->qz->rt->device));
    cudaStream_t s = pick_stream(c->qz->rt, stream);
    int launches = 0;
    if (launches_out != nullptr) *launches_out = 0;
    if (c->n == 0) {
        CUDA_TRY(cudaMemsetAsync(d_tau_out, 0, (size_t)q_count * sizeof(uint64_t), s));
        return EOS_B200_OK;
    }
    int rc = ensure_score_workspace(c, q_count, err);
    if (rc == EOS_B200_OK) rc = ensure_tc_workspace(c, 1, err);
    if (rc != EOS_B200_OK) return rc;
    const EosB200Corpus::TcPlan& p = c->tcp[1];
    const int q_pad = (q_count + p.queries - 1) / p.queries * p.queries;
    launch_tq_prepare(d_queries, q_count, q_pad, c->qz->spec(), nullptr, nullptr, c->qperm, s);
    launches++;
    CUDA_TRY(cudaMemsetAsync(c->shared_tau, 0, (size_t)q_pad * sizeof(unsigned long long), s));
    const int64_t seed_docs = (int64_t)p.grid * 256;
    if (c->n >= seed_docs && k <= seed_docs) {
        launches += enqueue_tc_passes(c, 1, seed_docs, q_count, k, true, false, nullptr, nullptr, nullptr, s);
        const int64_t second = second_sample_rows(c, seed_docs, k, sharing);
        if (second > 0) {
            launches += enqueue_tc_passes(c, 1, second, q_count, k, false, false, nullptr, nullptr, c->seed_keys, s);
            seed_tau_kernel<<<(q_count + 255) / 256, 256, 0, s>>>(c->seed_keys, q_count, k, c->shared_tau);
            launches++;
        }
    }
    CUDA_TRY(cudaMemcpyAsync(d_tau_out, c->shared_tau, (size_t)q_count * sizeof(uint64_t), cudaMemcpyDeviceToDevice, s));
    CUDA_TRY(cudaGetLastError());
    if (launches_out != nullptr) *launches_out = launches;
    return EOS_B200_OK;
}

int eos_b200_score_seed_device(EosB200Corpus* c, const float* d_queries, int q_count, int k, uint64_t* d_tau_out,
                               void* stream, char** err) {
    return score_seed_shared(c, d_queries, q_count, k, d_tau_out, 1, stream, nullptr, err);
}

int eos_b200_score_topk_seeded_device(EosB200Corpus* c, const float* d_queries, int q_count, int k, const uint64_t* d_tau,
                                      int64_t* d_ids, float* d_scores, uint64_t* d_keys, void* stream,
                                      EosB200Stats* stats, char** err) {
    if (c == nullptr || d_queries == nullptr || d_tau == nullptr) return fail(err, "score_topk_seeded: null argument");
    if ((d_ids == nullptr) != (d_scores == nullptr))
        return fail(err, "score_topk_seeded: d_ids and d_scores must be given together or both be null");
    if (d_ids == nullptr && d_keys == nullptr) return fail(err, "score_topk_seeded: no output requested");
    const int per_pass = q_count <= kTqTcQueries ? kTqTcQueries : kTqTc256Queries;
    std::string m = check_score_args(c, q_count, k, per_pass);
    if (!m.empty()) return fail(err, m);
    if (c->n == 0) return fail(err, "score_topk_seeded: empty corpus");
    CUDA_TRY(cudaSetDevice(c->qz->rt->device));
    const int plan = per_pass == kTqTc256Queries ? 1 : 0;
    int rc = ensure_score_workspace(c, q_count, err);
    if (rc == EOS_B200_OK) rc = ensure_tc_workspace(c, plan, err);
    if (rc != EOS_B200_OK) return rc;
    const int launches =
        enqueue_score_tc(c, plan, d_queries, q_count, k, d_ids, d_scores, d_keys, d_tau, pick_stream(c->qz->rt, stream));
    CUDA_TRY(cudaGetLastError());
    if (stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = launches;
    }
    return EOS_B200_OK;
}

int eos_b200_score_topk(EosB200Corpus* c, const float* h_queries, int q_count, int k, int per_pass, int64_t* h_ids,
                        float* h_scores, EosB200Stats* stats, char** err) {
    if (c == nullptr || h_queries == nullptr || h_ids == nullptr || h_scores == nullptr)
        return fail(err, "score_topk: null argument");
    per_pass = resolve_per_pass(per_pass, q_count);
    const bool wide = k > kTqMaxK && k <= kTqWideK;   // over-fetch sizes: all scores of a query chunk, then one select
    std::string m = check_score_args(c, q_count, wide ? kTqMaxK : k, per_pass);
    if (!m.empty()) return fail(err, m);
    if (c->n == 0) {  // topK > len(docs): nothing to return (runtime/retrieval_turboquant.go:1854-1860)
        for (size_t i = 0; i < (size_t)q_count * k; ++i) {
            h_ids[i] = -1;
            h_scores[i] = -INFINITY;
        }
        if (stats != nullptr) std::memset(stats, 0, sizeof(*stats));
        return EOS_B200_OK;
    }
    EosB200Runtime* rt = c->qz->rt;
    CUDA_TRY(cudaSetDevice(rt->device));
    if (wide) {
        // One pass of the 256-query batch kernel answers k up to 256 whenever its lists were never cut (the usual
        // case on a seeded corpus: a few thousand candidates per query spread over the CTAs' lists); the queries for
        // which that cannot be shown (flag 0) are answered by the all-scores path.
        int rc = ensure_score_workspace(c, q_count, err);
        if (rc == EOS_B200_OK) rc = ensure_tc_workspace(c, 1, err);
        if (rc != EOS_B200_OK) return rc;
        if (c->n < 8 * (int64_t)c->tcp[1].grid * 256)
            return wide_topk(c, nullptr, h_queries, nullptr, 0.f, q_count, k, h_ids, h_scores, stats, "score_topk", err);
        cudaStream_t s = rt->stream;
        int64_t* d_ids = nullptr;
        float* d_scores = nullptr;
        int* d_valid = nullptr;
        cudaError_t e = dev_alloc(&d_ids, (size_t)q_count * k);
        if (e == cudaSuccess) e = dev_alloc(&d_scores, (size_t)q_count * k);
        if (e == cudaSuccess) e = dev_alloc(&d_valid, (size_t)q_count);
        std::vector<int> valid((size_t)q_count, 0);
        int launches = 0;
        if (e == cudaSuccess) e = cudaEventRecord(rt->ev0, s);
        if (e == cudaSuccess) e = cudaMemsetAsync(rt->d_status, 0, sizeof(int), s);
        if (e == cudaSuccess) e = cudaMemcpyAsync(c->d_queries, h_queries, (size_t)q_count * c->qz->dim * 4, cudaMemcpyHostToDevice, s);
        if (e == cudaSuccess) {
            launches = enqueue_score_tc_wide(c, c->d_queries, q_count, k, d_ids, d_scores, d_valid, s);
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = cudaMemcpyAsync(h_ids, d_ids, (size_t)q_count * k * 8, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess) e = cudaMemcpyAsync(h_scores, d_scores, (size_t)q_count * k * 4, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess) e = cudaMemcpyAsync(valid.data(), d_valid, (size_t)q_count * 4, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess) e = cudaEventRecord(rt->ev1, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
        dev_free(d_ids);
        dev_free(d_scores);
        dev_free(d_valid);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(err, std::string("score_topk: ") + cudaGetErrorString(e));
        }
        rc = read_status(rt, s, err);
        if (rc != EOS_B200_OK) return rc;
        float device_ms = 0.f;
        cudaEventElapsedTime(&device_ms, rt->ev0, rt->ev1);
        std::vector<int> redo;
        for (int q = 0; q < q_count; ++q)
            if (!valid[q]) redo.push_back(q);
        if (!redo.empty()) {
            const int dim = c->qz->dim;
            std::vector<float> rq(redo.size() * (size_t)dim);
            std::vector<int64_t> rid(redo.size() * (size_t)k);
            std::vector<float> rsc(redo.size() * (size_t)k);
            for (size_t i = 0; i < redo.size(); ++i)
                std::memcpy(rq.data() + i * dim, h_queries + (size_t)redo[i] * dim, (size_t)dim * 4);
            EosB200Stats st2{};
            rc = wide_topk(c, nullptr, rq.data(), nullptr, 0.f, (int)redo.size(), k, rid.data(), rsc.data(), &st2, "score_topk", err);
            if (rc != EOS_B200_OK) return rc;
            for (size_t i = 0; i < redo.size(); ++i) {
                std::memcpy(h_ids + (size_t)redo[i] * k, rid.data() + i * k, (size_t)k * 8);
                std::memcpy(h_scores + (size_t)redo[i] * k, rsc.data() + i * k, (size_t)k * 4);
            }
            launches += st2.kernel_launches;
            device_ms += st2.device_ms;
        }
        if (stats != nullptr) {
            std::memset(stats, 0, sizeof(*stats));
            stats->kernel_launches = launches;
            stats->uploaded_bytes = (int64_t)q_count * c->qz->dim * 4;
            stats->downloaded_bytes = (int64_t)q_count * k * 12;
            stats->reserved = (int32_t)redo.size();   // queries answered by the all-scores path
            stats->device_ms = device_ms;
        }
        return EOS_B200_OK;
    }
    int rc = ensure_score_workspace(c, q_count, err);
    if (rc == EOS_B200_OK && (per_pass == kTqTcQueries || per_pass == kTqTc256Queries))
        rc = ensure_tc_workspace(c, per_pass == kTqTc256Queries ? 1 : 0, err);
    if (rc != EOS_B200_OK) return rc;
    cudaStream_t s = rt->stream;
    CUDA_TRY(cudaEventRecord(rt->ev0, s));
    CUDA_TRY(cudaMemsetAsync(rt->d_status, 0, sizeof(int), s));
    CUDA_TRY(cudaMemcpyAsync(c->d_queries, h_queries, (size_t)q_count * c->qz->dim * 4, cudaMemcpyHostToDevice, s));
    const int launches = enqueue_score(c, c->d_queries, q_count, k, per_pass, c->d_ids, c->d_scores, nullptr, s);
    CUDA_TRY(cudaGetLastError());
    CUDA_TRY(cudaMemcpyAsync(h_ids, c->d_ids, (size_t)q_count * k * 8, cudaMemcpyDeviceToHost, s));
    CUDA_TRY(cudaMemcpyAsync(h_scores, c->d_scores, (size_t)q_count * k * 4, cudaMemcpyDeviceToHost, s));
    CUDA_TRY(cudaEventRecord(rt->ev1, s));
    rc = read_status(rt, s, err);   // synchronises; a bounded wait that ran out inside a kernel is an error, not a result
    if (stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = launches;
        stats->uploaded_bytes = (int64_t)q_count * c->qz->dim * 4;
        stats->downloaded_bytes = (int64_t)q_count * k * 12;
        cudaEventElapsedTime(&stats->device_ms, rt->ev0, rt->ev1);
    }
    return rc;
}

int eos_b200_corpus_sync(EosB200Corpus* c, void* stream, char** err) {
    if (c == nullptr) return fail(err, "corpus_sync: null corpus");
    CUDA_TRY(cudaSetDevice(c->qz->rt->device));
    return read_status(c->qz->rt, pick_stream(c->qz->rt, stream), err);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// wide path: all scores of a chunk of queries, optional sign stage, keys, one select per query
// ------------------------------------------------------------------------------------------------
struct EosB200IpCorpus {
    EosB200Quantizer* qz = nullptr;   // 4-bit view of the MSE stage (owned)
    EosB200Corpus* base = nullptr;    // MSE codes as scan tiles + norms (owned)
    uint32_t* signs = nullptr;        // [n][ceil(dim / 32)]
    float* resnorms = nullptr;        // [n]
    int levels = 0;                   // levels of the MSE stage
};

namespace {
constexpr int kWideSegLen = 4096;   // keys per merge segment (one warp each)

// Exact top-k (k <= kTqWideK) of q_count host queries over the whole corpus.  ip == nullptr: the Hadamard/MSE score.
int wide_topk(EosB200Corpus* c, const EosB200IpCorpus* ip, const float* h_queries, const float* h_sketch, float qjl_scale,
              int q_count, int k, int64_t* h_ids, float* h_scores, EosB200Stats* stats, const char* what, char** err) {
    EosB200Runtime* rt = c->qz->rt;
    const int dim = c->qz->dim;
    const int64_t n = c->n;
    const int64_t n_pad = (n + kWideSegLen - 1) / kWideSegLen * kWideSegLen;
    const int64_t n_segs = n_pad / kWideSegLen;
    if (n_segs > 0x7fffffffLL) return fail(err, std::string(what) + ": too many rows");
    // queries per chunk: 12 bytes (score + key) per (query, row), about 3 GB at most, a multiple of 8
    int chunk = (int)std::min<int64_t>(q_count, std::max<int64_t>(8, (int64_t)3e9 / (12 * n_pad)));
    chunk = (chunk + 7) / 8 * 8;
    int rc = ensure_score_workspace(c, chunk, err);
    if (rc != EOS_B200_OK) return rc;
    cudaStream_t s = rt->stream;
    float *d_all = nullptr, *d_sketch = nullptr, *d_scores = nullptr;
    uint64_t* d_keys = nullptr;
    int64_t* d_ids = nullptr;
    cudaError_t e = dev_alloc(&d_all, (size_t)chunk * n);
    if (e == cudaSuccess) e = dev_alloc(&d_keys, (size_t)chunk * n_pad);
    if (e == cudaSuccess) e = dev_alloc(&d_ids, (size_t)chunk * k);
    if (e == cudaSuccess) e = dev_alloc(&d_scores, (size_t)chunk * k);
    if (e == cudaSuccess && ip != nullptr) e = dev_alloc(&d_sketch, (size_t)chunk * dim);
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev0, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(rt->d_status, 0, sizeof(int), s);
    const int ksteps = tq_ksteps(dim);
    int launches = 0;
    for (int q0 = 0; q0 < q_count && e == cudaSuccess; q0 += chunk) {
        const int qn = std::min(chunk, q_count - q0);
        const int q_pad = (qn + 7) / 8 * 8;
        e = cudaMemcpyAsync(c->d_queries, h_queries + (size_t)q0 * dim, (size_t)qn * dim * 4, cudaMemcpyHostToDevice, s);
        if (e != cudaSuccess) break;
        launch_tq_prepare(c->d_queries, qn, q_pad, c->qz->spec(), c->bfrag, nullptr, nullptr, s);
        for (int t = 0; t < q_pad / 8; ++t) {
            TqScanArgs a{};
            a.tiles = c->tiles;
            a.norms = c->norms;
            a.n_docs = n;
            a.id_base = 0;
            a.dim = dim;
            a.bfrag = c->bfrag + (size_t)t * ksteps * 32;
            a.query_tiles = 1;
            a.k = 1;
            a.mag_hi[0] = c->qz->mag_hi[0];
            a.mag_hi[1] = c->qz->mag_hi[1];
            a.mag_lo[0] = c->qz->mag_lo[0];
            a.mag_lo[1] = c->qz->mag_lo[1];
            a.cand_keys = c->cand;
            a.cand_count = c->cand_count;
            a.grid = c->grid;
            a.all_scores = d_all + (size_t)t * 8 * n;
            a.all_stride = n;
            a.status = rt->d_status;
            launch_tq_scan(a, s);
        }
        launches += 1 + q_pad / 8;
        if (ip != nullptr) {
            e = cudaMemcpyAsync(d_sketch, h_sketch + (size_t)q0 * dim, (size_t)qn * dim * 4, cudaMemcpyHostToDevice, s);
            if (e != cudaSuccess) break;
            launch_tq_ip_sign_stage(ip->signs, ip->resnorms, c->norms, n, d_sketch, qn, dim, qjl_scale, d_all, n,
                                    rt->sm_count, s);
            ++launches;
        }
        launch_tq_score_keys(d_all, n, qn, n, n_pad, d_keys, rt->sm_count, s);
        launch_tq_merge(d_keys, n_pad, kWideSegLen, (int)n_segs, kWideSegLen, nullptr, qn, k, c->id_base, d_ids, d_scores,
                        nullptr, s);
        launches += 2;
        e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaMemcpyAsync(h_ids + (size_t)q0 * k, d_ids, (size_t)qn * k * 8, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(h_scores + (size_t)q0 * k, d_scores, (size_t)qn * k * 4, cudaMemcpyDeviceToHost, s);
        // the next chunk reuses the buffers the copies read
        if (e == cudaSuccess && q0 + chunk < q_count) e = cudaStreamSynchronize(s);
    }
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev1, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    dev_free(d_all);
    dev_free(d_keys);
    dev_free(d_ids);
    dev_free(d_scores);
    dev_free(d_sketch);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(err, std::string(what) + ": " + cudaGetErrorString(e));
    }
    if (stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = launches;
        stats->uploaded_bytes = (int64_t)q_count * dim * 4 * (ip != nullptr ? 2 : 1);
        stats->downloaded_bytes = (int64_t)q_count * k * 12;
        cudaEventElapsedTime(&stats->device_ms, rt->ev0, rt->ev1);
    }
    return read_status(rt, s, err);
}
}  // namespace

extern "C" {

void eos_b200_ip_corpus_destroy(EosB200IpCorpus* ip) {
    if (ip == nullptr) return;
    if (ip->base != nullptr) eos_b200_corpus_destroy(ip->base);
    dev_free(ip->signs);
    dev_free(ip->resnorms);
    if (ip->qz != nullptr) eos_b200_quantizer_destroy(ip->qz);
    delete ip;
}

int eos_b200_ip_corpus_bind(EosB200Runtime* rt, int dim, int mse_levels, const int32_t* perm, const float* signs1,
                            const float* signs2, const float* centroids, const uint8_t* h_mse_indices,
                            const uint8_t* h_signs, const float* h_resnorms, const float* h_norms, int64_t n,
                            int64_t id_base, int allow_zero_norm, EosB200IpCorpus** out, char** err) {
    if (rt == nullptr || perm == nullptr || signs1 == nullptr || signs2 == nullptr || centroids == nullptr || out == nullptr ||
        (n > 0 && (h_mse_indices == nullptr || h_signs == nullptr || h_resnorms == nullptr || h_norms == nullptr)))
        return fail(err, "ip_corpus_bind: null argument");
    *out = nullptr;
    if (mse_levels != 2 && mse_levels != 4 && mse_levels != 8 && mse_levels != 16)
        return fail(err, "ip_corpus_bind: the MSE stage must have 2, 4, 8 or 16 levels");
    if (n < 0 || dim <= 0) return fail(err, "ip_corpus_bind: bad sizes");
    for (int64_t i = 0; i < n; ++i) {
        const float r = h_resnorms[i];
        if (std::isnan(r) || std::isinf(r) || r < 0)
            return fail(err, "ip_corpus_bind: residual norm must be finite and non-negative (row " + std::to_string(i) + ")");
    }
    // The scan kernels read 4-bit codes as sign + magnitude of a symmetric 16-level table: level i of the L-level table
    // becomes code 8 - L/2 + i, and the magnitudes the codes never use are filled with larger dummies.
    const int half = mse_levels / 2;
    float c16[16], b15[15];
    for (int m = 0; m < 8; ++m) {
        const float v = m < half ? centroids[half + m] : centroids[mse_levels - 1] + (float)(m - half + 1);
        c16[8 + m] = v;
        c16[7 - m] = m < half ? centroids[half - 1 - m] : -v;
    }
    for (int i = 0; i < 15; ++i) b15[i] = 0.5f * (c16[i] + c16[i + 1]);
    auto* ip = new EosB200IpCorpus();
    ip->levels = mse_levels;
    int rc = eos_b200_quantizer_create(rt, dim, 4, perm, signs1, signs2, c16, b15, &ip->qz, err);
    if (rc != EOS_B200_OK) {
        eos_b200_ip_corpus_destroy(ip);
        return rc;
    }
    const size_t cb = ((size_t)dim + 1) / 2;
    const int words = (dim + 31) / 32;
    std::vector<uint8_t> packed((size_t)(n > 0 ? n : 1) * cb, 0);
    std::vector<uint32_t> sw((size_t)(n > 0 ? n : 1) * words, 0u);
    const size_t sign_bytes = ((size_t)dim + 7) / 8;
    for (int64_t r = 0; r < n; ++r) {
        const uint8_t* src = h_mse_indices + (size_t)r * dim;
        uint8_t* dst = packed.data() + (size_t)r * cb;
        for (int cidx = 0; cidx < dim; ++cidx) {
            if (src[cidx] >= mse_levels) {
                eos_b200_ip_corpus_destroy(ip);
                return fail(err, "ip_corpus_bind: MSE index out of range (row " + std::to_string(r) + ")");
            }
            const uint8_t code = (uint8_t)(8 - half + src[cidx]);
            dst[cidx >> 1] |= (uint8_t)(code << ((cidx & 1) * 4));
        }
        const uint8_t* sb = h_signs + (size_t)r * sign_bytes;
        for (size_t j = 0; j < sign_bytes; ++j) sw[(size_t)r * words + j / 4] |= (uint32_t)sb[j] << (8 * (j % 4));
        if (dim % 8 != 0) sw[(size_t)r * words + (dim >> 5)] &= (dim & 31) ? ((1u << (dim & 31)) - 1u) : 0xffffffffu;
    }
    rc = eos_b200_corpus_bind(ip->qz, packed.data(), h_norms, n, id_base, allow_zero_norm, &ip->base, err);
    if (rc != EOS_B200_OK) {
        eos_b200_ip_corpus_destroy(ip);
        return rc;
    }
    cudaError_t e = dev_alloc(&ip->signs, sw.size());
    if (e == cudaSuccess) e = dev_alloc(&ip->resnorms, (size_t)(n > 0 ? n : 1));
    if (e == cudaSuccess) e = cudaMemcpy(ip->signs, sw.data(), sw.size() * 4, cudaMemcpyHostToDevice);
    if (e == cudaSuccess && n > 0) e = cudaMemcpy(ip->resnorms, h_resnorms, (size_t)n * 4, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaGetLastError();
        eos_b200_ip_corpus_destroy(ip);
        return fail(err, std::string("ip_corpus_bind: ") + cudaGetErrorString(e));
    }
    *out = ip;
    return EOS_B200_OK;
}

// 8-bit log-scale norm side-car of the reference's device encode (manta_tq_quantize_norm / manta_tq_dequantize_norm,
// runtime/backends/cuda/native_linux.go:1879-1904).  Host arithmetic: a caller holding that side-car turns it into
// the fp32 norms eos_b200_corpus_bind takes, or produces it from the norms eos_b200_quantize returns.
void eos_b200_norm_encode_log8(const float* norms, int64_t n, uint8_t* codes) {
    for (int64_t i = 0; i < n; ++i) {
        const float norm = norms[i];
        int code;
        if (norm <= 0.0f || std::isnan(norm)) {
            code = 0;
        } else if (std::isinf(norm)) {
            code = 255;
        } else {
            const float t = (logf(norm) + 16.0f) / 32.0f;
            code = t <= 0.0f ? 0 : (t >= 1.0f ? 255 : (int)roundf(t * 255.0f));
        }
        codes[i] = (uint8_t)code;
    }
}

void eos_b200_norm_decode_log8(const uint8_t* codes, int64_t n, float* norms) {
    for (int64_t i = 0; i < n; ++i) norms[i] = expf(-16.0f + ((float)codes[i] / 255.0f) * 32.0f);
}

int64_t eos_b200_ip_corpus_vector_bytes(int dim, int bit_width) {
    // turboquantVectorBytes (runtime/turboquant_bytes.go:22-25): MSE payload at bit_width - 1 bits, one sign bit per
    // coordinate, two fp32 norm fields
    if (dim <= 0 || bit_width < 2) return 0;
    return ((int64_t)dim * (bit_width - 1) + 7) / 8 + ((int64_t)dim + 7) / 8 + 8;
}

int eos_b200_ip_score_topk(EosB200IpCorpus* ip, const float* h_queries, const float* h_query_sketch, float qjl_scale,
                           int q_count, int k, int64_t* h_ids, float* h_scores, EosB200Stats* stats, char** err) {
    if (ip == nullptr || h_queries == nullptr || h_query_sketch == nullptr || h_ids == nullptr || h_scores == nullptr)
        return fail(err, "ip_score_topk: null argument");
    if (q_count <= 0) return fail(err, "ip_score_topk: no queries");
    if (k <= 0 || k > kTqWideK) return fail(err, "ip_score_topk: k must be in [1, 256]");
    EosB200Corpus* c = ip->base;
    if (c->n == 0) {
        for (size_t i = 0; i < (size_t)q_count * k; ++i) {
            h_ids[i] = -1;
            h_scores[i] = -INFINITY;
        }
        if (stats != nullptr) std::memset(stats, 0, sizeof(*stats));
        return EOS_B200_OK;
    }
    if (tq_ip_sign_stage_smem(c->qz->dim) > 100 * 1024) return fail(err, "ip_score_topk: dim is too wide for the sign stage");
    CUDA_TRY(cudaSetDevice(c->qz->rt->device));
    return wide_topk(c, ip, h_queries, h_query_sketch, qjl_scale, q_count, k, h_ids, h_scores, stats, "ip_score_topk", err);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// multi-GPU scoring: one process per GPU, NCCL between them
// ------------------------------------------------------------------------------------------------
namespace {
// NCCL is resolved at run time (dlopen) so that the library loads, and everything single-GPU works, on a machine
// without it.  Only the handful of entry points the sharded call needs.
struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(void**, int, EosB200NcclId, int) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    std::string error;
};
NcclApi* nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle != nullptr) break;
        }
        if (api.handle == nullptr) {
            api.error = "NCCL library (libnccl.so.2) not found";
            return;
        }
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(api.handle, "ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(api.handle, "ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(api.handle, "ncclCommDestroy"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(api.handle, "ncclAllGather"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(api.handle, "ncclGetErrorString"));
        if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllGather || !api.GetErrorString)
            api.error = "NCCL library lacks a required entry point";
    });
    return &api;
}
constexpr int kNcclChar = 0;  // ncclInt8 / ncclChar: all transfers are counted in bytes
}  // namespace

struct EosB200Comm {
    EosB200Runtime* rt = nullptr;
    void* comm = nullptr;
    int rank = 0, world = 1;
    // buffers of the sharded scoring call, grown on demand
    int cap_queries = 0, cap_k = 0;
    uint64_t *tau_local = nullptr, *tau_all = nullptr, *keys = nullptr, *keys_all = nullptr;
};

extern "C" {

int eos_b200_comm_unique_id(EosB200NcclId* out, char** err) {
    if (out == nullptr) return fail(err, "comm_unique_id: null argument");
    NcclApi* api = nccl_api();
    if (!api->error.empty()) return fail(err, "comm_unique_id: " + api->error);
    const int r = api->GetUniqueId(out);
    if (r != 0) return fail(err, std::string("ncclGetUniqueId: ") + api->GetErrorString(r));
    return EOS_B200_OK;
}

int eos_b200_comm_init(EosB200Runtime* rt, int rank, int world, const EosB200NcclId* id, EosB200Comm** out, char** err) {
    if (rt == nullptr || id == nullptr || out == nullptr) return fail(err, "comm_init: null argument");
    *out = nullptr;
    if (world <= 0 || rank < 0 || rank >= world) return fail(err, "comm_init: rank must be in [0, world)");
    NcclApi* api = nccl_api();
    if (!api->error.empty()) return fail(err, "comm_init: " + api->error);
    CUDA_TRY(cudaSetDevice(rt->device));
    EosB200Comm* c = new EosB200Comm();
    c->rt = rt;
    c->rank = rank;
    c->world = world;
    const int r = api->CommInitRank(&c->comm, world, *id, rank);
    if (r != 0) {
        delete c;
        return fail(err, std::string("ncclCommInitRank: ") + api->GetErrorString(r));
    }
    *out = c;
    return EOS_B200_OK;
}

void eos_b200_comm_destroy(EosB200Comm* c) {
    if (c == nullptr) return;
    cudaSetDevice(c->rt->device);
    cudaStreamSynchronize(c->rt->stream);
    dev_free(c->tau_local);
    dev_free(c->tau_all);
    dev_free(c->keys);
    dev_free(c->keys_all);
    if (c->comm != nullptr) nccl_api()->CommDestroy(c->comm);
    delete c;
}

int eos_b200_score_topk_sharded(EosB200Corpus* c, EosB200Comm* comm, const float* d_queries, int q_count, int k,
                                int queries_per_pass, int64_t* d_ids, float* d_scores, void* stream, EosB200Stats* stats,
                                char** err) {
    if (c == nullptr || comm == nullptr || d_queries == nullptr || d_ids == nullptr || d_scores == nullptr)
        return fail(err, "score_topk_sharded: null argument");
    if (comm->rt != c->qz->rt) return fail(err, "score_topk_sharded: corpus and communicator belong to different runtimes");
    const int per_pass = resolve_per_pass(queries_per_pass, q_count);
    std::string m = check_score_args(c, q_count, k, per_pass);
    if (!m.empty()) return fail(err, m);
    EosB200Runtime* rt = c->qz->rt;
    NcclApi* api = nccl_api();
    CUDA_TRY(cudaSetDevice(rt->device));
    cudaStream_t s = pick_stream(rt, stream);
    const int world = comm->world;
    // thresholds are seeded cooperatively (batch kernels only): slices of the queries, a multiple of 256 each
    const int slice = ((q_count + world - 1) / world + kTqTc256Queries - 1) / kTqTc256Queries * kTqTc256Queries;
    if (q_count > comm->cap_queries || k > comm->cap_k) {
        const int qcap = q_count > comm->cap_queries ? q_count : comm->cap_queries;
        const int kcap = k > comm->cap_k ? k : comm->cap_k;
        CUDA_TRY(cudaStreamSynchronize(s));
        dev_free(comm->tau_local);
        dev_free(comm->tau_all);
        dev_free(comm->keys);
        dev_free(comm->keys_all);
        comm->cap_queries = comm->cap_k = 0;
        const size_t slice_cap = (size_t)((qcap + kTqTc256Queries - 1) / kTqTc256Queries * kTqTc256Queries + kTqTc256Queries);
        CUDA_TRY(dev_alloc(&comm->tau_local, slice_cap));
        CUDA_TRY(dev_alloc(&comm->tau_all, slice_cap * world));
        CUDA_TRY(dev_alloc(&comm->keys, (size_t)qcap * kcap));
        CUDA_TRY(dev_alloc(&comm->keys_all, (size_t)qcap * kcap * world));
        comm->cap_queries = qcap;
        comm->cap_k = kcap;
    }
    int launches = 0;
    int rc = EOS_B200_OK;
    auto nccl_try = [&](int r, const char* what) {
        if (r != 0 && rc == EOS_B200_OK) rc = fail(err, std::string(what) + ": " + api->GetErrorString(r));
    };
    // an empty shard contributes empty key lists (and no thresholds)
    if (c->n == 0) CUDA_TRY(cudaMemsetAsync(comm->keys, 0, (size_t)q_count * k * sizeof(uint64_t), s));
    if (per_pass >= kTqTcQueries) {
        // every rank takes part in the threshold exchange, whatever its shard holds
        const int q_lo = std::min(q_count, comm->rank * slice);
        const int q_n = std::min(q_count, q_lo + slice) - q_lo;
        CUDA_TRY(cudaMemsetAsync(comm->tau_local, 0, (size_t)slice * sizeof(uint64_t), s));
        if (q_n > 0 && c->n > 0) {
            int seed_launches = 0;
            rc = score_seed_shared(c, d_queries + (size_t)q_lo * c->qz->dim, q_n, k, comm->tau_local, world, s, &seed_launches,
                                   err);
            if (rc != EOS_B200_OK) return rc;
            launches += seed_launches;
        }
        nccl_try(api->AllGather(comm->tau_local, comm->tau_all, (size_t)slice * sizeof(uint64_t), kNcclChar, comm->comm, s),
                 "ncclAllGather(thresholds)");
        if (rc != EOS_B200_OK) return rc;
        if (c->n > 0) {
            EosB200Stats st{};
            // tau_all is [world][slice]: query q's threshold sits at (q / slice) * slice + q % slice = q
            rc = eos_b200_score_topk_seeded_device(c, d_queries, q_count, k, comm->tau_all, nullptr, nullptr, comm->keys, s,
                                                   &st, err);
            if (rc != EOS_B200_OK) return rc;
            launches += st.kernel_launches;
        }
    } else if (c->n > 0) {
        EosB200Stats st{};
        rc = eos_b200_score_topk_device(c, d_queries, q_count, k, per_pass, nullptr, nullptr, comm->keys, s, &st, err);
        if (rc != EOS_B200_OK) return rc;
        launches += st.kernel_launches;
    }
    nccl_try(api->AllGather(comm->keys, comm->keys_all, (size_t)q_count * k * sizeof(uint64_t), kNcclChar, comm->comm, s),
             "ncclAllGather(keys)");
    if (rc != EOS_B200_OK) return rc;
    rc = eos_b200_topk_merge_device(rt, comm->keys_all, world, q_count, k, d_ids, d_scores, s, err);
    if (rc != EOS_B200_OK) return rc;
    launches += 1;
    if (stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = launches;
    }
    return EOS_B200_OK;
}

int eos_b200_maxsim_topk_device(EosB200Corpus* c, const float* d_queries, int q_vectors, int query_group,
                                int children_per_parent, int k, int64_t* d_ids, float* d_scores, uint64_t* d_keys,
                                void* stream, EosB200Stats* stats, char** err) {
    if (c == nullptr || d_queries == nullptr) return fail(err, "maxsim_topk: null argument");
    if ((d_ids == nullptr) != (d_scores == nullptr))
        return fail(err, "maxsim_topk: d_ids and d_scores must be given together or both be null");
    if (d_ids == nullptr && d_keys == nullptr) return fail(err, "maxsim_topk: no output requested");
    if (query_group < 1 || query_group > 32 || (query_group & (query_group - 1)) != 0)
        return fail(err, "maxsim_topk: query_group must be a power of two in [1, 32]");
    if (children_per_parent != 16 && children_per_parent != 32 && children_per_parent != 64 && children_per_parent != 128)
        return fail(err, "maxsim_topk: children_per_parent must be 16, 32, 64 or 128");
    if (q_vectors <= 0 || q_vectors % query_group != 0)
        return fail(err, "maxsim_topk: the number of query vectors must be a positive multiple of query_group");
    if (k <= 0 || k > kTqMaxK) return fail(err, "maxsim_topk: k must be in [1, 128]");
    if (c->n <= 0 || c->n % children_per_parent != 0 || c->id_base % children_per_parent != 0)
        return fail(err, "maxsim_topk: corpus rows and id_base must be multiples of children_per_parent");
    if (c->n + c->id_base > 0xffffffffLL || c->id_base < 0) return fail(err, "maxsim_topk: child ids must fit 32 bits");
    EosB200Runtime* rt = c->qz->rt;
    CUDA_TRY(cudaSetDevice(rt->device));
    int rc = ensure_score_workspace(c, q_vectors, err);
    if (rc == EOS_B200_OK) rc = ensure_tc_workspace(c, 0, err);
    if (rc != EOS_B200_OK) return rc;
    cudaStream_t s = pick_stream(rt, stream);
    const EosB200Corpus::TcPlan& p = c->tcp[0];
    const int q_pad = (q_vectors + p.queries - 1) / p.queries * p.queries;
    launch_tq_prepare(d_queries, q_vectors, q_pad, c->qz->spec(), nullptr, nullptr, c->qperm, s);
    CUDA_TRY(cudaMemsetAsync(c->shared_tau, 0, (size_t)q_pad * sizeof(unsigned long long), s));
    const int launches = 1 + enqueue_maxsim_passes(c, q_vectors, query_group, children_per_parent, k, d_ids, d_scores, d_keys, s);
    CUDA_TRY(cudaGetLastError());
    if (stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = launches;
    }
    return EOS_B200_OK;
}

int eos_b200_comm_merge_keys(EosB200Comm* comm, const uint64_t* d_keys, int q_count, int k, int64_t* d_ids, float* d_scores,
                             void* stream, char** err) {
    if (comm == nullptr || d_keys == nullptr || d_ids == nullptr || d_scores == nullptr)
        return fail(err, "comm_merge_keys: null argument");
    if (q_count <= 0 || k <= 0 || k > kTqMaxK) return fail(err, "comm_merge_keys: bad sizes");
    EosB200Runtime* rt = comm->rt;
    NcclApi* api = nccl_api();
    CUDA_TRY(cudaSetDevice(rt->device));
    cudaStream_t s = pick_stream(rt, stream);
    if ((size_t)q_count * k > (size_t)comm->cap_queries * comm->cap_k) {
        CUDA_TRY(cudaStreamSynchronize(s));
        dev_free(comm->keys_all);
        dev_free(comm->keys);
        dev_free(comm->tau_local);
        dev_free(comm->tau_all);
        comm->cap_queries = comm->cap_k = 0;
        const size_t slice_cap = (size_t)((q_count + kTqTc256Queries - 1) / kTqTc256Queries * kTqTc256Queries + kTqTc256Queries);
        CUDA_TRY(dev_alloc(&comm->tau_local, slice_cap));
        CUDA_TRY(dev_alloc(&comm->tau_all, slice_cap * comm->world));
        CUDA_TRY(dev_alloc(&comm->keys, (size_t)q_count * k));
        CUDA_TRY(dev_alloc(&comm->keys_all, (size_t)q_count * k * comm->world));
        comm->cap_queries = q_count;
        comm->cap_k = k;
    }
    const int r = api->AllGather(d_keys, comm->keys_all, (size_t)q_count * k * sizeof(uint64_t), kNcclChar, comm->comm, s);
    if (r != 0) return fail(err, std::string("ncclAllGather(keys): ") + api->GetErrorString(r));
    return eos_b200_topk_merge_device(rt, comm->keys_all, comm->world, q_count, k, d_ids, d_scores, s, err);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// scoring without any allocation: scratch in a file-scope device array
// ------------------------------------------------------------------------------------------------
namespace {
constexpr int kNoAllocMaxQueries = 32;
constexpr int kNoAllocMaxGrid = 160;
constexpr int kNoAllocMaxKsteps = 64;  // dim <= 1024
constexpr size_t kNoAllocBfragBytes = (size_t)(kNoAllocMaxQueries / 8) * kNoAllocMaxKsteps * 32 * sizeof(uint2);
constexpr size_t kNoAllocCandBytes = (size_t)kNoAllocMaxQueries * kNoAllocMaxGrid * kTqMaxK * sizeof(uint64_t);
constexpr size_t kNoAllocCountBytes = (size_t)kNoAllocMaxQueries * kNoAllocMaxGrid * sizeof(int);
constexpr size_t kNoAllocOffCand = (kNoAllocBfragBytes + 255) / 256 * 256;
constexpr size_t kNoAllocOffCount = kNoAllocOffCand + (kNoAllocCandBytes + 255) / 256 * 256;
constexpr size_t kNoAllocBytes = kNoAllocOffCount + (kNoAllocCountBytes + 255) / 256 * 256;

// In host code this name is only a handle for the runtime's symbol table, not an address a kernel
// could use: the device address is fetched once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_score_scratch[kNoAllocBytes];

constexpr int kNoAllocMaxDevices = 64;
std::mutex g_noalloc_mu;
unsigned char* g_noalloc_ptr[kNoAllocMaxDevices] = {};
}  // namespace

extern "C" {

int eos_b200_score_topk_noalloc(EosB200Corpus* c, const float* d_queries, int q_count, int k, int per_pass,
                                int64_t* d_ids, float* d_scores, void* stream, char** err) {
    if (c == nullptr || d_queries == nullptr || d_ids == nullptr || d_scores == nullptr)
        return fail(err, "score_topk_noalloc: null argument");
    std::string m = check_score_args(c, q_count, k, per_pass);
    if (!m.empty()) return fail(err, m);
    if (per_pass > 32) return fail(err, "score_topk_noalloc: queries_per_pass must be 8, 16 or 32");
    if (c->n == 0) return fail(err, "score_topk_noalloc: empty corpus");
    EosB200Quantizer* qz = c->qz;
    const int ksteps = tq_ksteps(qz->dim);
    if (q_count > kNoAllocMaxQueries)
        return fail(err, "score_topk_noalloc: at most 32 queries per call (got " + std::to_string(q_count) + ")");
    if (ksteps > kNoAllocMaxKsteps) return fail(err, "score_topk_noalloc: dim above 1024 is not supported");
    if (c->grid > kNoAllocMaxGrid) return fail(err, "score_topk_noalloc: more than 160 SMs are not supported");
    const int dev = qz->rt->device;
    if (dev < 0 || dev >= kNoAllocMaxDevices) return fail(err, "score_topk_noalloc: device index above 63");
    CUDA_TRY(cudaSetDevice(dev));
    unsigned char* base = nullptr;
    {
        // once per device, with that device current: the device address of the static array
        std::lock_guard<std::mutex> lock(g_noalloc_mu);
        if (g_noalloc_ptr[dev] == nullptr) {
            void* p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_score_scratch);
            if (e != cudaSuccess || p == nullptr) {
                cudaGetLastError();
                return fail(err, std::string("score_topk_noalloc: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
            }
            g_noalloc_ptr[dev] = static_cast<unsigned char*>(p);
        }
        base = g_noalloc_ptr[dev];
    }
    uint2* bfrag = reinterpret_cast<uint2*>(base);
    uint64_t* cand = reinterpret_cast<uint64_t*>(base + kNoAllocOffCand);
    int* cand_count = reinterpret_cast<int*>(base + kNoAllocOffCount);
    cudaStream_t s = pick_stream(qz->rt, stream);
    // the array still holds the previous call's lists: the counts are what a stale read would trust
    CUDA_TRY(cudaMemsetAsync(cand_count, 0, kNoAllocCountBytes, s));
    launch_tq_prepare(d_queries, q_count, kNoAllocMaxQueries, qz->spec(), bfrag, nullptr, nullptr, s);
    const int j = per_pass / 8;
    const int g_tiles = (q_count + 7) / 8;
    for (int t0 = 0; t0 < g_tiles; t0 += j) {
        TqScanArgs a{};
        a.tiles = c->tiles;
        a.norms = c->norms;
        a.n_docs = c->n;
        a.id_base = (uint32_t)c->id_base;
        a.dim = qz->dim;
        a.bfrag = bfrag + (size_t)t0 * ksteps * 32;
        a.query_tiles = j;
        a.k = k;
        a.mag_hi[0] = qz->mag_hi[0];
        a.mag_hi[1] = qz->mag_hi[1];
        a.mag_lo[0] = qz->mag_lo[0];
        a.mag_lo[1] = qz->mag_lo[1];
        a.cand_keys = cand + (size_t)t0 * 8 * c->grid * kTqMaxK;
        a.cand_count = cand_count + (size_t)t0 * 8 * c->grid;
        a.grid = c->grid;
        a.all_scores = nullptr;
        a.status = qz->rt->d_status;
        a.all_stride = 0;
        launch_tq_scan(a, s);
    }
    launch_tq_merge(cand, (int64_t)c->grid * kTqMaxK, kTqMaxK, c->grid, kTqMaxK, cand_count, q_count, k, 0, d_ids,
                    d_scores, nullptr, s);
    CUDA_TRY(cudaGetLastError());
    return EOS_B200_OK;
}

int eos_b200_topk_merge_device(EosB200Runtime* rt, const uint64_t* d_keys, int shards, int q_count, int k,
                               int64_t* d_ids, float* d_scores, void* stream, char** err) {
    if (rt == nullptr || d_keys == nullptr || d_ids == nullptr || d_scores == nullptr)
        return fail(err, "topk_merge: null argument");
    if (shards <= 0 || q_count <= 0 || k <= 0 || k > kTqMaxK) return fail(err, "topk_merge: bad sizes");
    CUDA_TRY(cudaSetDevice(rt->device));
    // gathered layout [shards][q_count][k]: a query's segments are q_count*k keys apart
    launch_tq_merge(d_keys, (int64_t)k, (int64_t)q_count * k, shards, k, nullptr, q_count, k, 0, d_ids, d_scores,
                    nullptr, pick_stream(rt, stream));
    CUDA_TRY(cudaGetLastError());
    return EOS_B200_OK;
}

int eos_b200_score_all(EosB200Corpus* c, const float* h_queries, int q_count, float* h_scores, char** err) {
    if (c == nullptr || h_queries == nullptr || h_scores == nullptr) return fail(err, "score_all: null argument");
    if (q_count <= 0 || c->n <= 0) return fail(err, "score_all: empty input");
    EosB200Runtime* rt = c->qz->rt;
    CUDA_TRY(cudaSetDevice(rt->device));
    int rc = ensure_score_workspace(c, q_count, err);
    if (rc != EOS_B200_OK) return rc;
    const int q_pad = (q_count + 7) / 8 * 8;
    float* d_all = nullptr;
    CUDA_TRY(dev_alloc(&d_all, (size_t)q_pad * c->n));
    cudaStream_t s = rt->stream;
    cudaError_t e = cudaMemsetAsync(rt->d_status, 0, sizeof(int), s);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(c->d_queries, h_queries, (size_t)q_count * c->qz->dim * 4, cudaMemcpyHostToDevice, s);
    launch_tq_prepare(c->d_queries, q_count, q_pad, c->qz->spec(), c->bfrag, nullptr, nullptr, s);
    const int ksteps = tq_ksteps(c->qz->dim);
    for (int t = 0; t < q_pad / 8; ++t) {
        TqScanArgs a{};
        a.tiles = c->tiles;
        a.norms = c->norms;
        a.n_docs = c->n;
        a.id_base = 0;
        a.dim = c->qz->dim;
        a.bfrag = c->bfrag + (size_t)t * ksteps * 32;
        a.query_tiles = 1;
        a.k = 1;
        a.mag_hi[0] = c->qz->mag_hi[0];
        a.mag_hi[1] = c->qz->mag_hi[1];
        a.mag_lo[0] = c->qz->mag_lo[0];
        a.mag_lo[1] = c->qz->mag_lo[1];
        a.cand_keys = c->cand;
        a.cand_count = c->cand_count;
        a.grid = c->grid;
        a.all_scores = d_all + (size_t)t * 8 * c->n;
        a.all_stride = c->n;
        a.status = rt->d_status;
        launch_tq_scan(a, s);
    }
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_scores, d_all, (size_t)q_count * c->n * 4, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    dev_free(d_all);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(err, std::string("score_all: ") + cudaGetErrorString(e));
    }
    return read_status(rt, s, err);
}

int eos_b200_parent_topk(EosB200Corpus* c, const int32_t* h_parent_of_child, int parents, const float* h_queries,
                         int q_count, int query_group, int top_n, double penalty, int k, int64_t* h_ids,
                         float* h_scores, EosB200Stats* stats, char** err) {
    if (c == nullptr || h_parent_of_child == nullptr || h_queries == nullptr || h_ids == nullptr || h_scores == nullptr)
        return fail(err, "parent_topk: null argument");
    if (c->n <= 0 || parents <= 0 || q_count <= 0) return fail(err, "parent_topk: empty input");
    if (k <= 0 || k > kTqMaxK) return fail(err, "parent_topk: k must be in [1, 128]");
    if (query_group < 1 || query_group > 32 || (query_group & (query_group - 1)) != 0)
        return fail(err, "parent_topk: query_group must be a power of two in [1, 32]");
    if (q_count % query_group != 0) return fail(err, "parent_topk: q_count must be a multiple of query_group");
    if (c->n > 0x7fffffffLL) return fail(err, "parent_topk: too many child vectors");
    EosB200Runtime* rt = c->qz->rt;
    CUDA_TRY(cudaSetDevice(rt->device));
    const int n = (int)c->n;
    // children grouped by parent (counting sort keeps child order inside a parent)
    std::vector<int> offsets((size_t)parents + 1, 0), order((size_t)n);
    for (int i = 0; i < n; ++i) {
        const int p = h_parent_of_child[i];
        if (p < 0 || p >= parents) return fail(err, "parent_topk: parent index out of range");
        offsets[(size_t)p + 1]++;
    }
    for (int p = 0; p < parents; ++p) offsets[(size_t)p + 1] += offsets[p];
    {
        std::vector<int> cursor(offsets.begin(), offsets.end() - 1);
        for (int i = 0; i < n; ++i) order[(size_t)cursor[h_parent_of_child[i]]++] = i;
    }
    int rc = ensure_score_workspace(c, q_count, err);
    if (rc != EOS_B200_OK) return rc;
    const int groups = q_count / query_group;
    int *d_order = nullptr, *d_offsets = nullptr;
    float *d_all = nullptr, *d_agg = nullptr, *d_sc = nullptr;
    uint64_t* d_keys = nullptr;
    int64_t* d_ids = nullptr;
    cudaStream_t s = rt->stream;
    cudaError_t e = dev_alloc(&d_order, (size_t)n);
    if (e == cudaSuccess) e = cudaMemsetAsync(rt->d_status, 0, sizeof(int), s);
    if (e == cudaSuccess) e = dev_alloc(&d_offsets, (size_t)parents + 1);
    if (e == cudaSuccess) e = dev_alloc(&d_all, (size_t)32 * n);
    if (e == cudaSuccess) e = dev_alloc(&d_agg, (size_t)query_group * parents);
    if (e == cudaSuccess) e = dev_alloc(&d_keys, (size_t)groups * parents);
    if (e == cudaSuccess) e = dev_alloc(&d_ids, (size_t)groups * k);
    if (e == cudaSuccess) e = dev_alloc(&d_sc, (size_t)groups * k);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_order, order.data(), (size_t)n * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(d_offsets, offsets.data(), ((size_t)parents + 1) * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev0, s);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(c->d_queries, h_queries, (size_t)q_count * c->qz->dim * 4, cudaMemcpyHostToDevice, s);
    int launches = 0;
    if (e == cudaSuccess) {
        const int q_pad = (q_count + 31) / 32 * 32;
        launch_tq_prepare(c->d_queries, q_count, q_pad, c->qz->spec(), c->bfrag, nullptr, nullptr, s);
        launches++;
        const int ksteps = tq_ksteps(c->qz->dim);
        for (int r0 = 0; r0 < q_count; r0 += 32) {
            TqScanArgs a{};
            a.tiles = c->tiles;
            a.norms = c->norms;
            a.n_docs = c->n;
            a.id_base = 0;
            a.dim = c->qz->dim;
            a.bfrag = c->bfrag + (size_t)(r0 / 8) * ksteps * 32;
            a.query_tiles = 4;
            a.k = 1;
            a.mag_hi[0] = c->qz->mag_hi[0];
            a.mag_hi[1] = c->qz->mag_hi[1];
            a.mag_lo[0] = c->qz->mag_lo[0];
            a.mag_lo[1] = c->qz->mag_lo[1];
            a.cand_keys = c->cand;
            a.cand_count = c->cand_count;
            a.grid = c->grid;
            a.all_scores = d_all;
            a.all_stride = n;
            a.status = rt->d_status;
            launch_tq_scan(a, s);
            launches++;
            const int rows_here = (q_count - r0) < 32 ? (q_count - r0) : 32;
            for (int r = 0; r < rows_here; r += query_group) {
                launch_parent_keys(d_all + (size_t)r * n, n, query_group, d_order, d_offsets, parents, top_n, penalty,
                                   d_agg, d_keys + (size_t)((r0 + r) / query_group) * parents, s);
                launches += 2;
            }
        }
        launch_tq_merge(d_keys, (int64_t)parents, (int64_t)parents, 1, parents, nullptr, groups, k, 0, d_ids, d_sc,
                        nullptr, s);
        launches++;
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_ids, d_ids, (size_t)groups * k * 8, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_scores, d_sc, (size_t)groups * k * 4, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev1, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e == cudaSuccess && stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = launches;
        stats->uploaded_bytes = (int64_t)q_count * c->qz->dim * 4;
        stats->downloaded_bytes = (int64_t)groups * k * 12;
        cudaEventElapsedTime(&stats->device_ms, rt->ev0, rt->ev1);
    }
    dev_free(d_order);
    dev_free(d_offsets);
    dev_free(d_all);
    dev_free(d_agg);
    dev_free(d_keys);
    dev_free(d_ids);
    dev_free(d_sc);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(err, std::string("parent_topk: ") + cudaGetErrorString(e));
    }
    return read_status(rt, s, err);
}

int eos_b200_synth_gaussian_device(EosB200Runtime* rt, uint64_t seed, int64_t row_offset, int64_t n, int dim,
                                   int normalize, float* d_out, void* stream, char** err) {
    if (rt == nullptr || d_out == nullptr) return fail(err, "synth_gaussian: null argument");
    if (n <= 0 || dim <= 0) return fail(err, "synth_gaussian: sizes must be positive");
    CUDA_TRY(cudaSetDevice(rt->device));
    synth_gaussian_kernel<<<rt->sm_count * 8, 256, 0, pick_stream(rt, stream)>>>(
        (unsigned long long)seed, (long long)row_offset, (long long)n, dim, normalize ? 1 : 0, d_out);
    CUDA_TRY(cudaGetLastError());
    return EOS_B200_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// dense candidates
// ------------------------------------------------------------------------------------------------
struct EosB200DenseIndex {
    EosB200Runtime* rt = nullptr;
    int64_t n = 0;
    int dim = 0;
    bool f16 = false;
    void* vectors = nullptr;  // [n, dim] fp32 or f16
};

namespace {
__global__ void f32_to_f16_kernel(const float* __restrict__ in, long long count, __half* __restrict__ out) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride)
        out[i] = __float2half_rn(in[i]);
}

// shared tail of the two dense entry points: keys [q, cand] -> top-k on the host buffers
int dense_finish(EosB200DenseIndex* ix, uint64_t* d_keys, int q_count, int64_t cand, int k, int launches,
                 int64_t uploaded, int64_t* h_ids, float* h_scores, EosB200Stats* stats, const char* what, char** err) {
    EosB200Runtime* rt = ix->rt;
    cudaStream_t s = rt->stream;
    int64_t* d_ids = nullptr;
    float* d_scores = nullptr;
    cudaError_t e = dev_alloc(&d_ids, (size_t)q_count * k);
    if (e == cudaSuccess) e = dev_alloc(&d_scores, (size_t)q_count * k);
    if (e == cudaSuccess) {
        launch_tq_merge(d_keys, cand, cand, 1, (int)cand, nullptr, q_count, k, 0, d_ids, d_scores, nullptr, s);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_ids, d_ids, (size_t)q_count * k * 8, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_scores, d_scores, (size_t)q_count * k * 4, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev1, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    dev_free(d_ids);
    dev_free(d_scores);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(err, std::string(what) + ": " + cudaGetErrorString(e));
    }
    if (stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = launches + 1;
        stats->uploaded_bytes = uploaded;
        stats->downloaded_bytes = (int64_t)q_count * k * 12;
        cudaEventElapsedTime(&stats->device_ms, rt->ev0, rt->ev1);
    }
    return EOS_B200_OK;
}
}  // namespace

extern "C" {

int eos_b200_dense_bind(EosB200Runtime* rt, const float* h_vectors, int64_t n, int dim, int store_f16,
                        EosB200DenseIndex** out, char** err) {
    if (rt == nullptr || h_vectors == nullptr || out == nullptr) return fail(err, "dense_bind: null argument");
    if (n <= 0 || dim <= 0) return fail(err, "dense_bind: empty input");
    if (dim > 1024) return fail(err, "dense_bind: dim must be at most 1024");
    if (n > 0x7fffffffLL) return fail(err, "dense_bind: too many rows");
    CUDA_TRY(cudaSetDevice(rt->device));
    auto* ix = new EosB200DenseIndex();
    ix->rt = rt;
    ix->n = n;
    ix->dim = dim;
    ix->f16 = store_f16 != 0;
    const size_t count = (size_t)n * dim;
    float* d_f32 = nullptr;
    cudaError_t e = dev_alloc(&d_f32, count);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_f32, h_vectors, count * 4, cudaMemcpyHostToDevice, rt->stream);
    if (e == cudaSuccess && ix->f16) {
        __half* d_f16 = nullptr;
        e = dev_alloc(&d_f16, count);
        if (e == cudaSuccess) {
            f32_to_f16_kernel<<<rt->sm_count * 8, 256, 0, rt->stream>>>(d_f32, (long long)count, d_f16);
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = cudaStreamSynchronize(rt->stream);
        dev_free(d_f32);
        d_f32 = nullptr;
        ix->vectors = d_f16;
    } else {
        if (e == cudaSuccess) e = cudaStreamSynchronize(rt->stream);
        ix->vectors = d_f32;
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        dev_free(ix->vectors);
        delete ix;
        return fail(err, std::string("dense_bind: ") + cudaGetErrorString(e));
    }
    *out = ix;
    return EOS_B200_OK;
}

void eos_b200_dense_destroy(EosB200DenseIndex* ix) {
    if (ix == nullptr) return;
    cudaSetDevice(ix->rt->device);
    dev_free(ix->vectors);
    delete ix;
}

int eos_b200_dense_score_topk(EosB200DenseIndex* ix, const float* h_queries, int q_count, int metric, int k,
                              int64_t* h_ids, float* h_scores, EosB200Stats* stats, char** err) {
    if (ix == nullptr || h_queries == nullptr || h_ids == nullptr || h_scores == nullptr)
        return fail(err, "dense_score_topk: null argument");
    if (q_count <= 0) return fail(err, "dense_score_topk: empty input");
    if (metric != EOS_B200_METRIC_DOT && metric != EOS_B200_METRIC_COSINE) return fail(err, "dense_score_topk: unknown metric");
    if (k <= 0 || k > kTqWideK || k > ix->n) return fail(err, "dense_score_topk: k must be in [1, min(256, rows)]");
    EosB200Runtime* rt = ix->rt;
    CUDA_TRY(cudaSetDevice(rt->device));
    cudaStream_t s = rt->stream;
    float* d_q = nullptr;
    uint64_t* d_keys = nullptr;
    cudaError_t e = dev_alloc(&d_q, (size_t)q_count * ix->dim);
    if (e == cudaSuccess) e = dev_alloc(&d_keys, (size_t)q_count * ix->n);
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev0, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_q, h_queries, (size_t)q_count * ix->dim * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) {
        launch_dense_keys(ix->vectors, ix->f16, ix->n, ix->dim, d_q, q_count, nullptr, ix->n, metric, d_keys, rt->sm_count, s);
        e = cudaGetLastError();
    }
    int rc = EOS_B200_OK;
    if (e != cudaSuccess) {
        cudaGetLastError();
        rc = fail(err, std::string("dense_score_topk: ") + cudaGetErrorString(e));
    } else {
        rc = dense_finish(ix, d_keys, q_count, ix->n, k, 1, (int64_t)q_count * ix->dim * 4, h_ids, h_scores, stats,
                          "dense_score_topk", err);
    }
    dev_free(d_q);
    dev_free(d_keys);
    return rc;
}

int eos_b200_dense_rerank(EosB200DenseIndex* ix, const float* h_queries, int q_count, const int64_t* h_candidates,
                          int cand, int k, int64_t* h_ids, float* h_scores, EosB200Stats* stats, char** err) {
    if (ix == nullptr || h_queries == nullptr || h_candidates == nullptr || h_ids == nullptr || h_scores == nullptr)
        return fail(err, "dense_rerank: null argument");
    if (q_count <= 0 || cand <= 0) return fail(err, "dense_rerank: empty input");
    if (k <= 0 || k > cand) k = cand;  // the reference clamps topK to the candidate count
    if (k > kTqWideK) return fail(err, "dense_rerank: k must be at most 256");
    EosB200Runtime* rt = ix->rt;
    CUDA_TRY(cudaSetDevice(rt->device));
    cudaStream_t s = rt->stream;
    float* d_q = nullptr;
    int64_t* d_cand = nullptr;
    uint64_t* d_keys = nullptr;
    cudaError_t e = dev_alloc(&d_q, (size_t)q_count * ix->dim);
    if (e == cudaSuccess) e = dev_alloc(&d_cand, (size_t)q_count * cand);
    if (e == cudaSuccess) e = dev_alloc(&d_keys, (size_t)q_count * cand);
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev0, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_q, h_queries, (size_t)q_count * ix->dim * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_cand, h_candidates, (size_t)q_count * cand * 8, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) {
        launch_dense_keys(ix->vectors, ix->f16, ix->n, ix->dim, d_q, q_count, d_cand, cand, EOS_B200_METRIC_DOT, d_keys,
                          rt->sm_count, s);
        e = cudaGetLastError();
    }
    int rc = EOS_B200_OK;
    if (e != cudaSuccess) {
        cudaGetLastError();
        rc = fail(err, std::string("dense_rerank: ") + cudaGetErrorString(e));
    } else {
        rc = dense_finish(ix, d_keys, q_count, cand, k, 1, (int64_t)q_count * (ix->dim * 4 + (int64_t)cand * 8), h_ids,
                          h_scores, stats, "dense_rerank", err);
    }
    dev_free(d_q);
    dev_free(d_cand);
    dev_free(d_keys);
    return rc;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// sparse attention
// ------------------------------------------------------------------------------------------------
namespace {
// sparseAttentionBudget / normalizeSparseAttentionRoute, runtime/backend/attention_ops.go:445-460, 503-516
int sparse_budget(int top_k, int key_len) {
    if (key_len <= 0) return 0;
    int budget = top_k;
    if (budget <= 0) budget = (int)std::ceil(std::sqrt((double)key_len));
    if (budget < 1) budget = 1;
    if (budget > key_len) budget = key_len;
    return budget;
}
void sparse_route(int key_len, int block_size, int top_blocks, int* bs, int* tb) {
    *bs = *tb = 0;
    if (key_len <= 0 || block_size <= 0 || top_blocks <= 0) return;
    if (block_size > key_len) block_size = key_len;
    const int block_count = (key_len + block_size - 1) / block_size;
    if (top_blocks > block_count) top_blocks = block_count;
    *bs = block_size;
    *tb = top_blocks;
}

std::string sparse_check(int batches, int q_len, int k_len, int dim, int vdim, int top_k, int rbs, int rtb, int* budget,
                         int* bs, int* tb) {
    if (batches <= 0 || q_len <= 0 || dim <= 0 || vdim <= 0 || k_len < 0) return "sparse_attention: sizes must be positive";
    if (dim > 4096) return "sparse_attention: query dim above 4096 is not supported";
    *budget = sparse_budget(top_k, k_len);
    sparse_route(k_len, rbs, rtb, bs, tb);
    if (*budget > kSaMaxBudget) return "sparse_attention: top_k above 128 is not supported";
    if (*tb > kSaMaxBudget) return "sparse_attention: route_top_blocks above 128 is not supported";
    return "";
}
}  // namespace

extern "C" {

int eos_b200_sparse_attention(EosB200Runtime* rt, const float* h_query, const float* h_key, const float* h_value, int batches,
                              int q_len, int k_len, int dim, int value_dim, int top_k, int route_block_size,
                              int route_top_blocks, float* h_out, EosB200Stats* stats, char** err) {
    if (rt == nullptr || h_query == nullptr || h_out == nullptr || (k_len > 0 && (h_key == nullptr || h_value == nullptr)))
        return fail(err, "sparse_attention expects query, key, and value");
    int budget = 0, bs = 0, tb = 0;
    std::string m = sparse_check(batches, q_len, k_len, dim, value_dim, top_k, route_block_size, route_top_blocks, &budget,
                                 &bs, &tb);
    if (!m.empty()) return fail(err, m);
    const size_t nq = (size_t)batches * q_len * dim, nk = (size_t)batches * k_len * dim, nv = (size_t)batches * k_len * value_dim;
    const size_t no = (size_t)batches * q_len * value_dim;
    if (k_len == 0) {
        std::memset(h_out, 0, no * sizeof(float));
        if (stats != nullptr) std::memset(stats, 0, sizeof(*stats));
        return EOS_B200_OK;
    }
    CUDA_TRY(cudaSetDevice(rt->device));
    float *dq = nullptr, *dk = nullptr, *dv = nullptr, *dout = nullptr;
    cudaStream_t s = rt->stream;
    cudaError_t e = dev_alloc(&dq, nq);
    if (e == cudaSuccess) e = dev_alloc(&dk, nk);
    if (e == cudaSuccess) e = dev_alloc(&dv, nv);
    if (e == cudaSuccess) e = dev_alloc(&dout, no);
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev0, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dq, h_query, nq * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dk, h_key, nk * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dv, h_value, nv * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) {
        launch_sparse_attention(dq, dk, dv, batches, q_len, k_len, dim, value_dim, budget, bs, tb, dout, rt->sm_count, s);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_out, dout, no * 4, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev1, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e == cudaSuccess && stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = 1;
        stats->uploaded_bytes = (int64_t)(nq + nk + nv) * 4;
        stats->downloaded_bytes = (int64_t)no * 4;
        cudaEventElapsedTime(&stats->device_ms, rt->ev0, rt->ev1);
    }
    dev_free(dq);
    dev_free(dk);
    dev_free(dv);
    dev_free(dout);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(err, std::string("sparse_attention: ") + cudaGetErrorString(e));
    }
    return EOS_B200_OK;
}

int eos_b200_turbo_sparse_attention(EosB200Quantizer* key_qz, EosB200Quantizer* value_qz, const float* h_query,
                                    const uint8_t* h_key_codes, const uint8_t* h_key_norm_codes,
                                    const uint8_t* h_value_codes, const uint8_t* h_value_norm_codes, int batches, int q_len,
                                    int k_len, int top_k, int route_block_size, int route_top_blocks, float* h_out,
                                    EosB200Stats* stats, char** err) {
    if (key_qz == nullptr || value_qz == nullptr || h_query == nullptr || h_out == nullptr)
        return fail(err, "turbo_sparse_attention expects query");
    if (k_len > 0 && (h_key_codes == nullptr || h_key_norm_codes == nullptr || h_value_codes == nullptr ||
                      h_value_norm_codes == nullptr))
        return fail(err, "turbo_sparse_attention: missing compressed key / value tensors");
    if (key_qz->rt != value_qz->rt) return fail(err, "turbo_sparse_attention: quantizers belong to different runtimes");
    EosB200Runtime* rt = key_qz->rt;
    const int dim = key_qz->dim, vdim = value_qz->dim;
    int budget = 0, bs = 0, tb = 0;
    std::string m = sparse_check(batches, q_len, k_len, dim, vdim, top_k, route_block_size, route_top_blocks, &budget, &bs, &tb);
    if (!m.empty()) return fail(err, m);
    const size_t nq = (size_t)batches * q_len * dim, rows = (size_t)batches * k_len;
    const size_t no = (size_t)batches * q_len * vdim;
    if (k_len == 0) {
        std::memset(h_out, 0, no * sizeof(float));
        if (stats != nullptr) std::memset(stats, 0, sizeof(*stats));
        return EOS_B200_OK;
    }
    CUDA_TRY(cudaSetDevice(rt->device));
    float *dq = nullptr, *dk = nullptr, *dv = nullptr, *dout = nullptr;
    uint8_t *ck = nullptr, *cv = nullptr, *nk = nullptr, *nv = nullptr;
    cudaStream_t s = rt->stream;
    cudaError_t e = dev_alloc(&dq, nq);
    if (e == cudaSuccess) e = dev_alloc(&dk, rows * dim);
    if (e == cudaSuccess) e = dev_alloc(&dv, rows * vdim);
    if (e == cudaSuccess) e = dev_alloc(&dout, no);
    if (e == cudaSuccess) e = dev_alloc(&ck, rows * dim);
    if (e == cudaSuccess) e = dev_alloc(&cv, rows * vdim);
    if (e == cudaSuccess) e = dev_alloc(&nk, rows);
    if (e == cudaSuccess) e = dev_alloc(&nv, rows);
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev0, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dq, h_query, nq * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(ck, h_key_codes, rows * dim, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(cv, h_value_codes, rows * vdim, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(nk, h_key_norm_codes, rows, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(nv, h_value_norm_codes, rows, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) {
        // the compressed K / V are decoded on the device (the reference decodes them on the host), then attended to
        launch_tq_decode_rows(ck, nk, (int64_t)rows, key_qz->spec(), dk, rt->sm_count, s);
        launch_tq_decode_rows(cv, nv, (int64_t)rows, value_qz->spec(), dv, rt->sm_count, s);
        launch_sparse_attention(dq, dk, dv, batches, q_len, k_len, dim, vdim, budget, bs, tb, dout, rt->sm_count, s);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_out, dout, no * 4, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev1, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e == cudaSuccess && stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = 3;
        stats->uploaded_bytes = (int64_t)nq * 4 + (int64_t)rows * (dim + vdim + 2);
        stats->downloaded_bytes = (int64_t)no * 4;
        cudaEventElapsedTime(&stats->device_ms, rt->ev0, rt->ev1);
    }
    dev_free(dq);
    dev_free(dk);
    dev_free(dv);
    dev_free(dout);
    dev_free(ck);
    dev_free(cv);
    dev_free(nk);
    dev_free(nv);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(err, std::string("turbo_sparse_attention: ") + cudaGetErrorString(e));
    }
    return EOS_B200_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// token-pool encoder: fp32 single-head layers -> per-token rows -> span-pooled child vectors
// ------------------------------------------------------------------------------------------------
struct EosB200TokenPool {
    EosB200Runtime* rt = nullptr;
    EosB200TokenPoolDesc d{};
    float *table = nullptr, *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr, *w1 = nullptr, *w2 = nullptr;
};

namespace {
// sparseTokenPoolTokenSpans, runtime/sparse_token_pool_vector_export.go:1561-1595
void token_spans(int token_count, int span_tokens, int overlap, int min_tokens, std::vector<int>* starts,
                 std::vector<int>* ends) {
    starts->clear();
    ends->clear();
    if (token_count <= 0 || span_tokens <= 0) return;
    if (min_tokens <= 0) min_tokens = 1;
    if (token_count <= span_tokens) {
        if (token_count < min_tokens) return;
        starts->push_back(0);
        ends->push_back(token_count);
        return;
    }
    const int step = span_tokens - overlap;
    if (step <= 0) return;
    for (int start = 0; start < token_count; start += step) {
        int end = start + span_tokens;
        if (end > token_count) end = token_count;
        if (end - start < min_tokens) break;
        starts->push_back(start);
        ends->push_back(end);
        if (end >= token_count) break;
    }
}
}  // namespace

extern "C" {

void eos_b200_token_pool_destroy(EosB200TokenPool* tp) {
    if (tp == nullptr) return;
    cudaSetDevice(tp->rt->device);
    dev_free(tp->table);
    dev_free(tp->wq);
    dev_free(tp->wk);
    dev_free(tp->wv);
    dev_free(tp->wo);
    dev_free(tp->w1);
    dev_free(tp->w2);
    delete tp;
}

int eos_b200_token_pool_bind(EosB200Runtime* rt, const EosB200TokenPoolDesc* desc, EosB200TokenPool** out, char** err) {
    if (rt == nullptr || desc == nullptr || out == nullptr) return fail(err, "token_pool_bind: null argument");
    *out = nullptr;
    const EosB200TokenPoolDesc& d = *desc;
    if (d.vocab <= 0 || d.dim <= 0 || d.hidden <= 0 || d.encoder_repeats < 0)
        return fail(err, "token_pool_bind: sizes must be positive");
    if (d.token_embedding == nullptr || d.attention_query == nullptr || d.attention_key == nullptr ||
        d.attention_value == nullptr || d.attention_output == nullptr || d.hidden_projection == nullptr ||
        d.projection == nullptr)
        return fail(err, "token_pool_bind: the full encoder needs all seven weight tensors");
    CUDA_TRY(cudaSetDevice(rt->device));
    auto* tp = new EosB200TokenPool();
    tp->rt = rt;
    tp->d = d;
    const size_t dd = (size_t)d.dim * d.dim, dh = (size_t)d.dim * d.hidden;
    std::string msg = upload_f32(d.token_embedding, (size_t)d.vocab * d.dim, &tp->table);
    if (msg.empty()) msg = upload_f32(d.attention_query, dd, &tp->wq);
    if (msg.empty()) msg = upload_f32(d.attention_key, dd, &tp->wk);
    if (msg.empty()) msg = upload_f32(d.attention_value, dd, &tp->wv);
    if (msg.empty()) msg = upload_f32(d.attention_output, dd, &tp->wo);
    if (msg.empty()) msg = upload_f32(d.hidden_projection, dh, &tp->w1);
    if (msg.empty()) msg = upload_f32(d.projection, dh, &tp->w2);
    tp->d.token_embedding = tp->d.attention_query = tp->d.attention_key = tp->d.attention_value = nullptr;
    tp->d.attention_output = tp->d.hidden_projection = tp->d.projection = nullptr;
    if (!msg.empty()) {
        eos_b200_token_pool_destroy(tp);
        return fail(err, "token_pool_bind: " + msg);
    }
    *out = tp;
    return EOS_B200_OK;
}

int eos_b200_token_pool_encode(EosB200TokenPool* tp, const int32_t* h_tokens, const int32_t* h_mask, int seq_len,
                               int attention_mode, EosB200Quantizer* key_qz, EosB200Quantizer* value_qz, int top_k,
                               int route_block_size, int route_top_blocks, int span_tokens, int span_overlap,
                               int span_min_tokens, float* h_rows, float* h_pooled, float* h_children, int max_children,
                               int* n_children, EosB200Stats* stats, char** err) {
    if (tp == nullptr || h_tokens == nullptr) return fail(err, "token_pool_encode: null argument");
    if (seq_len <= 0) return fail(err, "token_pool_encode: empty sequence");
    if (attention_mode != EOS_B200_TOKEN_POOL_DENSE && attention_mode != EOS_B200_TOKEN_POOL_TURBO_SPARSE)
        return fail(err, "token_pool_encode: unsupported attention mode");
    if ((h_pooled != nullptr || h_children != nullptr) && h_mask == nullptr)
        return fail(err, "token_pool_encode: pooling needs the attention mask");
    if (h_children != nullptr && n_children == nullptr) return fail(err, "token_pool_encode: n_children is required");
    EosB200Runtime* rt = tp->rt;
    const int D = tp->d.dim, H = tp->d.hidden, T = seq_len;
    int budget = 0, bs = 0, tb = 0;
    if (attention_mode == EOS_B200_TOKEN_POOL_TURBO_SPARSE) {
        if (key_qz == nullptr || value_qz == nullptr || key_qz->dim != D || value_qz->dim != D || key_qz->rt != rt ||
            value_qz->rt != rt)
            return fail(err, "token_pool_encode: the turbo-sparse mode needs key and value quantizers of the model width");
        std::string m = sparse_check(1, T, T, D, D, top_k, route_block_size, route_top_blocks, &budget, &bs, &tb);
        if (!m.empty()) return fail(err, m);
    }
    std::vector<int> starts, ends;
    if (h_children != nullptr) {
        token_spans(T, span_tokens, span_overlap, span_min_tokens, &starts, &ends);
        if (starts.empty()) return fail(err, "token_pool_encode: token-span mode selected no spans");
        if ((int)starts.size() > max_children) return fail(err, "token_pool_encode: more spans than max_children");
    }
    CUDA_TRY(cudaSetDevice(rt->device));
    cudaStream_t s = rt->stream;
    const size_t td = (size_t)T * D;
    int32_t *d_tok = nullptr, *d_mask = nullptr;
    float *cur = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *hid = nullptr, *ffn = nullptr, *tmp = nullptr;
    float *scores = nullptr, *pooled = nullptr, *children = nullptr;
    uint8_t *kc = nullptr, *vc = nullptr, *ku = nullptr, *vu = nullptr, *kn = nullptr, *vn = nullptr;
    float *knf = nullptr, *vnf = nullptr;
    int *d_spans = nullptr, *d_flags = nullptr;
    const bool turbo = attention_mode == EOS_B200_TOKEN_POOL_TURBO_SPARSE;
    const int n_spans = (int)starts.size();
    cudaError_t e = dev_alloc(&d_tok, (size_t)T);
    if (e == cudaSuccess) e = dev_alloc(&d_mask, (size_t)T);
    for (float** p : {&cur, &q, &k, &v, &att, &hid, &tmp})
        if (e == cudaSuccess) e = dev_alloc(p, td);
    if (e == cudaSuccess) e = dev_alloc(&ffn, (size_t)T * H);
    if (e == cudaSuccess && !turbo) e = dev_alloc(&scores, (size_t)T * T);
    if (e == cudaSuccess) e = dev_alloc(&pooled, (size_t)D);
    if (e == cudaSuccess) e = dev_alloc(&children, (size_t)(n_spans > 0 ? n_spans : 1) * D);
    if (e == cudaSuccess) e = dev_alloc(&d_spans, (size_t)2 * (n_spans + 1));
    if (e == cudaSuccess) e = dev_alloc(&d_flags, (size_t)(n_spans + 1));
    size_t kcb = 0, vcb = 0;
    if (turbo) {
        kcb = ((size_t)D * key_qz->bits + 7) / 8;
        vcb = ((size_t)D * value_qz->bits + 7) / 8;
        if (e == cudaSuccess) e = dev_alloc(&kc, (size_t)T * kcb);
        if (e == cudaSuccess) e = dev_alloc(&vc, (size_t)T * vcb);
        if (e == cudaSuccess) e = dev_alloc(&ku, td);
        if (e == cudaSuccess) e = dev_alloc(&vu, td);
        if (e == cudaSuccess) e = dev_alloc(&kn, (size_t)T);
        if (e == cudaSuccess) e = dev_alloc(&vn, (size_t)T);
        if (e == cudaSuccess) e = dev_alloc(&knf, (size_t)T);
        if (e == cudaSuccess) e = dev_alloc(&vnf, (size_t)T);
    }
    int launches = 0;
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev0, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_tok, h_tokens, (size_t)T * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess && h_mask != nullptr) e = cudaMemcpyAsync(d_mask, h_mask, (size_t)T * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) {
        launch_tp_gather(tp->table, tp->d.vocab, D, d_tok, T, cur, s);
        ++launches;
    }
    std::vector<float> h_norms((size_t)T);
    std::vector<uint8_t> h_codes((size_t)T);
    for (int layer = 0; layer < tp->d.encoder_repeats && e == cudaSuccess; ++layer) {
        launch_tp_matmul(cur, T, D, tp->wq, D, 0, q, s);
        launch_tp_matmul(cur, T, D, tp->wk, D, 0, k, s);
        launch_tp_matmul(cur, T, D, tp->wv, D, 0, v, s);
        launches += 3;
        if (!turbo) {
            launch_tp_dense_attention(q, k, v, T, D, scores, att, rt->sm_count, s);
            ++launches;
        } else {
            // TurboQuantEncodeReference on the key and value rows (codes + 8-bit log norm), then the compressed
            // sparse attention; the norm codes are formed on the host so that they are the host library's logf
            launch_tq_pack(k, T, key_qz->spec(), kc, knf, s);
            launch_tq_pack(v, T, value_qz->spec(), vc, vnf, s);
            launches += 4;
            for (int side = 0; side < 2 && e == cudaSuccess; ++side) {
                e = cudaMemcpyAsync(h_norms.data(), side == 0 ? knf : vnf, (size_t)T * 4, cudaMemcpyDeviceToHost, s);
                if (e == cudaSuccess) e = cudaStreamSynchronize(s);
                if (e != cudaSuccess) break;
                eos_b200_norm_encode_log8(h_norms.data(), T, h_codes.data());
                e = cudaMemcpyAsync(side == 0 ? kn : vn, h_codes.data(), (size_t)T, cudaMemcpyHostToDevice, s);
                if (e == cudaSuccess) e = cudaStreamSynchronize(s);
            }
            if (e != cudaSuccess) break;
            launch_tp_unpack_codes(kc, T, D, key_qz->bits, ku, s);
            launch_tp_unpack_codes(vc, T, D, value_qz->bits, vu, s);
            launch_tq_decode_rows(ku, kn, T, key_qz->spec(), k, rt->sm_count, s);
            launch_tq_decode_rows(vu, vn, T, value_qz->spec(), v, rt->sm_count, s);
            launch_sparse_attention(q, k, v, 1, T, T, D, D, budget, bs, tb, att, rt->sm_count, s);
            launches += 5;
        }
        launch_tp_matmul(att, T, D, tp->wo, D, 0, hid, s);
        ++launches;
        if (tp->d.attention_residual) {
            launch_tp_add(hid, cur, (long long)td, hid, s);
            ++launches;
        }
        if (tp->d.attention_layer_norm) {
            launch_tp_layernorm(hid, T, D, tmp, s);
            std::swap(hid, tmp);
            ++launches;
        }
        launch_tp_matmul(hid, T, D, tp->w1, H, 1, ffn, s);
        launch_tp_matmul(ffn, T, H, tp->w2, D, 0, tmp, s);
        launches += 2;
        if (tp->d.ffn_residual) {
            launch_tp_add(tmp, hid, (long long)td, tmp, s);
            ++launches;
        }
        if (tp->d.ffn_layer_norm) {
            launch_tp_layernorm(tmp, T, D, cur, s);
            ++launches;
        } else {
            std::swap(cur, tmp);
        }
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) {
        launch_tp_normalize(cur, T, D, s);
        ++launches;
        e = cudaGetLastError();
    }
    std::vector<int> h_flags((size_t)n_spans + 1, 0);
    if (e == cudaSuccess && h_rows != nullptr) e = cudaMemcpyAsync(h_rows, cur, td * 4, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess && h_pooled != nullptr) {
        const int span01[2] = {0, T};
        e = cudaMemcpyAsync(d_spans, span01, sizeof(span01), cudaMemcpyHostToDevice, s);
        if (e == cudaSuccess) {
            launch_tp_span_pool(cur, d_mask, d_spans, d_spans + 1, 1, D, 1, pooled, nullptr, s);
            ++launches;
            e = cudaMemcpyAsync(h_pooled, pooled, (size_t)D * 4, cudaMemcpyDeviceToHost, s);
        }
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);   // span01 and d_spans are reused below
    }
    if (e == cudaSuccess && h_children != nullptr) {
        std::vector<int> se((size_t)2 * n_spans);
        for (int i = 0; i < n_spans; ++i) {
            se[i] = starts[i];
            se[n_spans + i] = ends[i];
        }
        e = cudaMemcpyAsync(d_spans, se.data(), se.size() * 4, cudaMemcpyHostToDevice, s);
        if (e == cudaSuccess) {
            launch_tp_span_pool(cur, d_mask, d_spans, d_spans + n_spans, n_spans, D, 0, children, d_flags, s);
            ++launches;
            e = cudaMemcpyAsync(h_children, children, (size_t)n_spans * D * 4, cudaMemcpyDeviceToHost, s);
        }
        if (e == cudaSuccess) e = cudaMemcpyAsync(h_flags.data(), d_flags, (size_t)n_spans * 4, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    }
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev1, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e == cudaSuccess && stats != nullptr) {
        std::memset(stats, 0, sizeof(*stats));
        stats->kernel_launches = launches;
        stats->uploaded_bytes = (int64_t)T * 8;
        stats->downloaded_bytes = (int64_t)((h_rows != nullptr ? td : 0) + (h_pooled != nullptr ? D : 0) + (size_t)n_spans * D) * 4;
        stats->valid_tokens = T;
        cudaEventElapsedTime(&stats->device_ms, rt->ev0, rt->ev1);
    }
    dev_free(d_tok);
    dev_free(d_mask);
    for (float** p : {&cur, &q, &k, &v, &att, &hid, &tmp, &ffn, &scores, &pooled, &children, &knf, &vnf}) dev_free(*p);
    for (uint8_t** p : {&kc, &vc, &ku, &vu, &kn, &vn}) dev_free(*p);
    dev_free(d_spans);
    dev_free(d_flags);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(err, std::string("token_pool_encode: ") + cudaGetErrorString(e));
    }
    if (n_children != nullptr) *n_children = n_spans;
    for (int i = 0; i < n_spans; ++i)
        if (h_flags[i] != 0)
            return fail(err, "token_pool_encode: span [" + std::to_string(starts[i]) + "," + std::to_string(ends[i]) +
                                 ") has no active tokens");
    return EOS_B200_OK;
}

}  // extern "C"
