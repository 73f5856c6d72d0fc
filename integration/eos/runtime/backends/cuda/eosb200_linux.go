//go:build linux && cgo && eosb200

// Drop-in device path for the embed half of Eos's query-time embed-and-score path, backed by libeos_b200.so
// (hand-written sm_100a kernels, no NVRTC, no cuBLAS).  Place this file in runtime/backends/cuda/ of odvcencio/eos
// and build with `-tags eosb200`; it supplies dispatchStep's StepBERTEmbedder branch (cuda.go:394-452), the
// dense projection accelerator and the compiled embed_pooled_batch pipeline.  Every exported symbol used below is
// declared in include/eos_b200.h; the Python tests of the library bind the same symbols with the same structs.
//
// This file was written against the Eos tree without a Go toolchain at hand: it has been read against the types it
// names (backend.Tensor, eosartifact.Step, backend.StepDispatchResult) but not compiled.
package cuda

/*
#cgo CFLAGS: -I${SRCDIR}/../../../third_party/eos_b200/include
#cgo LDFLAGS: -L${SRCDIR}/../../../third_party/eos_b200 -leos_b200 -Wl,-rpath,$ORIGIN
#include <stdlib.h>
#include <string.h>
#include "eos_b200.h"
*/
import "C"

import (
	"crypto/sha256"
	"encoding/hex"
	"errors"
	"fmt"
	"strconv"
	"sync"
	"unsafe"

	eosartifact "github.com/odvcencio/eos/artifact/eos"
	"github.com/odvcencio/eos/runtime/backend"
)

// b200Error is the twin of cStringError (native_linux.go:8601): int return code, caller-owned message.
func b200Error(rc C.int, cerr *C.char) error {
	if rc == C.EOS_B200_OK {
		return nil
	}
	msg := "eos_b200: unknown error"
	if cerr != nil {
		msg = C.GoString(cerr)
		C.eos_b200_free_cstring(cerr)
	}
	if rc == C.EOS_B200_DEVICE_STATUS {
		// same class as the status-word errors of the NVRTC kernels (native_linux.go:699-705, 2726-2728)
		return fmt.Errorf("cuda device status: %s", msg)
	}
	return errors.New(msg)
}

// b200Runtime replaces deviceRuntime for this path (newDeviceRuntime, native_linux.go:3127).
type b200Runtime struct {
	h        *C.EosB200Runtime
	mu       sync.Mutex
	encoders map[string]*b200Encoder // keyed by the weight fingerprint, like bindBGEFullEncoder (cuda.go:174-228)
}

func newB200Runtime(device int) (*b200Runtime, error) {
	var h *C.EosB200Runtime
	var cerr *C.char
	if err := b200Error(C.eos_b200_runtime_create(C.int(device), &h, &cerr), cerr); err != nil {
		return nil, err
	}
	return &b200Runtime{h: h, encoders: map[string]*b200Encoder{}}, nil
}

func (rt *b200Runtime) Close() {
	rt.mu.Lock()
	defer rt.mu.Unlock()
	for k, e := range rt.encoders {
		C.eos_b200_encoder_destroy(e.h)
		delete(rt.encoders, k)
	}
	if rt.h != nil {
		C.eos_b200_runtime_destroy(rt.h)
		rt.h = nil
	}
}

type b200Encoder struct {
	h      *C.EosB200Encoder
	outDim int
}

// cBuf copies a Go slice into C memory for the duration of a bind call (no Go pointer is retained by C).
type cArena struct{ ptrs []unsafe.Pointer }

func (a *cArena) f32(v []float32) *C.float {
	if len(v) == 0 {
		return nil
	}
	n := C.size_t(len(v)) * 4
	p := C.malloc(n)
	C.memcpy(p, unsafe.Pointer(&v[0]), n)
	a.ptrs = append(a.ptrs, p)
	return (*C.float)(p)
}

func (a *cArena) i8(v []int8) *C.int8_t {
	if len(v) == 0 {
		return nil
	}
	n := C.size_t(len(v))
	p := C.malloc(n)
	C.memcpy(p, unsafe.Pointer(&v[0]), n)
	a.ptrs = append(a.ptrs, p)
	return (*C.int8_t)(p)
}

func (a *cArena) free() {
	for _, p := range a.ptrs {
		C.free(p)
	}
	a.ptrs = nil
}

// q8Codes recovers the int8 codes of a "q8" tensor from its dequantised values and its scale(s), the inverse of
// packQuantizedTensorStorage (runtime/mll_export.go:897-962): code = round(value / scale), |code| <= 127.
func q8Codes(values []float32, scales []float32, rows, cols int) []int8 {
	out := make([]int8, len(values))
	for r := 0; r < rows; r++ {
		s := scales[0]
		if len(scales) == rows {
			s = scales[r]
		}
		for c := 0; c < cols; c++ {
			i := r*cols + c
			if s == 0 {
				continue
			}
			q := values[i] / s
			if q >= 0 {
				q += 0.5
			} else {
				q -= 0.5
			}
			v := int(q)
			if v > 127 {
				v = 127
			} else if v < -127 {
				v = -127
			}
			out[i] = int8(v)
		}
	}
	return out
}

// matrix fills an EosB200Matrix from a backend.Tensor holding a dense weight in HF [out, in] layout.  A "q8" tensor
// carries its scale(s) in the step attribute "<role>_scales" (the per-tensor scale of weight_file.go:305-356 has
// one entry); any other dtype is passed as dense values.
func (a *cArena) matrix(t *backend.Tensor, scales []float32) C.EosB200Matrix {
	var m C.EosB200Matrix
	m.rows, m.cols = C.int32_t(t.Shape[0]), C.int32_t(t.Shape[1])
	if t.DType == "q8" && len(scales) > 0 {
		m.q8_codes = a.i8(q8Codes(t.F32, scales, t.Shape[0], t.Shape[1]))
		m.q8_scales = a.f32(scales)
		m.n_scales = C.int32_t(len(scales))
	} else {
		m.dense = a.f32(t.F32)
	}
	return m
}

func attrInt(step eosartifact.Step, key string, def int) int {
	if v, ok := step.Attributes[key]; ok {
		if n, err := strconv.Atoi(v); err == nil {
			return n
		}
	}
	return def
}

func attrFloat(step eosartifact.Step, key string, def float64) float64 {
	if v, ok := step.Attributes[key]; ok {
		if f, err := strconv.ParseFloat(v, 64); err == nil {
			return f
		}
	}
	return def
}

func weightFingerprint(inputs []*backend.Tensor) string {
	h := sha256.New()
	for _, t := range inputs[3:] {
		if len(t.F32) > 0 {
			h.Write(unsafe.Slice((*byte)(unsafe.Pointer(&t.F32[0])), len(t.F32)*4))
		}
	}
	return hex.EncodeToString(h.Sum(nil))
}

// bindB200Encoder binds the 8 + 16*L tensors of a StepBERTEmbedder once
// (order: input_ids, attention_mask, token_type_ids, word / position / token-type embeddings, embedding LayerNorm
// weight / bias, then 16 tensors per layer, runtime/pretrained_bert_importer.go:920-984).
func (rt *b200Runtime) bindB200Encoder(step eosartifact.Step, in []*backend.Tensor, scales map[int][]float32, head *backend.Tensor) (*b200Encoder, error) {
	if len(in) < 8+16 || (len(in)-8)%16 != 0 {
		return nil, fmt.Errorf("bert_embedder expects 8 + 16*L inputs, got %d", len(in))
	}
	key := weightFingerprint(in)
	rt.mu.Lock()
	defer rt.mu.Unlock()
	if e, ok := rt.encoders[key]; ok {
		return e, nil
	}
	layers := (len(in) - 8) / 16
	hidden := in[3].Shape[1]
	arena := &cArena{}
	defer arena.free()
	desc := (*C.EosB200EncoderDesc)(C.calloc(1, C.sizeof_EosB200EncoderDesc))
	defer C.free(unsafe.Pointer(desc))
	lw := (*C.EosB200EncoderLayer)(C.calloc(C.size_t(layers), C.sizeof_EosB200EncoderLayer))
	defer C.free(unsafe.Pointer(lw))
	lws := unsafe.Slice(lw, layers)
	desc.layers, desc.hidden = C.int32_t(layers), C.int32_t(hidden)
	desc.heads = C.int32_t(attrInt(step, "num_attention_heads", 0))
	desc.intermediate = C.int32_t(in[8+10].Shape[0])
	desc.vocab, desc.max_positions, desc.type_vocab = C.int32_t(in[3].Shape[0]), C.int32_t(in[4].Shape[0]), C.int32_t(in[5].Shape[0])
	desc.epsilon = C.double(attrFloat(step, "epsilon", 1e-12))
	desc.activation = C.EOS_B200_ACT_GELU_ERF
	if step.Attributes["hidden_act"] == "gelu_tanh" {
		desc.activation = C.EOS_B200_ACT_GELU_TANH
	}
	desc.pooling = C.EOS_B200_POOL_MASKED_MEAN
	if step.Attributes["pooling"] == "cls" {
		desc.pooling = C.EOS_B200_POOL_CLS
	}
	// q8 codes expanded to f16 once at bind (exact; the faster mode).  EOS_B200_WEIGHTS_Q8_SMEM_DEQUANT keeps one
	// byte per weight in HBM and expands in shared memory: the outputs are bit-identical.
	desc.weight_mode = C.EOS_B200_WEIGHTS_F16_RESIDENT
	desc.token_embeddings = arena.f32(in[3].F32)
	desc.position_embeddings = arena.f32(in[4].F32)
	desc.type_embeddings = arena.f32(in[5].F32)
	desc.embedding_ln_gamma = arena.f32(in[6].F32)
	desc.embedding_ln_beta = arena.f32(in[7].F32)
	for l := 0; l < layers; l++ {
		b := 8 + 16*l
		lws[l].query, lws[l].query_bias = arena.matrix(in[b+0], scales[b+0]), arena.f32(in[b+1].F32)
		lws[l].key, lws[l].key_bias = arena.matrix(in[b+2], scales[b+2]), arena.f32(in[b+3].F32)
		lws[l].value, lws[l].value_bias = arena.matrix(in[b+4], scales[b+4]), arena.f32(in[b+5].F32)
		lws[l].attn_out, lws[l].attn_out_bias = arena.matrix(in[b+6], scales[b+6]), arena.f32(in[b+7].F32)
		lws[l].attn_ln_gamma, lws[l].attn_ln_beta = arena.f32(in[b+8].F32), arena.f32(in[b+9].F32)
		lws[l].inter, lws[l].inter_bias = arena.matrix(in[b+10], scales[b+10]), arena.f32(in[b+11].F32)
		lws[l].out, lws[l].out_bias = arena.matrix(in[b+12], scales[b+12]), arena.f32(in[b+13].F32)
		lws[l].out_ln_gamma, lws[l].out_ln_beta = arena.f32(in[b+14].F32), arena.f32(in[b+15].F32)
	}
	desc.layer = lw
	outDim := hidden
	if head != nil { // PretrainedBERTProjectionHead ([in, out], no bias; pretrained_bert_projection_head.go:84-100)
		desc.head_out = C.int32_t(head.Shape[1])
		desc.head_weights = arena.f32(head.F32)
		outDim = head.Shape[1]
	}
	var h *C.EosB200Encoder
	var cerr *C.char
	if err := b200Error(C.eos_b200_encoder_bind(rt.h, desc, &h, &cerr), cerr); err != nil {
		return nil, err
	}
	e := &b200Encoder{h: h, outDim: outDim}
	rt.encoders[key] = e
	return e, nil
}

// runB200Embedder is the body of dispatchStep(StepBERTEmbedder): host [B,T] int32 inputs in, [B,E] f32 out.
func (rt *b200Runtime) runB200Embedder(e *b200Encoder, ids, mask, types *backend.Tensor, outputType eosartifact.ValueType) (backend.StepDispatchResult, error) {
	if len(ids.Shape) != 2 || len(ids.I32) == 0 {
		return backend.StepDispatchResult{}, fmt.Errorf("bert_embedder input_ids must be a non-empty [B,T] tensor")
	}
	b, t := ids.Shape[0], ids.Shape[1]
	out := make([]float32, b*e.outDim)
	var st C.EosB200Stats
	var cerr *C.char
	var typesPtr *C.int32_t
	if types != nil && len(types.I32) == b*t {
		typesPtr = (*C.int32_t)(unsafe.Pointer(&types.I32[0]))
	}
	// the host pointers are only used during the call (cgo pointer-passing rule: no Go pointer is kept)
	rc := C.eos_b200_encoder_run(e.h, (*C.int32_t)(unsafe.Pointer(&ids.I32[0])), (*C.int32_t)(unsafe.Pointer(&mask.I32[0])),
		typesPtr, C.int(b), C.int(t), (*C.float)(unsafe.Pointer(&out[0])), &st, &cerr)
	if err := b200Error(rc, cerr); err != nil {
		return backend.StepDispatchResult{}, err
	}
	tensor := backend.NewTensorF32([]int{b, e.outDim}, out)
	if outputType.DType == "f16" { // dtype tagging stays in the adapter (newStepOutputTensor, native_linux.go:9492-9503)
		tensor.DType = "f16"
	}
	return backend.StepDispatchResult{
		Outputs:      []*backend.Tensor{tensor},
		VariantEntry: "eos_b200_encoder_run",
		SourceHash:   C.GoString(C.eos_b200_version()),
		Metadata: map[string]any{
			"kernel_launches":  int(st.kernel_launches),
			"uploaded_bytes":   int64(st.uploaded_bytes),
			"downloaded_bytes": int64(st.downloaded_bytes),
			"valid_tokens":     int64(st.valid_tokens),
			"device_ms":        float64(st.device_ms),
		},
	}, nil
}

// runB200EmbedderBatches embeds several [B,T] batches back to back (the loop of EmbedBatch,
// runtime/embedding_model.go:664-700) without a host stall between them: every batch is submitted with
// eos_b200_encoder_submit and one eos_b200_encoder_wait completes them all.  C keeps the host pointers until the wait,
// so the inputs and outputs of the batches in flight live in C memory (cgo pointer-passing rule) and are copied out
// after the wait.  ids[i], mask[i] are [B_i, T_i] int32 tensors; types may be nil.
func (rt *b200Runtime) runB200EmbedderBatches(e *b200Encoder, ids, mask, types []*backend.Tensor) ([]*backend.Tensor, error) {
	var arena cArena
	defer arena.free()
	i32 := func(v []int32) *C.int32_t {
		n := C.size_t(len(v)) * 4
		p := C.malloc(n)
		C.memcpy(p, unsafe.Pointer(&v[0]), n)
		arena.ptrs = append(arena.ptrs, p)
		return (*C.int32_t)(p)
	}
	outs := make([]unsafe.Pointer, len(ids))
	var cerr *C.char
	for i := range ids {
		if len(ids[i].Shape) != 2 || len(ids[i].I32) == 0 || len(mask[i].I32) != len(ids[i].I32) {
			return nil, fmt.Errorf("bert_embedder input_ids / attention_mask must be non-empty [B,T] tensors of one shape")
		}
		b, t := ids[i].Shape[0], ids[i].Shape[1]
		var typesPtr *C.int32_t
		if types != nil && types[i] != nil && len(types[i].I32) == b*t {
			typesPtr = i32(types[i].I32)
		}
		outs[i] = C.malloc(C.size_t(b*e.outDim) * 4)
		arena.ptrs = append(arena.ptrs, outs[i])
		rc := C.eos_b200_encoder_submit(e.h, i32(ids[i].I32), i32(mask[i].I32), typesPtr, C.int(b), C.int(t),
			(*C.float)(outs[i]), &cerr)
		if err := b200Error(rc, cerr); err != nil {
			var werr *C.char
			C.eos_b200_encoder_wait(e.h, nil, &werr) // nothing may stay in flight over buffers about to be freed
			if werr != nil {
				C.eos_b200_free_cstring(werr)
			}
			return nil, err
		}
	}
	var st C.EosB200Stats
	if err := b200Error(C.eos_b200_encoder_wait(e.h, &st, &cerr), cerr); err != nil {
		return nil, err
	}
	res := make([]*backend.Tensor, len(ids))
	for i := range ids {
		b := ids[i].Shape[0]
		out := make([]float32, b*e.outDim)
		C.memcpy(unsafe.Pointer(&out[0]), outs[i], C.size_t(len(out))*4)
		res[i] = backend.NewTensorF32([]int{b, e.outDim}, out)
	}
	return res, nil
}

// dispatchStepB200 is what executor.dispatchStep calls first when the build tag is set; (result, handled, error)
// as in cuda.go:394.
func (e *executor) dispatchStepB200(step eosartifact.Step, outputType eosartifact.ValueType, inputs []*backend.Tensor) (backend.StepDispatchResult, bool, error) {
	if e.b200 == nil {
		return backend.StepDispatchResult{}, false, nil
	}
	switch step.Kind {
	case eosartifact.StepBERTEmbedder:
		enc, err := e.b200.bindB200Encoder(step, inputs, e.q8Scales(step), e.projectionHead(step))
		if err != nil {
			return backend.StepDispatchResult{}, true, err
		}
		res, err := e.b200.runB200Embedder(enc, inputs[0], inputs[1], inputs[2], outputType)
		return res, true, err
	case eosartifact.StepMatMul:
		if len(inputs) != 2 || len(inputs[1].Shape) != 2 {
			return backend.StepDispatchResult{}, false, nil
		}
		out, err := e.b200.linear(inputs[0], inputs[1])
		if err != nil {
			return backend.StepDispatchResult{}, true, err
		}
		return backend.StepDispatchResult{Outputs: []*backend.Tensor{out}, VariantEntry: "eos_b200_linear"}, true, nil
	case eosartifact.StepSparseAttention:
		// cuda.go:565-577: query, key, value [T, D] or [B, T, D] fp32; top_k / route_* attributes
		if len(inputs) != 3 {
			return backend.StepDispatchResult{}, false, nil
		}
		out, err := e.b200.sparseAttention(inputs[0], inputs[1], inputs[2], attrInt(step, "top_k", 0),
			attrInt(step, "route_block_size", 0), attrInt(step, "route_top_blocks", 0))
		if err != nil {
			return backend.StepDispatchResult{}, true, err
		}
		return backend.StepDispatchResult{Outputs: []*backend.Tensor{out}, VariantEntry: "eos_b200_sparse_attention"}, true, nil
	}
	return backend.StepDispatchResult{}, false, nil
}

// sparseAttention maps sparseAttentionTensor (runtime/backend/attention_ops.go:218-276).  Budgets above 128 keys or
// route blocks are outside the library's limit (EOS_SPARSE_ATTENTION_MAX_TOPK): the error falls through to the host.
func (rt *b200Runtime) sparseAttention(q, k, v *backend.Tensor, topK, routeBlock, routeTop int) (*backend.Tensor, error) {
	rank := len(q.Shape)
	if rank != len(k.Shape) || rank != len(v.Shape) || (rank != 2 && rank != 3) {
		return nil, errors.New("sparse_attention expects rank-2 or rank-3 query/key/value tensors")
	}
	batches := 1
	if rank == 3 {
		batches = q.Shape[0]
	}
	qLen, dim := q.Shape[rank-2], q.Shape[rank-1]
	kLen, vDim := k.Shape[rank-2], v.Shape[rank-1]
	out := make([]float32, batches*qLen*vDim)
	var st C.EosB200Stats
	var cerr *C.char
	var kp, vp *C.float
	if kLen > 0 {
		kp, vp = (*C.float)(unsafe.Pointer(&k.F32[0])), (*C.float)(unsafe.Pointer(&v.F32[0]))
	}
	rc := C.eos_b200_sparse_attention(rt.h, (*C.float)(unsafe.Pointer(&q.F32[0])), kp, vp, C.int(batches), C.int(qLen),
		C.int(kLen), C.int(dim), C.int(vDim), C.int(topK), C.int(routeBlock), C.int(routeTop),
		(*C.float)(unsafe.Pointer(&out[0])), &st, &cerr)
	if err := b200Error(rc, cerr); err != nil {
		return nil, err
	}
	shape := append(append([]int(nil), q.Shape[:rank-1]...), vDim)
	return backend.NewTensorF16(shape, out), nil
}

// linear maps a single dense projection (MatMulAccelerator, backend.go:785-795): x [rows, k] times rhs [k, n]
// (Eos's [in, out] layout), fp32 accumulate, f16-rounded operands.
func (rt *b200Runtime) linear(x, rhs *backend.Tensor) (*backend.Tensor, error) {
	k, n := rhs.Shape[0], rhs.Shape[1]
	rows := len(x.F32) / k
	// the library takes HF [out, in]: transpose once
	wt := make([]float32, n*k)
	for i := 0; i < k; i++ {
		for j := 0; j < n; j++ {
			wt[j*k+i] = rhs.F32[i*n+j]
		}
	}
	var m C.EosB200Matrix
	m.rows, m.cols = C.int32_t(n), C.int32_t(k)
	m.dense = (*C.float)(unsafe.Pointer(&wt[0]))
	out := make([]float32, rows*n)
	var st C.EosB200Stats
	var cerr *C.char
	rc := C.eos_b200_linear(rt.h, (*C.float)(unsafe.Pointer(&x.F32[0])), C.int64_t(rows), &m, nil, 0, nil,
		C.EOS_B200_WEIGHTS_F16_RESIDENT, (*C.float)(unsafe.Pointer(&out[0])), &st, &cerr)
	if err := b200Error(rc, cerr); err != nil {
		return nil, err
	}
	shape := append(append([]int(nil), x.Shape[:len(x.Shape)-1]...), n)
	return backend.NewTensorF32(shape, out), nil
}

// embedPooled is the fused fast path of the compiled pipeline embed_pooled_batch
// (examples/embed_masked_pooled.eos:11-16; executor.Run, cuda.go:344-363).
type b200EmbedPooled struct{ h *C.EosB200EmbedPooled }

func (rt *b200Runtime) bindEmbedPooled(table, projection *backend.Tensor) (*b200EmbedPooled, error) {
	var h *C.EosB200EmbedPooled
	var cerr *C.char
	rc := C.eos_b200_embed_pooled_bind(rt.h, (*C.float)(unsafe.Pointer(&table.F32[0])), C.int(table.Shape[0]), C.int(table.Shape[1]),
		(*C.float)(unsafe.Pointer(&projection.F32[0])), C.int(projection.Shape[1]), &h, &cerr)
	if err := b200Error(rc, cerr); err != nil {
		return nil, err
	}
	return &b200EmbedPooled{h: h}, nil
}

// setMatMulScale forwards the matmul step's `scale` attribute, already resolved to a number by matmulScale
// (runtime/backend/tensor_ops.go:1291-1315).
func (p *b200EmbedPooled) setMatMulScale(scale float32) error {
	var cerr *C.char
	return b200Error(C.eos_b200_embed_pooled_set_matmul_scale(p.h, C.float(scale), &cerr), cerr)
}

func (p *b200EmbedPooled) run(tokens, mask *backend.Tensor, outDim int) (*backend.Tensor, error) {
	b, t := tokens.Shape[0], tokens.Shape[1]
	out := make([]float32, b*outDim)
	var st C.EosB200Stats
	var cerr *C.char
	rc := C.eos_b200_embed_pooled_run(p.h, (*C.int32_t)(unsafe.Pointer(&tokens.I32[0])), (*C.int32_t)(unsafe.Pointer(&mask.I32[0])),
		C.int(b), C.int(t), 0, (*C.float)(unsafe.Pointer(&out[0])), &st, &cerr)
	if err := b200Error(rc, cerr); err != nil {
		return nil, err
	}
	return backend.NewTensorF32([]int{b, outDim}, out), nil
}

func (p *b200EmbedPooled) Close() { C.eos_b200_embed_pooled_destroy(p.h) }

// b200KernelBinary describes the offline-compiled image for the module manifest (KernelVariant.Binary,
// artifact/eos/module.go:216-224).  The kernels are linked into libeos_b200.so rather than loaded through the
// driver's module loader, so the manifest entry records the shared library itself: Format "so", Arch "sm_100a".
func b200KernelBinary(libBytes []byte, sourceSHA string) *eosartifact.KernelBinary {
	sum := sha256.Sum256(libBytes)
	return &eosartifact.KernelBinary{
		Format:       "so",
		Arch:         "sm_100a",
		Toolchain:    "nvcc 12.9 -gencode arch=compute_100a,code=sm_100a",
		SourceSHA256: sourceSHA,
		SHA256:       hex.EncodeToString(sum[:]),
		Data:         libBytes,
	}
}
