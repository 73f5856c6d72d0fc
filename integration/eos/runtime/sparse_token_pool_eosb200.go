//go:build linux && cgo && eosb200

// Device path for sparseTokenPoolEncoder (runtime/sparse_token_pool_vector_export.go): embedTextFullEncoderRows
// (:1301-1335), embedTextFullEncoder (:1290-1299) and the span pooling of
// writeSparseTokenPoolTokenSpanChildVectorCache (:802-890) call the library instead of the host loops; tokenizing,
// resume files and progress reporting stay as they are.  Place this file in runtime/ of odvcencio/eos and build with
// `-tags eosb200`.
//
// Written against the Eos tree without a Go toolchain at hand: read against the types it names, not compiled.
package runtime

/*
#cgo CFLAGS: -I${SRCDIR}/../third_party/eos_b200/include
#cgo LDFLAGS: -L${SRCDIR}/../third_party/eos_b200 -leos_b200 -Wl,-rpath,$ORIGIN
#include <stdlib.h>
#include "eos_b200.h"
*/
import "C"

import (
	"fmt"
	"unsafe"

	"m31labs.dev/turboquant"
)

type eosB200TokenPool struct {
	rt     *C.EosB200Runtime
	h      *C.EosB200TokenPool
	keyQz  *C.EosB200Quantizer
	valQz  *C.EosB200Quantizer
	dim    int
	hidden int
}

func b2i(v bool) C.int32_t {
	if v {
		return 1
	}
	return 0
}

func eosB200Quantizer(rt *C.EosB200Runtime, dim, bits int, seed int64) (*C.EosB200Quantizer, error) {
	spec := turboquant.NewHadamardRoundsWithSeed(dim, bits, 1, seed).Spec() // the module's own tables
	perm := make([]int32, dim)
	for i, p := range spec.Perm {
		perm[i] = int32(p)
	}
	var qz *C.EosB200Quantizer
	var cerr *C.char
	rc := C.eos_b200_quantizer_create(rt, C.int(dim), C.int(bits), (*C.int32_t)(unsafe.Pointer(&perm[0])),
		(*C.float)(unsafe.Pointer(&spec.Signs1[0])), (*C.float)(unsafe.Pointer(&spec.Signs2[0])),
		(*C.float)(unsafe.Pointer(&spec.Centroids[0])), (*C.float)(unsafe.Pointer(&spec.Boundaries[0])), &qz, &cerr)
	return qz, eosB200Err(rc, cerr)
}

// newEosB200TokenPool uploads the seven weight tensors of a sparseTokenPoolEncoder whose fullEncoderOK is set.
func newEosB200TokenPool(rt *C.EosB200Runtime, e *sparseTokenPoolEncoder) (*eosB200TokenPool, error) {
	if !e.fullEncoderOK {
		return nil, fmt.Errorf("token-pool device path requires full manifest encoder weights; missing/invalid weights: %v", e.skippedWeights)
	}
	dim, hidden := e.tokenEmbedding.Shape[1], e.hiddenProjection.Shape[1]
	var d C.EosB200TokenPoolDesc
	d.vocab, d.dim, d.hidden = C.int32_t(e.tokenEmbedding.Shape[0]), C.int32_t(dim), C.int32_t(hidden)
	d.encoder_repeats = C.int32_t(e.manifest.EncoderRepeats)
	d.attention_residual, d.attention_layer_norm = b2i(e.manifest.AttentionResidual), b2i(e.manifest.AttentionLayerNorm)
	d.ffn_residual, d.ffn_layer_norm = b2i(e.manifest.FFNResidual), b2i(e.manifest.FFNLayerNorm)
	f := func(v []float32) *C.float { return (*C.float)(unsafe.Pointer(&v[0])) }
	d.token_embedding, d.attention_query, d.attention_key = f(e.tokenEmbedding.F32), f(e.attentionQuery.F32), f(e.attentionKey.F32)
	d.attention_value, d.attention_output = f(e.attentionValue.F32), f(e.attentionOutput.F32)
	d.hidden_projection, d.projection = f(e.hiddenProjection.F32), f(e.projection.F32)
	tp := &eosB200TokenPool{rt: rt, dim: dim, hidden: hidden}
	var cerr *C.char
	if err := eosB200Err(C.eos_b200_token_pool_bind(rt, &d, &tp.h, &cerr), cerr); err != nil {
		return nil, err
	}
	if e.cfg.AttentionMode == SparseTokenPoolAttentionModeTurboQuantSparse {
		var err error
		if tp.keyQz, err = eosB200Quantizer(rt, dim, e.cfg.KeyBits, e.cfg.Seed); err != nil {
			tp.Close()
			return nil, err
		}
		if tp.valQz, err = eosB200Quantizer(rt, dim, e.cfg.ValueBits, e.cfg.Seed); err != nil {
			tp.Close()
			return nil, err
		}
	}
	return tp, nil
}

func (tp *eosB200TokenPool) Close() {
	if tp.h != nil {
		C.eos_b200_token_pool_destroy(tp.h)
	}
	if tp.keyQz != nil {
		C.eos_b200_quantizer_destroy(tp.keyQz)
	}
	if tp.valQz != nil {
		C.eos_b200_quantizer_destroy(tp.valQz)
	}
	*tp = eosB200TokenPool{}
}

// spanChildVectors replaces embedTextTokenRows + the poolSparseTokenRowsRange loop for one record: one unit vector
// per token span, in span order.
func (tp *eosB200TokenPool) spanChildVectors(e *sparseTokenPoolEncoder, tokens, mask []int32) ([][]float32, error) {
	spans := sparseTokenPoolTokenSpans(len(tokens), e.cfg.TokenSpanTokens, e.cfg.TokenSpanOverlap, e.cfg.TokenSpanMinTokens)
	if len(spans) == 0 {
		return nil, fmt.Errorf("token-span mode selected no spans")
	}
	mode := C.int(C.EOS_B200_TOKEN_POOL_DENSE)
	if e.cfg.AttentionMode == SparseTokenPoolAttentionModeTurboQuantSparse {
		mode = C.int(C.EOS_B200_TOKEN_POOL_TURBO_SPARSE)
	}
	flat := make([]float32, len(spans)*tp.dim)
	var n C.int
	var st C.EosB200Stats
	var cerr *C.char
	rc := C.eos_b200_token_pool_encode(tp.h, (*C.int32_t)(unsafe.Pointer(&tokens[0])), (*C.int32_t)(unsafe.Pointer(&mask[0])),
		C.int(len(tokens)), mode, tp.keyQz, tp.valQz, C.int(e.cfg.TopK), C.int(e.cfg.RouteBlockSize), C.int(e.cfg.RouteTopBlocks),
		C.int(e.cfg.TokenSpanTokens), C.int(e.cfg.TokenSpanOverlap), C.int(e.cfg.TokenSpanMinTokens), nil, nil,
		(*C.float)(unsafe.Pointer(&flat[0])), C.int(len(spans)), &n, &st, &cerr)
	if err := eosB200Err(rc, cerr); err != nil {
		return nil, err
	}
	out := make([][]float32, int(n))
	for i := range out {
		out[i] = flat[i*tp.dim : (i+1)*tp.dim]
	}
	return out, nil
}
