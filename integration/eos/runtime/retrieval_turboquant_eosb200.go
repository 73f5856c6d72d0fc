//go:build linux && cgo && eosb200

// Scoring seam for runtime/retrieval_turboquant.go: the `qdocs` slice (:700-711) and the per-query call of
// topTurboQuantRetrievalScoresWithStats (:1306-1331, :1853-1887) are replaced by a packed corpus resident on the
// GPU and one batched exact top-k call; the multi-vector evaluation (retrieval_multivector_turboquant.go:746-810)
// and the dense / fp16 rerank stage (:1610-1662) map to their own entry points.  Place this file in runtime/ of
// odvcencio/eos and build with `-tags eosb200`.
//
// Scope: the library scores the Hadamard/MSE stage of the quantiser (norm * <R q, centroids[codes]>).  The QJL sign
// stage of turboquant.IPQuantizer (Signs, ResNorm) is not an operand of these calls; a caller that needs the IP
// variant's exact ranking keeps the host loop for it.
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
	"errors"
	"fmt"
	"sort"
	"unsafe"

	"m31labs.dev/turboquant"
)

func eosB200Err(rc C.int, cerr *C.char) error {
	if rc == C.EOS_B200_OK {
		return nil
	}
	msg := "eos_b200: unknown error"
	if cerr != nil {
		msg = C.GoString(cerr)
		C.eos_b200_free_cstring(cerr)
	}
	if rc == C.EOS_B200_DEVICE_STATUS {
		return fmt.Errorf("cuda device status: %s", msg)
	}
	return errors.New(msg)
}

// eosB200Scorer owns one runtime, one quantiser spec and one packed corpus on one GPU.
type eosB200Scorer struct {
	rt     *C.EosB200Runtime
	qz     *C.EosB200Quantizer
	corpus *C.EosB200Corpus
	ids    []string // document ids in row order (sorted ascending, so row order == id order)
	dim    int
}

// newEosB200Scorer packs and binds the documents once.  The rotation tables come from the real module's
// Spec() (the fields native_linux.go:9532-9545 uploads), so codes are the module's own Hadamard/MSE codes.
func newEosB200Scorer(device, dim, bits int, seed int64, docs []retrievalVectorRecord) (*eosB200Scorer, error) {
	spec := turboquant.NewHadamardRoundsWithSeed(dim, bits, 1, seed).Spec()
	s := &eosB200Scorer{dim: dim}
	var cerr *C.char
	if err := eosB200Err(C.eos_b200_runtime_create(C.int(device), &s.rt, &cerr), cerr); err != nil {
		return nil, err
	}
	perm := make([]int32, dim)
	for i, p := range spec.Perm {
		perm[i] = int32(p)
	}
	rc := C.eos_b200_quantizer_create(s.rt, C.int(dim), C.int(bits), (*C.int32_t)(unsafe.Pointer(&perm[0])),
		(*C.float)(unsafe.Pointer(&spec.Signs1[0])), (*C.float)(unsafe.Pointer(&spec.Signs2[0])),
		(*C.float)(unsafe.Pointer(&spec.Centroids[0])), (*C.float)(unsafe.Pointer(&spec.Boundaries[0])), &s.qz, &cerr)
	if err := eosB200Err(rc, cerr); err != nil {
		s.Close()
		return nil, err
	}
	// rows in ascending id order: "score descending, then id ascending" (retrievalScoreBetter,
	// retrieval_eval.go:1153-1161) is then "score descending, then row ascending", which is what the kernels break
	// ties by
	order := make([]int, len(docs))
	for i := range order {
		order[i] = i
	}
	sort.Slice(order, func(a, b int) bool { return docs[order[a]].ID < docs[order[b]].ID })
	n := len(docs)
	vecs := make([]float32, n*dim)
	s.ids = make([]string, n)
	for r, i := range order {
		copy(vecs[r*dim:(r+1)*dim], docs[i].Vector)
		s.ids[r] = docs[i].ID
	}
	codeBytes := (dim*bits + 7) / 8
	codes := make([]byte, n*codeBytes)
	norms := make([]float32, n)
	var st C.EosB200Stats
	rc = C.eos_b200_quantize(s.qz, (*C.float)(unsafe.Pointer(&vecs[0])), C.int64_t(n), (*C.uint8_t)(unsafe.Pointer(&codes[0])),
		(*C.float)(unsafe.Pointer(&norms[0])), &st, &cerr) // replaces `for doc: q.Quantize(doc.Vector)`
	if err := eosB200Err(rc, cerr); err != nil {
		s.Close()
		return nil, err
	}
	rc = C.eos_b200_corpus_bind(s.qz, (*C.uint8_t)(unsafe.Pointer(&codes[0])), (*C.float)(unsafe.Pointer(&norms[0])),
		C.int64_t(n), 0, 0, &s.corpus, &cerr)
	if err := eosB200Err(rc, cerr); err != nil {
		s.Close()
		return nil, err
	}
	return s, nil
}

func (s *eosB200Scorer) Close() {
	if s.corpus != nil {
		C.eos_b200_corpus_destroy(s.corpus)
	}
	if s.qz != nil {
		C.eos_b200_quantizer_destroy(s.qz)
	}
	if s.rt != nil {
		C.eos_b200_runtime_destroy(s.rt)
	}
	*s = eosB200Scorer{}
}

// topK scores every query against the whole corpus: the batched replacement of the loop at
// retrieval_turboquant.go:1306-1331.  queries_per_pass = 0 lets the library pick the kernel.
func (s *eosB200Scorer) topK(queries [][]float32, topK int) ([][]retrievalScoredDoc, error) {
	nq := len(queries)
	if nq == 0 {
		return nil, nil
	}
	if topK <= 0 || topK > len(s.ids) {
		topK = len(s.ids)
	}
	flat := make([]float32, nq*s.dim)
	for i, q := range queries {
		copy(flat[i*s.dim:(i+1)*s.dim], q)
	}
	ids := make([]int64, nq*topK)
	scores := make([]float32, nq*topK)
	var st C.EosB200Stats
	var cerr *C.char
	rc := C.eos_b200_score_topk(s.corpus, (*C.float)(unsafe.Pointer(&flat[0])), C.int(nq), C.int(topK), 0,
		(*C.int64_t)(unsafe.Pointer(&ids[0])), (*C.float)(unsafe.Pointer(&scores[0])), &st, &cerr)
	if err := eosB200Err(rc, cerr); err != nil {
		return nil, err
	}
	out := make([][]retrievalScoredDoc, nq)
	for i := 0; i < nq; i++ {
		row := make([]retrievalScoredDoc, 0, topK)
		for j := 0; j < topK; j++ {
			id := ids[i*topK+j]
			if id < 0 {
				break
			}
			row = append(row, retrievalScoredDoc{ID: s.ids[id], Score: scores[i*topK+j]})
		}
		out[i] = row
	}
	return out, nil
}

// parentTopK is topTurboQuantMultiVectorParentScores (retrieval_multivector_turboquant.go:746-810) for all queries:
// rows of the corpus are child vectors, parentOfChild[i] names the parent of row i.
func (s *eosB200Scorer) parentTopK(parentOfChild []int32, parents int, queries [][]float32, topK, topN int, penalty float64) ([][]int64, [][]float32, error) {
	nq := len(queries)
	flat := make([]float32, nq*s.dim)
	for i, q := range queries {
		copy(flat[i*s.dim:(i+1)*s.dim], q)
	}
	ids := make([]int64, nq*topK)
	scores := make([]float32, nq*topK)
	var st C.EosB200Stats
	var cerr *C.char
	rc := C.eos_b200_parent_topk(s.corpus, (*C.int32_t)(unsafe.Pointer(&parentOfChild[0])), C.int(parents),
		(*C.float)(unsafe.Pointer(&flat[0])), C.int(nq), 1, C.int(topN), C.double(penalty), C.int(topK),
		(*C.int64_t)(unsafe.Pointer(&ids[0])), (*C.float)(unsafe.Pointer(&scores[0])), &st, &cerr)
	if err := eosB200Err(rc, cerr); err != nil {
		return nil, nil, err
	}
	oi, os := make([][]int64, nq), make([][]float32, nq)
	for i := 0; i < nq; i++ {
		oi[i], os[i] = ids[i*topK:(i+1)*topK], scores[i*topK:(i+1)*topK]
	}
	return oi, os, nil
}

// eosB200Reranker is the rerank stage after an over-fetched top-k: topDenseRerankScores / topFP16RerankScores
// (retrieval_turboquant.go:1610-1662).
type eosB200Reranker struct{ ix *C.EosB200DenseIndex }

func newEosB200Reranker(rt *C.EosB200Runtime, vectors []float32, n, dim int, fp16Sidecar bool) (*eosB200Reranker, error) {
	var ix *C.EosB200DenseIndex
	var cerr *C.char
	f16 := C.int(0)
	if fp16Sidecar {
		f16 = 1
	}
	rc := C.eos_b200_dense_bind(rt, (*C.float)(unsafe.Pointer(&vectors[0])), C.int64_t(n), C.int(dim), f16, &ix, &cerr)
	if err := eosB200Err(rc, cerr); err != nil {
		return nil, err
	}
	return &eosB200Reranker{ix: ix}, nil
}

func (r *eosB200Reranker) rerank(queries []float32, nq int, candidates []int64, cand, topK int) ([]int64, []float32, error) {
	ids := make([]int64, nq*topK)
	scores := make([]float32, nq*topK)
	var st C.EosB200Stats
	var cerr *C.char
	rc := C.eos_b200_dense_rerank(r.ix, (*C.float)(unsafe.Pointer(&queries[0])), C.int(nq), (*C.int64_t)(unsafe.Pointer(&candidates[0])),
		C.int(cand), C.int(topK), (*C.int64_t)(unsafe.Pointer(&ids[0])), (*C.float)(unsafe.Pointer(&scores[0])), &st, &cerr)
	return ids, scores, eosB200Err(rc, cerr)
}

func (r *eosB200Reranker) Close() { C.eos_b200_dense_destroy(r.ix) }

// Sharded corpus, one process per GPU.  Rank 0 makes the 128-byte id and hands it to the other ranks by whatever
// channel the launcher has; every rank then binds rows [lo, hi) with id_base = lo and calls scoreSharded with the
// same queries.  The exchange (thresholds, per-shard key lists) is NCCL inside the library.
func eosB200CommID() ([128]byte, error) {
	var id C.EosB200NcclId
	var cerr *C.char
	if err := eosB200Err(C.eos_b200_comm_unique_id(&id, &cerr), cerr); err != nil {
		return [128]byte{}, err
	}
	var out [128]byte
	copy(out[:], C.GoBytes(unsafe.Pointer(&id), 128))
	return out, nil
}

type eosB200Comm struct{ h *C.EosB200Comm }

func newEosB200Comm(rt *C.EosB200Runtime, rank, world int, id [128]byte) (*eosB200Comm, error) {
	var cid C.EosB200NcclId
	for i := range id {
		cid.internal[i] = C.char(id[i])
	}
	var h *C.EosB200Comm
	var cerr *C.char
	if err := eosB200Err(C.eos_b200_comm_init(rt, C.int(rank), C.int(world), &cid, &h, &cerr), cerr); err != nil {
		return nil, err
	}
	return &eosB200Comm{h: h}, nil
}

func (c *eosB200Comm) Close() { C.eos_b200_comm_destroy(c.h) }
