//go:build b200

package b200

// SOURCE ONLY: not compiled here (see doc.go).

import (
	"errors"
	"fmt"
	"sync"
	"unsafe"

	"github.com/ebitengine/purego"
)

// Status codes of include/b200_resident.h.
const (
	stOK = iota
	stDeclined
	stKVPoolFull
	stBadArgument
	stCUDAError
	stTimeout
	stNCCLError
)

// Tensor roles (B200_T_*), tensor kinds (B200_K_*), draw kinds (B200_DRAW_*), kernel classes (B200_CLASS_*): the values
// of include/b200_resident.h, kept in the header's order.
const (
	tEmbed = iota
	tFinalNorm
	tLMHead
	tAttnNorm
	tWQ
	tWK
	tWV
	tWO
	tQNorm
	tKNorm
	tFFNNorm
	tGate
	tUp
	tDown
	tRouter
	tExpertGate
	tExpertUp
	tExpertDown
)
const (
	kF32 = iota
	kF16
	kQ4K
	kQ5K
	kQ6K
	kI8 // int8 rows followed by one f32 scale per row: linalg.WeightMat's W8A8 form
)
const (
	drawLogits = iota
	drawGreedy
	drawMinP
	drawGumbel
)
const (
	classAuto  = 0
	classExact = 1
)

// modelCfg mirrors b200_model_cfg: 23 int32 then 6 float32, 116 bytes.
type modelCfg struct {
	Hidden, NLayers, NHeads, NKVHeads, HeadDim, FFN, Vocab int32
	RotaryDim                                              int32
	QKNorm                                                 int32
	NExperts, TopK, NormTopK, MoEFFN                       int32
	KVBlockRows, KVPoolBlocks, NSlots, CtxCap, MaxRows     int32
	TPRank, TPSize                                         int32
	KernelClass, FastFloor, KVDtype                        int32
	RMSEps, RopeTheta                                      float32
	AttnScale, AttnSoftcap, FinalSoftcap, EmbedScale       float32
}

// drawC mirrors b200_draw: 24 bytes, u at offset 16. A Gumbel draw carries 1/T in Temperature and its 64-bit seed and draw
// index in the bytes of MinP.._pad and U (the header's note on B200_DRAW_GUMBEL).
type drawC struct {
	Kind        int32
	Temperature float32
	MinP        float32
	Pad         float32
	U           float64
}

// capsC mirrors b200_caps: 8 int32 then 3 int64, 56 bytes.
type capsC struct {
	ContextCap, KVSlots, BatchLo, BatchHi                         int32
	HasFastPrefill, FastPrefillFloor, TailMinRows, BatchGreedyDraw int32
	WeightBytes, KVBytes, ScratchBytes                            int64
}

// statsC mirrors b200_stats_t: 6 int64 then one float64, 56 bytes.
type statsC struct {
	Steps, Rows, PrefillRows, KernelLaunches, KVBlocksInUse, KVPoolFull int64
	LastStepDeviceMs                                                     float64
}

// One variable per symbol of include/b200_resident.h, in the header's order. Pointers into Go slices are passed as
// unsafe.Pointer of the first element; the library reads them during the call only.
var (
	b200Open          func(device int32, stream unsafe.Pointer, out *unsafe.Pointer) int32
	b200Close         func(ctx unsafe.Pointer)
	b200LastError     func(ctx unsafe.Pointer) *byte
	b200TPUniqueID    func(ctx unsafe.Pointer, idOut unsafe.Pointer, bytes uintptr) int32
	b200TPInit        func(ctx unsafe.Pointer, id unsafe.Pointer, bytes uintptr, rank, size int32) int32
	b200TPDestroy     func(ctx unsafe.Pointer) int32
	b200ModelCreate   func(ctx unsafe.Pointer, cfg *modelCfg, out *unsafe.Pointer) int32
	b200UploadTensor  func(m unsafe.Pointer, which, layer, expert, kind, rows, cols int32, host unsafe.Pointer, bytes uintptr) int32
	b200SetRopeInv    func(m unsafe.Pointer, layer int32, invFreq *float64, n int32) int32
	b200ModelFinalize func(m unsafe.Pointer, caps *capsC) int32
	b200ModelFree     func(m unsafe.Pointer)
	b200KVSlots       func(m unsafe.Pointer) int32
	b200ResetSlot     func(m unsafe.Pointer, slot int32) int32
	b200Reset         func(m unsafe.Pointer) int32
	b200BlockTable    func(m unsafe.Pointer, slot int32, out *int32, n int32) int32
	b200UploadKV      func(m unsafe.Pointer, slot, layer, base, n int32, keys, vals *float32) int32
	b200StepRagged    func(m unsafe.Pointer, nSeqs int32, slot, pos, nRows, prefillPromptLen *int32, prefillLast *uint8,
		embs *float32, tokenIDs *int32, draws *drawC, maskIndex *int32, logitMask *uint32, nMasks int32,
		logitsOut *float32, idsOut *int32, nLogitRowsOut *int32) int32
	b200Forward     func(m unsafe.Pointer, slot int32, emb *float32, tokenID, pos, outKind int32, logitsOut *float32, idOut *int32) int32
	b200ForwardTopK func(m unsafe.Pointer, slot int32, emb *float32, tokenID, pos, k int32, invTemperature float32,
		idsOut *int32, logitsOut *float32, zOut *float64) int32
	b200CopyKV      func(m unsafe.Pointer, dstSlot, srcSlot, nRows int32) int32
	b200PrefillLast func(m unsafe.Pointer, slot, n int32, embs *float32, tokenIDs *int32, startPos int32, logitsOut *float32) int32
	b200Stats       func(m unsafe.Pointer, out *statsC) int32
	// the device batch: admission and retirement applied on the device, k steps a call
	b200BatchOpen   func(m unsafe.Pointer, nSeats, firstSlot, parkSlot, maxSteps int32) int32
	b200BatchAdmit  func(m unsafe.Pointer, seat, pos, token, maxNew, eosID int32) int32
	b200BatchRetire func(m unsafe.Pointer, seat int32) int32
	b200BatchRun    func(m unsafe.Pointer, steps int32, eventsOut *int32, maxEvents int32, nEventsOut *int32) int32
	b200BatchClose  func(m unsafe.Pointer) int32
	// operator-level entry points (host buffers in and out): what a kernel test on the Go side calls, the way
	// backend/cuda/kernels/*_test.go call their kernels against host twins
	b200OpQuantG32      func(ctx unsafe.Pointer, x *float32, rows, k int32, codes *int8, scales *float32) int32
	b200OpQ4KDequant    func(ctx unsafe.Pointer, w *byte, rows, cols int32, out *float32) int32
	b200OpQ4KMatmul     func(ctx unsafe.Pointer, w *byte, a *float32, M, K, N, klass int32, dst *float32) int32
	b200OpF16Matmul     func(ctx unsafe.Pointer, w *uint16, a *float32, M, K, N, klass int32, dst *float32) int32
	b200OpQ4KQuantize   func(ctx unsafe.Pointer, w *float32, rows, cols int32, out *byte) int32
	b200OpRMSNorm       func(ctx unsafe.Pointer, x, w *float32, rows, dim int32, eps float32, out *float32) int32
	b200OpRoute         func(ctx unsafe.Pointer, logits *float32, rows, nExperts, k, normTopK int32, idx *int32, weights *float32) int32
	b200OpDraw          func(ctx unsafe.Pointer, logits *float32, rows, vocab int32, draws *drawC, maskIndex *int32, masks *uint32, nMasks int32, ids *int32) int32
	b200OpTopK          func(ctx unsafe.Pointer, logits *float32, rows, vocab, k int32, invTemperature float32, ids *int32, vals *float32, z *float64) int32
	b200OpPhilox        func(ctx unsafe.Pointer, ctr, key *uint32, n int32, out *uint32) int32
	b200OpAttention     func(ctx unsafe.Pointer, q, k, v *float32, nKeys *int32, rows, maxKeys, nHeads, nKVHeads, headDim int32, scale, softcap float32, blockRows, klass int32, out *float32) int32
	b200OpPrefillAttn   func(ctx unsafe.Pointer, q, k, v *float32, rows, pos0, nHeads, nKVHeads, headDim int32, scale, softcap float32, blockRows int32, out *float32) int32
	b200OpGateUpSwiglu  func(ctx unsafe.Pointer, w *byte, x *float32, M, K, F, mode int32, codes *int8, scales *float32) int32
	b200OpKQMatmul      func(ctx unsafe.Pointer, kind int32, w *byte, x *float32, M, K, N int32, dst *float32) int32
	b200AttentionNoAlloc func(ctx unsafe.Pointer, q *float32, ldq, rows, nHeads, nKVHeads, headDim int32, scale, softcap float32,
		rowSlot, rowPos *int32, maxKeys int32, kPool, vPool unsafe.Pointer, table *int32, maxBlocks, blockRows int32, out *float32) int32
)

var (
	loadOnce sync.Once
	loadErr  error
)

// load opens the library once and binds every symbol; a missing symbol panics inside RegisterLibFunc, which is the
// right outcome for a header/library mismatch.
func load() error {
	loadOnce.Do(func() {
		if unsafe.Sizeof(modelCfg{}) != 116 || unsafe.Sizeof(drawC{}) != 24 || unsafe.Offsetof(drawC{}.U) != 16 ||
			unsafe.Sizeof(capsC{}) != 56 || unsafe.Sizeof(statsC{}) != 56 {
			loadErr = errors.New("b200: a struct mirror no longer matches include/b200_resident.h")
			return
		}
		lib, err := purego.Dlopen("libgoinfer_b200.so", purego.RTLD_NOW|purego.RTLD_GLOBAL)
		if err != nil {
			loadErr = fmt.Errorf("b200: %w", err)
			return
		}
		for _, s := range []struct {
			fptr any
			name string
		}{
			{&b200Open, "b200_open"}, {&b200Close, "b200_close"}, {&b200LastError, "b200_last_error"},
			{&b200TPUniqueID, "b200_tp_unique_id"}, {&b200TPInit, "b200_tp_init"}, {&b200TPDestroy, "b200_tp_destroy"},
			{&b200ModelCreate, "b200_model_create"}, {&b200UploadTensor, "b200_upload_tensor"},
			{&b200SetRopeInv, "b200_set_rope_inv_freq"}, {&b200ModelFinalize, "b200_model_finalize"},
			{&b200ModelFree, "b200_model_free"}, {&b200KVSlots, "b200_kv_slots"}, {&b200ResetSlot, "b200_reset_slot"},
			{&b200Reset, "b200_reset"}, {&b200BlockTable, "b200_block_table"}, {&b200UploadKV, "b200_upload_kv"},
			{&b200StepRagged, "b200_step_ragged"}, {&b200Forward, "b200_forward"}, {&b200ForwardTopK, "b200_forward_topk"},
			{&b200CopyKV, "b200_copy_kv"}, {&b200PrefillLast, "b200_prefill_last"}, {&b200Stats, "b200_stats"},
			{&b200BatchOpen, "b200_batch_open"}, {&b200BatchAdmit, "b200_batch_admit"}, {&b200BatchRetire, "b200_batch_retire"},
			{&b200BatchRun, "b200_batch_run"}, {&b200BatchClose, "b200_batch_close"},
			{&b200OpQuantG32, "b200_op_quant_g32"}, {&b200OpQ4KDequant, "b200_op_q4k_dequant"},
			{&b200OpQ4KMatmul, "b200_op_q4k_matmul"}, {&b200OpF16Matmul, "b200_op_f16_matmul"},
			{&b200OpQ4KQuantize, "b200_op_q4k_quantize"}, {&b200OpRMSNorm, "b200_op_rmsnorm"}, {&b200OpRoute, "b200_op_route"},
			{&b200OpDraw, "b200_op_draw"}, {&b200OpTopK, "b200_op_topk"}, {&b200OpPhilox, "b200_op_philox"},
			{&b200OpAttention, "b200_op_attention"}, {&b200OpPrefillAttn, "b200_op_prefill_attention"},
			{&b200OpGateUpSwiglu, "b200_op_gate_up_swiglu"}, {&b200OpKQMatmul, "b200_op_kq_matmul"},
			{&b200AttentionNoAlloc, "b200_attention_noalloc"},
		} {
			purego.RegisterLibFunc(s.fptr, lib, s.name)
		}
	})
	return loadErr
}

// errKVPoolFull is what a step returns when the block pool cannot take the step's new blocks: nothing was written, the
// caller retires or waits and calls again (the contract of decoder/mc3_batch.go:492-498).
var errKVPoolFull = errors.New("b200: kv pool full")

func lastError(ctx unsafe.Pointer) string {
	p := b200LastError(ctx)
	if p == nil {
		return "unknown error"
	}
	n := 0
	for *(*byte)(unsafe.Add(unsafe.Pointer(p), n)) != 0 {
		n++
	}
	return string(unsafe.Slice(p, n))
}

// check turns a status into an error: nil, the pool-full sentinel, or the library's text.
func check(ctx unsafe.Pointer, st int32, what string) error {
	switch st {
	case stOK:
		return nil
	case stKVPoolFull:
		return errKVPoolFull
	default:
		return fmt.Errorf("b200 %s: status %d: %s", what, st, lastError(ctx))
	}
}

func f32p(s []float32) *float32 {
	if len(s) == 0 {
		return nil
	}
	return &s[0]
}

func i32p(s []int32) *int32 {
	if len(s) == 0 {
		return nil
	}
	return &s[0]
}
