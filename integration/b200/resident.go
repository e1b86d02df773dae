//go:build b200

package b200

// SOURCE ONLY: not compiled here (see doc.go).

import (
	"context"
	"math"
	"unsafe"

	"github.com/townsendmerino/goinfer/decoder"
)

// resident is one model on the device. The library names a slot in every call; the reference's Forward methods work on
// "the bound slot" (KVSubsystem.UseKVSlot), so the binding lives here, as one integer.
type resident struct {
	ctx, h        unsafe.Pointer
	caps          capsC
	hidden, vocab int
	kvDim         int          // n_kv_heads * head_dim: the width of one position's K (or V) row
	blockRows     int
	bound         int          // the slot Forward / ForwardN / UploadKV / Reset act on (UseKVSlot)
	busy          map[int]bool // SetKVSlotBusy's marks: kept for KVPool's report, see subsystems.go
}

var _ decoder.ResidentForward = (*resident)(nil)

// ---- resident.Forward (decoder/resident/forward.go:5-33), on the bound slot ----

// Forward: one row at pos, its logits. b200_forward with out_kind 0.
func (r *resident) Forward(embedding []float32, pos int) ([]float32, error) {
	logits := make([]float32, r.vocab)
	st := b200Forward(r.h, int32(r.bound), &embedding[0], -1, int32(pos), 0, &logits[0], nil)
	return logits, check(r.ctx, st, "forward")
}

// ForwardArgmax (DecodeSubsystem): out_kind 1, four bytes come back.
func (r *resident) ForwardArgmax(embedding []float32, pos int) (int, error) {
	var id int32
	st := b200Forward(r.h, int32(r.bound), &embedding[0], -1, int32(pos), 1, nil, &id)
	return int(id), check(r.ctx, st, "forward argmax")
}

// ForwardNoLogits (DecodeSubsystem): out_kind 2, the row's K/V are written and nothing is read back.
func (r *resident) ForwardNoLogits(embedding []float32, pos int) error {
	return check(r.ctx, b200Forward(r.h, int32(r.bound), &embedding[0], -1, int32(pos), 2, nil, nil), "forward (no logits)")
}

// ForwardSample (DecodeSubsystem): a one-row step whose draw is the Gumbel kind. The id is the one the host's Philox
// stream gives for (seed, draw) on the same logits (internal/runtime/sampling/sampler_gumbel.go:37-64).
func (r *resident) ForwardSample(embedding []float32, pos int, temperature float64, seed, draw uint64) (int, error) {
	out, err := r.StepBatch([]decoder.ResidentBatchSeq{{Slot: r.bound, Pos: pos, Emb: embedding,
		Draw: &decoder.ResidentBatchDraw{Temperature: temperature, Seed: seed, Draw: draw}}})
	if err != nil {
		return 0, err
	}
	return out[0].ID, nil
}

// ForwardN: K rows at startPos.. on the bound slot, every row's logits: one ragged step with one sequence of K rows and
// no draw. In the exact kernel class a row's bits do not depend on how many rows ran beside it, which is what
// TestResidentForwardN_parity asks; in the fast class the rows are within the class's tolerance of K Forward calls, and
// Caps reports HasFastPrefill so the decoder does not mix them with rows it expects to be bit-equal.
func (r *resident) ForwardN(embeddings [][]float32, startPos int) ([][]float32, error) {
	if len(embeddings) == 0 {
		return nil, nil
	}
	out, err := r.StepRagged([]decoder.ResidentRaggedSeq{{Slot: r.bound, Pos: startPos, Embs: embeddings}})
	if err != nil {
		return nil, err
	}
	return out[0].Logits, nil
}

// ForwardTopK (DecodeSubsystem): b200_forward_topk; the ids and logits arrive in the host sampler's order.
func (r *resident) ForwardTopK(embedding []float32, pos, k int, temperature float64, wantZ bool) (decoder.TopKRow, error) {
	row := decoder.TopKRow{IDs: make([]int32, k), Logits: make([]float32, k)}
	var zp *float64
	if wantZ {
		zp = &row.Z
	}
	invT := float32(1)
	if temperature > 0 {
		invT = float32(1 / temperature)
	}
	st := b200ForwardTopK(r.h, int32(r.bound), &embedding[0], -1, int32(pos), int32(k), invT, &row.IDs[0], &row.Logits[0], zp)
	if err := check(r.ctx, st, "forward top-k"); err != nil {
		return decoder.TopKRow{}, err
	}
	bound := r.bound
	row.Full = func() ([]float32, error) { // the same position again, whole row (valid until the next forward)
		logits := make([]float32, r.vocab)
		st := b200Forward(r.h, int32(bound), &embedding[0], -1, int32(pos), 0, &logits[0], nil)
		return logits, check(r.ctx, st, "forward (full row)")
	}
	return row, nil
}

// UploadKV: rows [base, base+n) of one layer of the bound slot, f32 in, the cache's fp16 on the device.
func (r *resident) UploadKV(layer, base int, keys, vals []float32) error {
	n := len(keys) / r.kvDim
	return check(r.ctx, b200UploadKV(r.h, int32(r.bound), int32(layer), int32(base), int32(n), &keys[0], &vals[0]), "upload kv")
}

// TruncateTo is the no-op the interface describes: every call names its position, rows past it are never read and are
// overwritten by the next write at that position; blocks stay mapped to the slot until Reset.
func (r *resident) TruncateTo(pos int) {}

// Reset: the bound slot's blocks go back to the pool (b200_reset_slot).
func (r *resident) Reset() { _ = b200ResetSlot(r.h, int32(r.bound)) }

func (r *resident) Close() error {
	if r.h != nil {
		b200ModelFree(r.h)
		r.h = nil
	}
	return nil
}

// ---- the step (decoder/resident/subsystems.go:102-117; existing implementation backend/cuda/batchstep.go:49-182) ----

func (r *resident) BatchStepRange() (lo, hi int) { return int(r.caps.BatchLo), int(r.caps.BatchHi) }

// StepBatch is StepRagged with one row per sequence.
func (r *resident) StepBatch(seqs []decoder.ResidentBatchSeq) ([]decoder.ResidentBatchOut, error) {
	rs := make([]decoder.ResidentRaggedSeq, len(seqs))
	for i, s := range seqs {
		rs[i] = decoder.ResidentRaggedSeq{Slot: s.Slot, Pos: s.Pos, Embs: [][]float32{s.Emb}, Draw: s.Draw}
	}
	ro, err := r.StepRagged(rs)
	if err != nil {
		return nil, err
	}
	out := make([]decoder.ResidentBatchOut, len(seqs))
	for i := range ro {
		out[i].ID = ro[i].ID
		if ro[i].ID < 0 {
			out[i].Logits = ro[i].Logits[0]
		}
	}
	return out, nil
}

// StepRagged: one call into the library. The step descriptor is three ints per sequence; block tables, row maps and KV
// block allocation are built on the device from it (the per-step table uploads of backend/cuda/batchstep.go:306-381 have
// no counterpart here).
func (r *resident) StepRagged(seqs []decoder.ResidentRaggedSeq) ([]decoder.ResidentRaggedOut, error) {
	n := len(seqs)
	slot, pos, nRows, plen := make([]int32, n), make([]int32, n), make([]int32, n), make([]int32, n)
	plast, draws := make([]uint8, n), make([]drawC, n)
	rows, logitRows := 0, 0
	for i, s := range seqs {
		slot[i], pos[i], nRows[i] = int32(s.Slot), int32(s.Pos), int32(len(s.Embs))
		rows += len(s.Embs)
		switch {
		case s.Prefill != nil:
			plen[i] = int32(s.Prefill.PromptLen)
			if s.Prefill.Last {
				plast[i] = 1
				logitRows++
			}
		case s.Draw != nil:
			draws[i] = drawOf(s.Draw)
			logitRows += len(s.Embs) - 1
		default:
			logitRows += len(s.Embs)
		}
	}
	embs := make([]float32, 0, rows*r.hidden)
	for _, s := range seqs {
		for _, e := range s.Embs {
			embs = append(embs, e...)
		}
	}
	logits := make([]float32, maxInt(1, logitRows)*r.vocab)
	ids := make([]int32, n)
	var nOut int32
	st := b200StepRagged(r.h, int32(n), &slot[0], &pos[0], &nRows[0], &plen[0], &plast[0], &embs[0], nil, &draws[0], nil, nil, 0,
		&logits[0], &ids[0], &nOut)
	if err := check(r.ctx, st, "step"); err != nil {
		if err == errKVPoolFull {
			return nil, decoder.ErrKVPoolFull // decoder/mc3_batch.go:492-498: nothing was written, the coalescer retires or waits
		}
		return nil, err
	}
	// unpack: logits rows arrive packed in sequence order
	out := make([]decoder.ResidentRaggedOut, n)
	at := 0
	take := func() []float32 { row := logits[at*r.vocab : (at+1)*r.vocab : (at+1)*r.vocab]; at++; return row }
	for i, s := range seqs {
		out[i].ID = int(ids[i])
		out[i].Logits = make([][]float32, len(s.Embs))
		switch {
		case s.Prefill != nil:
			if s.Prefill.Last {
				out[i].Logits[len(s.Embs)-1] = take()
			}
		case s.Draw != nil:
			for j := 0; j < len(s.Embs)-1; j++ {
				out[i].Logits[j] = take()
			}
		default:
			for j := range s.Embs {
				out[i].Logits[j] = take()
			}
		}
	}
	return out, nil
}

// drawOf maps resident.BatchDraw (decoder/resident/forward.go:43-52) onto b200_draw: Greedy -> the first maximal index;
// a temperature-only draw -> the Gumbel kind, with invT as the host sampler computes it and the 64-bit seed and draw index
// in the struct's spare bytes.
func drawOf(d *decoder.ResidentBatchDraw) drawC {
	if d.Greedy {
		return drawC{Kind: drawGreedy}
	}
	c := drawC{Kind: drawGumbel, Temperature: float32(1 / d.Temperature)}
	*(*uint64)(unsafe.Pointer(&c.MinP)) = d.Seed // the 8 bytes of {min_p, _pad}
	c.U = math.Float64frombits(d.Draw)           // the 8 bytes of u
	return c
}

// ---- PrefillSubsystem.PrefillLast: n rows from startPos on the bound slot, the last row's logits ----

func (r *resident) PrefillLast(ctx context.Context, embeddings [][]float32, startPos int) ([]float32, error) {
	n := len(embeddings)
	embs := make([]float32, 0, n*r.hidden)
	for _, e := range embeddings {
		embs = append(embs, e...)
	}
	logits := make([]float32, r.vocab)
	// the library cuts the rows into passes of at most max_rows itself and runs every pass in the class the whole prompt takes
	st := b200PrefillLast(r.h, int32(r.bound), int32(n), &embs[0], nil, int32(startPos), &logits[0])
	return logits, check(r.ctx, st, "prefill")
}

// ---- KVSubsystem ----

func (r *resident) KVSlots() int { return int(b200KVSlots(r.h)) }

// UseKVSlot binds the slot the Forward methods act on. Nothing is encoded against a slot between calls (every library
// call completes before it returns), so there is nothing to flush.
func (r *resident) UseKVSlot(i int) error {
	if i < 0 || i >= r.KVSlots() {
		return decoder.DeclineResident("b200: slot %d of %d", i, r.KVSlots())
	}
	r.bound = i
	return nil
}

// CopyKV (KVCopierAvailable): the first n rows of src become dst's (whole blocks shared by reference, copy on write).
func (r *resident) CopyKV(dst, src, base, n int) error {
	if base != 0 {
		return decoder.DeclineResident("b200: a copy starts at row 0")
	}
	return check(r.ctx, b200CopyKV(r.h, int32(dst), int32(src), int32(n)), "copy kv")
}

func maxInt(a, b int) int {
	if a > b {
		return a
	}
	return b
}
