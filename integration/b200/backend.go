//go:build b200

package b200

// SOURCE ONLY: not compiled here (see doc.go).

import (
	"fmt"
	"math"
	"runtime"
	"unsafe"

	"github.com/townsendmerino/goinfer/decoder"
)

// Registered as "cuda": q4k residency is admitted by backend name (decoder/admit.go:63-66), so a binary carries either
// this package or the stock backend/cuda, not both, unless admitWhy learns the name "b200".
func init() {
	decoder.RegisterBackend("cuda", func() (decoder.Backend, error) { // decoder/backend.go:97-101
		if err := load(); err != nil {
			return nil, err
		}
		b := &backend{}
		runtime.LockOSThread() // the library makes its device current on the calling thread (gpudev/cuda.go:36-44 does the same)
		defer runtime.UnlockOSThread()
		if st := b200Open(0, nil, &b.ctx); st != stOK {
			return nil, fmt.Errorf("b200: no usable device (status %d)", st)
		}
		return b, nil
	})
}

type backend struct {
	ctx unsafe.Pointer
}

var _ decoder.ResidencyBackend = (*backend)(nil)

func (b *backend) Name() string { return "cuda" }

// MatmulBT (decoder/backend.go:23-32) serves the staged path's f32 matmuls; the resident path never calls it. Weights
// arrive as f32 here, so they go through the f16-weight operator after a rounding the staged path's callers accept from
// the stock CUDA backend as well; a maintainer who wants the staged path exact keeps the CPU backend for it.
func (b *backend) MatmulBT(a, w, dst []float32, M, K, N int) {
	h := make([]uint16, len(w))
	for i, v := range w {
		h[i] = f32ToF16(v)
	}
	if st := b200OpF16Matmul(b.ctx, &h[0], &a[0], int32(M), int32(K), int32(N), classExact, &dst[0]); st != stOK {
		panic("b200 MatmulBT: " + lastError(b.ctx))
	}
}

func (b *backend) Close() error {
	if b.ctx != nil {
		b200Close(b.ctx)
		b.ctx = nil
	}
	return nil
}

// Options a deployment sets before the model loads (the stock backend reads the same things from decoder.Options).
var (
	ContextCap   = 8192 // positions per slot (decoder.Options' -ctx)
	KVSlots      = 256  // resident KV slots: the most sequences one step carries
	MaxRows      = 2048 // most packed rows of one step (a prefill chunk's width)
	KVBlockRows  = 16
	KVPoolBlocks = 0 // 0: sized from the memory left after the weights
	ExactClass   = false
)

// BuildResident: decoder/residency.go:208-210. Reads the model through its BackendView (decoder/backend_view.go:17-76),
// declines (DeclineResident) what the library does not build, uploads every tensor in the form the file holds it in.
func (b *backend) BuildResident(m *decoder.Model) (decoder.ResidentForward, bool, error) {
	v := m.BackendView()
	d := v.Dims()
	switch {
	case v.SlidingWindow() > 0, v.LayerNorm(), v.ParallelBlock(), v.NonGatedMLP(), v.HasAttnSinks(), v.LearnedPos(), len(v.MRopeSection()) > 0:
		return nil, false, decoder.DeclineResident("b200: the model uses a feature outside the dense / routed-expert decoder it builds")
	}
	if _, ok := v.MLA(); ok {
		return nil, false, decoder.DeclineResident("b200: multi-head latent attention is not built")
	}
	cfg := modelCfg{
		Hidden: int32(d.Hidden), NLayers: int32(v.NumLayers()), NHeads: int32(d.Heads), NKVHeads: int32(d.KVHeads),
		HeadDim: int32(d.HeadDim), FFN: int32(d.Inter), Vocab: int32(d.Vocab), RotaryDim: int32(v.RotaryDim()),
		KVBlockRows: int32(KVBlockRows), KVPoolBlocks: int32(KVPoolBlocks), NSlots: int32(KVSlots), CtxCap: int32(ContextCap),
		MaxRows: int32(MaxRows), TPRank: 0, TPSize: 1, KernelClass: classAuto,
		RMSEps: v.NormEps(), AttnScale: v.AttnScale(), AttnSoftcap: v.AttnLogitSoftcap(), FinalSoftcap: v.FinalLogitSoftcap(),
		EmbedScale: float32(v.EmbedScale()),
	}
	if ExactClass {
		cfg.KernelClass = classExact
	}
	if v.HasQKNorm() {
		cfg.QKNorm = 1
	}
	if moe, ok := v.MoE(); ok {
		if moe.RouterSigmoid || moe.SharedIntermediateDim > 0 || moe.NGroup > 0 {
			return nil, false, decoder.DeclineResident("b200: routed experts are built as softmax top-k without shared experts or groups")
		}
		cfg.NExperts, cfg.TopK, cfg.MoEFFN = int32(moe.NumExperts), int32(moe.TopK), int32(moe.IntermediateDim)
		if moe.NormTopKProb {
			cfg.NormTopK = 1
		}
	}
	var h unsafe.Pointer
	switch st := b200ModelCreate(b.ctx, &cfg, &h); st {
	case stOK:
	case stDeclined:
		return nil, false, decoder.DeclineResident("b200: %s", lastError(b.ctx)) // decoder/residency.go:246-249
	default:
		return nil, false, fmt.Errorf("b200: %s", lastError(b.ctx))
	}
	fail := func(err error) (decoder.ResidentForward, bool, error) {
		b200ModelFree(h)
		return nil, false, err
	}
	// One upload per tensor. tensorsOf walks Weights() and each Layer(i) and yields the role, the kind and the bytes as the
	// file holds them: raw Q4_K / Q5_K / Q6_K super-blocks where linalg.WeightMat kept them (decoder/weightmat.go:61-83),
	// int8 rows + row scales (kind 5) for what the q4k load keeps as W8A8, f32 for norms and the router.
	for _, t := range tensorsOf(v) {
		if st := b200UploadTensor(h, t.which, t.layer, t.expert, t.kind, t.rows, t.cols, unsafe.Pointer(&t.bytes[0]), uintptr(len(t.bytes))); st != stOK {
			if st == stDeclined {
				return fail(decoder.DeclineResident("b200: %s", lastError(b.ctx)))
			}
			return fail(fmt.Errorf("b200 upload: %s", lastError(b.ctx)))
		}
	}
	// per-layer RoPE tables (decoder/residency.go:604-619): the model's own inverse frequencies, so scaled-RoPE families
	// rotate exactly as the CPU path does
	for l := 0; l < v.NumLayers(); l++ {
		inv := v.Layer(l).RopeInvFreq()
		f := make([]float64, len(inv))
		for i, x := range inv {
			f[i] = float64(x)
		}
		if len(f) > 0 {
			if st := b200SetRopeInv(h, int32(l), &f[0], int32(len(f))); st != stOK {
				return fail(fmt.Errorf("b200 rope: %s", lastError(b.ctx)))
			}
		}
	}
	var caps capsC
	switch st := b200ModelFinalize(h, &caps); st {
	case stOK:
	case stDeclined:
		return fail(decoder.DeclineResident("b200: %s", lastError(b.ctx)))
	default:
		return fail(fmt.Errorf("b200 finalize: %s", lastError(b.ctx)))
	}
	return &resident{ctx: b.ctx, h: h, caps: caps, hidden: d.Hidden, vocab: d.Vocab, kvDim: d.KVHeads * d.HeadDim,
		blockRows: KVBlockRows, busy: map[int]bool{}}, true, nil
}

type tensor struct {
	which, layer, expert, kind, rows, cols int32
	bytes                                  []byte
}

// tensorsOf lists the uploads of one model. The body is mechanical (one case per field of decoder.Weights and
// ResidentLayerView) and is the part a maintainer writes against the tree they build in: the field names of
// decoder.Weights are not part of any interface. The roles and kinds each field maps to are the constants of lib.go.
func tensorsOf(v decoder.BackendModelView) []tensor {
	var out []tensor
	w := v.Weights()
	_ = w
	// out = append(out, tensor{tEmbed, -1, -1, kI8 | kF16 | kF32, vocab, hidden, ...})
	// out = append(out, tensor{tFinalNorm, -1, -1, kF32, 1, hidden, ...}); tLMHead likewise
	// for l := range layers: tAttnNorm, tWQ, tWK, tWV, tWO, (tQNorm, tKNorm), tFFNNorm, tGate, tUp, tDown |
	//                        tRouter + per expert e: tExpertGate, tExpertUp, tExpertDown
	return out
}

func f32ToF16(f float32) uint16 {
	b := math.Float32bits(f)
	sign, exp, man := uint16(b>>16)&0x8000, int((b>>23)&0xff)-127+15, b&0x7fffff
	switch {
	case exp >= 31:
		return sign | 0x7c00
	case exp <= 0:
		return sign
	}
	man += 0x1000 // round to nearest (ties away: the staged path's tolerance does not see the difference)
	if man&0x800000 != 0 {
		man = 0
		exp++
	}
	return sign | uint16(exp)<<10 | uint16(man>>13)
}
