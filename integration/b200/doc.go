//go:build b200

// Package b200 binds libgoinfer_b200.so behind goinfer's resident-backend API.
//
// SOURCE ONLY: not compiled here. The image this library is built in has no Go toolchain, so these files have not been
// through `go vet` or `go build`; they are what a goinfer maintainer drops into backend/b200/ (module
// github.com/townsendmerino/goinfer/backend/b200, beside backend/cuda) and builds with `-tags b200`. They are written
// against the reference's own interfaces, cited at each use:
//
//	decoder.RegisterBackend                      decoder/backend.go:97-101
//	decoder.ResidencyBackend.BuildResident       decoder/residency.go:208-210
//	decoder.DeclineResident                      decoder/residency.go:246-249
//	resident.Forward                             decoder/resident/forward.go:5-33
//	resident.BatchSeq/BatchDraw/BatchOut/Ragged* decoder/resident/forward.go:35-84
//	resident.Caps                                decoder/resident/forward.go:119-146
//	resident.SubsystemProvider and the four      decoder/resident/subsystems.go:11-27, decoder/resident_subsystems.go:31-205
//	subsystem interfaces, Noop* defaults         (pattern: backend/cuda/subsystems.go:12-64)
//
// The library is loaded with github.com/ebitengine/purego (no cgo), the way goinfer reaches the CUDA driver already
// (backend/cuda/go.mod). Every entry point of include/b200_resident.h is registered in lib.go; the C structs are
// mirrored field for field, and init() refuses to run if a mirror's size differs from the header's
// (b200_model_cfg 116, b200_draw 24, b200_caps 56, b200_stats_t 56 bytes: the sizes the library's own ABI test pins).
//
// File map:
//
//	lib.go         dlopen, one RegisterLibFunc per symbol, struct mirrors, status -> error
//	backend.go     decoder.RegisterBackend("cuda", ...), BuildResident: BackendView -> b200_model_cfg, tensor upload, finalize
//	resident.go    resident.Forward on the bound slot, the KV slotter, StepBatch / StepRagged, PrefillLast, CopyKV
//	subsystems.go  ResidentSubsystems(): the four wrapper types, pinned to the interfaces at compile time
package b200
