"""The resident admission gate as a pure function, for the part of it this backend meets.

Mirrors decoder/admit.go:35-76 (`Admit`, `admitWhy`, `admitActSafe`) and decoder/residency.go:278-284
(`actGroupResidentDecline`) for a backend that registers under the name the Q4_K gate accepts: which loads may build a
resident on this library at all. It reads facts only (no device, no model). Gates of families this library does not run
(recurrent blocks, the Metal and WebGPU precision policies) are carried as the caller-supplied `Shape` decline: the
arch's own runner-shape verdict, which this function does not recompute.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List


@dataclass
class AdmitFacts:
    Backend: str = "cuda"        # the name the backend registers under
    Residency: bool = True       # the backend implements BuildResident
    QuantLabel: str = "q4k"      # the precision the weights loaded at
    ActGroup: int = 32           # Options.ActQuantGroup (0: per-vector scales)
    ProjsInt4: bool = False      # the resident projections load as the reference's own int4 kind
    Shape: str = ""              # the arch's runner-shape decline ("" when the uniform-layer runner can express it)
    Gates: List[str] = field(default_factory=list)   # capability-gate refusals of a backend that declares its features


@dataclass
class Admission:
    Why: str = ""                # "" when the backend may build; otherwise the first refusal, in the order the load applies them
    Shape: str = ""
    Gates: List[str] = field(default_factory=list)


def act_group_resident_decline(backend: str, act_group: int, quant: str) -> str:
    if act_group == 0 or backend == "cuda" or (backend == "metal" and quant == "q4k"):
        return ""
    return (f"ActQuantGroup {act_group}: {backend}'s resident projections use per-vector activation scales (per-group "
            "scales are implemented by CUDA residency only), so the load runs on the CPU, which honours the group")


def admit_act_safe(f: AdmitFacts) -> bool:
    """Per-32 activation scales over int8-activation projections clear the activation-quantization hazard; the
    reference's int4 kind does not yet. Metal's q4k lane quantizes no activation."""
    if f.Backend == "metal":
        return f.QuantLabel == "q4k"
    return f.ActGroup == 32 and not f.ProjsInt4


def admit(f: AdmitFacts) -> Admission:
    ad = Admission(Shape=f.Shape, Gates=list(f.Gates))
    if not f.Residency:
        ad.Why = "backend does not implement residency (not built in, or the CPU backend)"
    elif f.QuantLabel == "q4k" and f.Backend not in ("cuda", "metal"):
        ad.Why = f"--quant q4k (native Q4_K) has no resident kernel on {f.Backend} yet"
    elif f.Shape:
        ad.Why = "arch is not eligible for the resident decode runner: " + f.Shape
    else:
        ad.Why = act_group_resident_decline(f.Backend, f.ActGroup, f.QuantLabel) or (ad.Gates[0] if ad.Gates else "")
    return ad
