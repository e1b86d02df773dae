"""ctypes view of include/b200_resident.h: constants, structs and the function table."""
from __future__ import annotations

import ctypes as C

OK, DECLINED, KV_POOL_FULL, BAD_ARGUMENT, CUDA_ERROR, TIMEOUT, NCCL_ERROR = range(7)

T_EMBED, T_FINAL_NORM, T_LM_HEAD, T_ATTN_NORM, T_WQ, T_WK, T_WV, T_WO, T_Q_NORM, T_K_NORM, T_FFN_NORM, \
    T_GATE, T_UP, T_DOWN, T_ROUTER, T_EXP_GATE, T_EXP_UP, T_EXP_DOWN = range(18)
K_F32, K_F16, K_Q4K, K_Q5K, K_Q6K, K_I8 = 0, 1, 2, 3, 4, 5
DRAW_LOGITS, DRAW_GREEDY, DRAW_MINP, DRAW_GUMBEL = 0, 1, 2, 3
CLASS_AUTO, CLASS_EXACT = 0, 1


class ModelCfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "hidden", "n_layers", "n_heads", "n_kv_heads", "head_dim", "ffn", "vocab", "rotary_dim", "qk_norm",
        "n_experts", "top_k", "norm_topk", "moe_ffn", "kv_block_rows", "kv_pool_blocks", "n_slots",
        "ctx_cap", "max_rows", "tp_rank", "tp_size", "kernel_class", "fast_floor", "kv_dtype")] + [(n, C.c_float) for n in (
        "rms_eps", "rope_theta", "attn_scale", "attn_softcap", "final_softcap", "embed_scale")]


class Draw(C.Structure):
    _fields_ = [("kind", C.c_int32), ("temperature", C.c_float), ("min_p", C.c_float), ("_pad", C.c_float),
                ("u", C.c_double)]


def gumbel_draw(temperature: float, seed: int, draw: int) -> "Draw":
    """A B200_DRAW_GUMBEL entry: invT = float32(1/T), the seed in the bytes of {min_p, _pad}, the draw index in those of u."""
    import struct
    d = Draw()
    d.kind = DRAW_GUMBEL
    d.temperature = float(np_float32(1.0 / (temperature if temperature > 0 else 1.0)))
    raw = struct.pack("<Q", seed & 0xFFFFFFFFFFFFFFFF) + struct.pack("<Q", draw & 0xFFFFFFFFFFFFFFFF)
    C.memmove(C.addressof(d) + 8, raw, 16)
    return d


def np_float32(x):
    import numpy as np
    return np.float32(x)


class Caps(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "context_cap", "kv_slots", "batch_lo", "batch_hi", "has_fast_prefill", "fast_prefill_floor",
        "tail_min_rows", "batch_greedy_draw")] + [(n, C.c_int64) for n in (
        "weight_bytes", "kv_bytes", "scratch_bytes")]


class Stats(C.Structure):
    _fields_ = [(n, C.c_int64) for n in (
        "steps", "rows", "prefill_rows", "kernel_launches", "kv_blocks_in_use", "kv_pool_full")] + [
        ("last_step_device_ms", C.c_double)]


# Every symbol include/b200_resident.h declares (the resident backend's boundary); the loader checks each one resolves.
EXPORTS = (
    "b200_open", "b200_close", "b200_last_error", "b200_model_create", "b200_upload_tensor", "b200_set_rope_inv_freq",
    "b200_model_finalize", "b200_model_free", "b200_kv_slots", "b200_reset_slot", "b200_reset", "b200_block_table",
    "b200_upload_kv", "b200_copy_kv", "b200_step_ragged", "b200_forward", "b200_forward_topk", "b200_prefill_last",
    "b200_batch_open", "b200_batch_admit", "b200_batch_retire", "b200_batch_run", "b200_batch_close",
    "b200_stats", "b200_tp_unique_id", "b200_tp_init", "b200_tp_destroy",
    "b200_op_quant_g32", "b200_op_q4k_dequant", "b200_op_q4k_matmul", "b200_op_q4k_quantize", "b200_op_f16_matmul",
    "b200_op_rmsnorm", "b200_op_route", "b200_op_draw", "b200_op_topk", "b200_op_philox", "b200_op_attention",
    "b200_op_prefill_attention", "b200_op_gate_up_swiglu", "b200_op_kq_matmul", "b200_attention_noalloc",
)

# Every symbol include/b200_bench.h declares (measurement, synthetic workloads, test hooks).
BENCH_EXPORTS = (
    "b200_launch_count", "b200_synth_tensor", "b200_synth_kv", "b200_decode_loop_device", "b200_debug_read_hidden",
    "b200_profile", "b200_profile_read", "b200_bench_read", "b200_bench_kq_matmul", "b200_bench_q4k_matmul",
    "b200_bench_f16_matmul", "b200_bench_attention", "b200_bench_prefill_attention", "b200_debug_wait_fault", "b200_tp_fused_active", "b200_bench_tp_reduce", "b200_debug_q6k_matmul_umma", "b200_debug_kq_matmul_umma",
    "b200_debug_tp_reduce_emulated",
)
