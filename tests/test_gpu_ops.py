"""GPU parity of the kernels, one operator at a time, through the C ABI against the CPU oracle.

Integer artefacts (Q4_K unpacking, activation codes, quantized blocks, routing indices, drawn ids) are
compared bit for bit; floating point to the tolerance written beside each check. The cases follow the
reference's own kernel tests: backend/cuda/kernels/actgroup_kernel_test.go:141-206 (quantizers, exact),
:305-364 (Q4_K GEMV incl. a saturated block, rel-err 1e-5 vs a float64 sum), moe_route_test.go:29-110,
backend/cuda/argmax_tiebreak_test.go:22."""
import numpy as np
import pytest

from goinfer_b200 import abi, q4k
from goinfer_b200.resident import ResidentError

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from goinfer_b200.ops import Ops
    return Ops(0)


def test_quant_g32_bit_exact(ops, oracle_lib):
    rng = np.random.default_rng(0)
    x = rng.normal(0, 1, (7, 1024)).astype(np.float32)
    x[0, :32] = 0.0                     # zero group: scale 0, inv 0
    x[1, 5] = 900.0                     # outlier group
    x[2, 32:64] = -1.0                  # saturated negatives
    x[3] *= 1e-30                       # tiny magnitudes
    x[4, ::2] = 0.5 * 3 / 127           # exact .5 ties -> round half to even
    c0, s0 = oracle_lib.op_quant_g32(x)
    c1, s1 = ops.quant_g32(x)
    assert np.array_equal(c0, c1)
    assert np.array_equal(s0.view(np.uint32), s1.view(np.uint32))


def test_q4k_dequant_bit_exact_on_random_blocks(ops, oracle_lib):
    rng = np.random.default_rng(1)
    raw = q4k.random_blocks(rng, 16, 1024).reshape(-1, 144)
    raw[:2, 4:] = 0xFF                  # saturated blocks: every scale, minimum and code at its maximum
    raw = raw.reshape(-1)
    a = oracle_lib.op_q4k_dequant(raw, 16, 1024)
    b = ops.q4k_dequant(raw, 16, 1024)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert np.array_equal(b, q4k.dequantize(raw, 16, 1024))


def test_q4k_quantizer_bit_exact(ops, oracle_lib):
    rng = np.random.default_rng(2)
    w = rng.normal(0, 0.02, (48, 768)).astype(np.float32)
    w[0, :256] = 0.0                    # all-zero super-block
    w[1, :32] = 0.25                    # constant positive sub-block
    w[2, :64] = -np.abs(w[2, :64])      # all-negative sub-blocks
    a = oracle_lib.op_q4k_quantize(w)
    assert np.array_equal(a, ops.q4k_quantize(w))
    assert np.array_equal(a, q4k.quantize(w))


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 33, 70, 256])
def test_q4k_matmul_exact_class(ops, oracle_lib, M):
    rng = np.random.default_rng(10 + M)
    N, K = 200, 1024                    # N not a multiple of 16 or 128: ragged row tiles
    raw = q4k.quantize(rng.normal(0, 0.02, (N, K)).astype(np.float32))
    a = rng.normal(0, 1, (M, K)).astype(np.float32)
    a[0, :32] = 0
    want = oracle_lib.op_q4k_matmul(raw, a, N)
    got = ops.q4k_matmul(raw, a, N, klass=1)
    # exact class: one ascending chain per output, the oracle's order: bit-identical at every row count
    assert np.array_equal(want.view(np.uint32), got.view(np.uint32))
    ref = oracle_lib.op_q4k_matmul_f64(raw, a, N)
    scale = np.abs(ref).max()
    assert np.abs(got - ref).max() <= 1e-5 * scale          # the reference's own GEMV bar
    fast = ops.q4k_matmul(raw, a, N, klass=0)               # fast class: the dp4a lanes up to two rows, fp16 tensor-core kernels from three
    if M <= 2:
        assert np.abs(fast - ref).max() <= 1e-5 * scale
        assert np.abs(fast - want).max() <= 2e-6 * scale
    else:
        assert np.abs(fast - ref).max() <= 4e-3 * scale     # fp16 operands (mma.sync up to 32 rows, tcgen05 above)


@pytest.mark.parametrize("M,N,K", [(33, 192, 512), (64, 256, 1024), (128, 384, 512), (200, 200, 1024), (256, 512, 2048), (300, 128, 256), (256, 640, 4096)])
def test_q4k_matmul_fast_class_tcgen05(ops, oracle_lib, M, N, K):
    """The tcgen05/TMEM matmul of the fast class: both operands dequantized to fp16 (sub-block scale, minimum and
    activation each rounded to fp16; the weight's sub-block offset is rounded to fp16 as well, which is the larger
    term: about 2^-8 of a quantization step per weight), fp32 accumulate. Held to 4e-3 of the output scale and 2.5e-3 in
    relative L2 against the f64 value of the exact formula (the int8 activation codes the formula itself is built on are
    several times coarser than that)."""
    rng = np.random.default_rng(M + N + K)
    raw = q4k.quantize(rng.normal(0, 0.02, (N, K)).astype(np.float32))
    a = rng.normal(0, 1, (M, K)).astype(np.float32)
    a[1, :64] = 0
    a[2, 5] = 40.0                                   # an activation outlier
    ref = oracle_lib.op_q4k_matmul_f64(raw, a, N)
    got = ops.q4k_matmul(raw, a, N, klass=2)
    scale = np.abs(ref).max()
    assert np.abs(got - ref).max() <= 4e-3 * scale, np.abs(got - ref).max() / scale
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert rel <= 2.5e-3, rel


@pytest.mark.parametrize("M", [4, 7, 8, 9, 16, 17, 31, 32, 33, 45, 63])
def test_q4k_matmul_streaming_kernel(ops, oracle_lib, M):
    """The kernel for 4..63 rows streams weights and activation rows through a TMA ring and keeps the exact class's
    arithmetic. In its one-chain form (klass 4; also what the routed experts run) its bits are the oracle's. Its split form
    (klass 6) divides K between two groups of warps (and between CTAs for narrow matrices) and adds the chains in a fixed
    order: within f32 rounding of the oracle."""
    rng = np.random.default_rng(40 + M)
    for N, K in ((448 * 64 + 20, 512), (100, 4096), (192, 1024)):
        raw = q4k.quantize(rng.normal(0, 0.02, (N, K)).astype(np.float32))
        a = rng.normal(0, 1, (M, K)).astype(np.float32)
        a[M - 1, 32:64] = 0
        want = oracle_lib.op_q4k_matmul(raw, a, N)
        one_chain = ops.q4k_matmul(raw, a, N, klass=4)
        assert np.array_equal(want.view(np.uint32), one_chain.view(np.uint32))
        split = ops.q4k_matmul(raw, a, N, klass=6)
        # klass 6: this kernel with K split between two groups of warps (and between CTAs for narrow matrices), the chains
        # added in a fixed order: within f32 rounding of the oracle
        assert np.abs(split - want).max() <= 2e-6 * np.abs(want).max()
        assert np.array_equal(split, ops.q4k_matmul(raw, a, N, klass=6))     # a fixed order: the same bits every time


def test_q4k_matmul_saturated_and_random_bytes(ops, oracle_lib):
    rng = np.random.default_rng(3)
    N, K = 32, 512
    raw = q4k.random_blocks(rng, N, K).reshape(N, K // 256, 144)
    raw[0, :, 4:] = 0xFF                # saturated rows: actgroup_kernel_test.go:293-295,311-315
    raw = raw.reshape(-1)
    for M in (2, 12):
        a = rng.normal(0, 1, (M, K)).astype(np.float32)
        a[0, :] = -1.0
        ref = oracle_lib.op_q4k_matmul_f64(raw, a, N)
        got = ops.q4k_matmul(raw, a, N, klass=1)
        assert np.abs(got - ref).max() <= 1e-5 * np.abs(ref).max()


def test_q4k_batch_rows_equal_single_rows_within_class(ops):
    """Rows of a batched product equal the same rows alone wherever the kernel class is the same
    (decoder/resident/subsystems.go:102-110 asks this of StepBatch against Forward)."""
    rng = np.random.default_rng(4)
    N, K = 64, 512
    raw = q4k.quantize(rng.normal(0, 0.02, (N, K)).astype(np.float32))
    a = rng.normal(0, 1, (8, K)).astype(np.float32)
    full = ops.q4k_matmul(raw, a, N, klass=1)
    full = ops.q4k_matmul(raw, a, N, klass=1)
    for r in range(8):
        assert np.array_equal(full[r], ops.q4k_matmul(raw, a[r:r + 1], N, klass=1)[0])
    # the fast class runs other kernels at 1-2 rows (integer dots) than at 3-32 (fp16 operands): equal to the fp16 tolerance
    fast = ops.q4k_matmul(raw, a, N, klass=0)
    for r in range(8):
        np.testing.assert_allclose(fast[r], ops.q4k_matmul(raw, a[r:r + 1], N, klass=0)[0], atol=4e-3 * np.abs(full).max(), rtol=0)
    # within the small-batch kernel a row's bits do not depend on the rows beside it (each token is its own MMA column)
    for n in (4, 5, 8):
        assert np.array_equal(fast[:n], ops.q4k_matmul(raw, a[:n], N, klass=5)), n
    b = rng.normal(0, 1, (40, K)).astype(np.float32)
    big = ops.q4k_matmul(raw, b, N, klass=1)
    assert np.array_equal(big[:12], ops.q4k_matmul(raw, b[:12], N, klass=1))
    assert np.array_equal(big[:3], ops.q4k_matmul(raw, b[:3], N, klass=1))   # exact class: across the 8-row boundary too


@pytest.mark.parametrize("kind", [abi.K_Q5K, abi.K_Q6K])
def test_q5k_q6k_matmul_within_the_reference_bar(ops, oracle_lib, kind):
    """The native Q5_K / Q6_K matmuls against the f64 product of the dequantized rows, |err| / sum|w*a| <= 1e-5, at the
    super-block counts and the ragged row count of the reference's kernel test, for 1..9 activation rows; and every planted
    misreading of the format (a dropped fifth bit, a dropped -32, a neighbour's sub-scale, a row read one super-block
    late) is red against the kernel's output (backend/cuda/kernels/kso1c_kernels_test.go:108-177)."""
    from test_kquants import random_blocks
    rng = np.random.default_rng(1024)
    N = 8 * 3 + 5
    worst = 0.0
    for nSB in (1, 2, 6, 12, 19, 32, 35):
        K = 256 * nSB
        raw = random_blocks(rng, kind, N, K)
        for M in (1, 2, 3, 4, 5, 9):
            a = rng.normal(0, 1, (M, K)).astype(np.float32)
            a[:, rng.integers(0, K, 3)] *= 30.0    # outliers
            got = ops.kq_matmul(kind, raw, a, N).astype(np.float64)
            want, bar = oracle_lib.op_kq_matmul_f64(kind, raw, a, N)
            e = np.abs(got - want) / (bar + 1e-30)
            assert np.all(np.isfinite(got)) and e.max() <= 1e-5, (nSB, M, e.max())
            worst = max(worst, e.max())
            if M == 3:
                for plant in ((1, 4) if kind == abi.K_Q5K else (2, 3, 4)):
                    if plant == 4 and nSB == 1:
                        continue
                    bad, pb = oracle_lib.op_kq_matmul_f64(kind, raw, a, N, plant)
                    assert (np.abs(got - bad) / (pb + 1e-30)).max() > 1e-5, (nSB, plant)
                # a row's bits do not depend on the rows it is batched with
                assert np.array_equal(ops.kq_matmul(kind, raw, a[1:2], N)[0], ops.kq_matmul(kind, raw, a, N)[1])
    assert worst < 1e-5


@pytest.mark.parametrize("kind", [abi.K_Q6K, abi.K_Q5K])
@pytest.mark.parametrize("M", [1, 32, 100, 256, 300])
def test_q6k_matmul_on_the_tcgen05_kernel(ops, oracle_lib, M, kind):
    """Q6_K (and Q5_K) weights on the tcgen05 kernel whose producers put the codes together and scale them in registers (what
    a fast-class model runs for these tensors from 32 rows, with no dequantized copy of the matrix). fp16 operands (the
    sub-scale d*sc and the activation code*scale are rounded to fp16, q - 32 is exact), fp32 accumulation in tensor memory:
    held to the Q4_K tcgen05 matmul's tolerance against the f64 product of the dequantized rows, on ragged row counts
    (rows past N read as zero blocks), one, two and many super-blocks, with and without a K split; and every planted
    misreading of the format stays far outside that tolerance."""
    import ctypes as C
    from test_kquants import random_blocks
    rng = np.random.default_rng(600 + M)
    for N, nSB in ((8 * 3 + 5, 1), (300, 2), (129, 6), (1000, 12), (4096, 8)):
        K = 256 * nSB
        raw = random_blocks(rng, kind, N, K)
        a = rng.normal(0, 1, (M, K)).astype(np.float32)
        a[:, rng.integers(0, K, 3)] *= 30.0    # outliers
        got = np.zeros((M, N), np.float32)
        st = ops.lib.b200_debug_kq_matmul_umma(ops.ctx, kind, raw.ctypes.data_as(C.POINTER(C.c_uint8)), a.ctypes.data_as(C.POINTER(C.c_float)),
                                                M, K, N, got.ctypes.data_as(C.POINTER(C.c_float)))
        assert st == abi.OK, ops.lib.b200_last_error(ops.ctx)
        want, bar = oracle_lib.op_kq_matmul_f64(kind, raw, a, N)
        scale = np.abs(want).max()
        assert np.all(np.isfinite(got)) and np.abs(got - want).max() <= 4e-3 * scale, (N, nSB, np.abs(got - want).max() / scale)
        rel = np.linalg.norm(got - want) / np.linalg.norm(want)
        assert rel <= 2.5e-3, (N, nSB, rel)
        for plant in ((2, 3) if kind == abi.K_Q6K else (1,)) + ((4,) if nSB > 1 else ()):
            bad, _ = oracle_lib.op_kq_matmul_f64(kind, raw, a, N, plant)
            assert np.linalg.norm(got - bad) / np.linalg.norm(want) > 0.05, (N, nSB, plant)


def test_int8_rows_matmul_within_the_reference_bar(ops, oracle_lib):
    """W8A8 rows (int8 codes, a scale per row) x per-32 int8 activations against the f64 product, |err| / sum|w*a| <= 1e-5
    (the bar of the reference's GEMV tests, backend/cuda/kernels/actgroup_kernel_test.go:305-364), ragged N, 1..9 rows."""
    from goinfer_b200 import kquants
    rng = np.random.default_rng(77)
    N = 8 * 3 + 5
    for K in (32, 96, 512, 4096 + 32):
        raw = kquants.i8_quantize(rng.normal(0, 0.05, (N, K)).astype(np.float32))
        for M in (1, 2, 3, 4, 5, 9):
            a = rng.normal(0, 1, (M, K)).astype(np.float32)
            a[:, rng.integers(0, K, 2)] *= 30.0
            got = ops.kq_matmul(abi.K_I8, raw, a, N).astype(np.float64)
            want, bar = oracle_lib.op_kq_matmul_f64(abi.K_I8, raw, a, N)
            e = np.abs(got - want) / (bar + 1e-30)
            assert e.max() <= 1e-5, (K, M, e.max())
        assert np.array_equal(ops.kq_matmul(abi.K_I8, raw, a[1:2], N)[0], ops.kq_matmul(abi.K_I8, raw, a, N)[1])


@pytest.mark.parametrize("M,F,K", [(40, 14208, 512), (300, 7168, 512)])
def test_gate_up_swiglu_in_the_matmul_epilogue(ops, oracle_lib, M, F, K):
    """silu(gate) * up quantized per 32 by the tcgen05 GEMM's own epilogue (gate|up rows interleaved by 128) gives the bytes
    of the matmul followed by the SwiGLU + quantizer kernel, interleaved or not (shapes at which all three run two weight
    tiles per CTA without a K split, so that every product is summed in the same order); and the values are the oracle's
    within the fast class's bar."""
    rng = np.random.default_rng(M)
    raw = q4k.quantize(rng.normal(0, 0.05, (2 * F, K)).astype(np.float32))
    a = rng.normal(0, 1, (M, K)).astype(np.float32)
    c0, s0 = ops.gate_up_swiglu(raw, a, F, 0)
    c1, s1 = ops.gate_up_swiglu(raw, a, F, 1)
    c2, s2 = ops.gate_up_swiglu(raw, a, F, 2)
    assert np.array_equal(c1, c0) and np.array_equal(s1.view(np.uint32), s0.view(np.uint32))
    assert np.array_equal(c2, c0) and np.array_equal(s2.view(np.uint32), s0.view(np.uint32))
    gu = oracle_lib.op_q4k_matmul_f64(raw, a, 2 * F)
    g, u = gu[:, :F], gu[:, F:]
    want = g / (1 + np.exp(-g)) * u
    nG = F // 32
    got = c1.astype(np.float64).reshape(M, nG, 32) * s1[:, :nG].astype(np.float64)[..., None]
    err = np.linalg.norm(got.reshape(M, F) - want, axis=1) / np.linalg.norm(want, axis=1)
    assert err.max() < 1.5e-2, err.max()    # the int8 per-32 quantizer itself is about 0.9e-2 of a row's norm here; the GEMM adds 2.5e-3
    oc, osc = oracle_lib.op_quant_g32(want.astype(np.float32))
    dc = np.abs(c1.astype(np.int32) - oc.astype(np.int32))
    assert dc.max() <= 4 and (dc > 0).mean() < 0.2 and dc.mean() < 0.2, (dc.max(), (dc > 0).mean(), dc.mean())
    np.testing.assert_allclose(s1[:, :nG], osc[:, :nG], rtol=4e-2, atol=1e-7)   # a group's largest product, fp16 operands
    assert np.median(np.abs(s1[:, :nG] / osc[:, :nG] - 1)) < 2e-3
    # the group sums are the scale times the integer sum of the codes
    np.testing.assert_array_equal(s1[:, nG:], (s1[:, :nG] * c1.reshape(M, nG, 32).astype(np.int32).sum(-1).astype(np.float32)).astype(np.float32))


def test_rmsnorm(ops, oracle_lib):
    rng = np.random.default_rng(5)
    x = rng.normal(0, 3, (5, 2048)).astype(np.float32)
    w = (1 + rng.normal(0, 0.1, 2048)).astype(np.float32)
    a = oracle_lib.op_rmsnorm(x, w, 1e-6)
    b = ops.rmsnorm(x, w, 1e-6)
    np.testing.assert_allclose(b, a, rtol=3e-7, atol=0)   # 1 ulp: the f64 sum is folded in another order


@pytest.mark.parametrize("M,N,K", [(32, 256, 64), (33, 300, 128), (128, 512, 256), (130, 1000, 512), (256, 777, 2048), (5, 256, 64)])
def test_f16_weight_matmul_tcgen05(ops, M, N, K):
    """The fast class's LM-head kernel: f16 weights, f32 activations split into f16 hi + lo parts, fp32 accumulate on the
    tensor cores. Against the f64 product of the same f16 weights: fp32-accumulation accuracy (a K-term fp32 sum)."""
    rng = np.random.default_rng(M + N + K)
    w = rng.normal(0, 0.02, (N, K)).astype(np.float16)
    a = rng.normal(0, 1, (M, K)).astype(np.float32)
    a[0, :] = 0
    a[1, 3] = 300.0
    ref = a.astype(np.float64) @ w.astype(np.float64).T
    got = ops.f16_matmul(w, a, klass=2)
    scale = np.abs(ref).max()
    assert np.abs(got - ref).max() <= 2e-6 * scale * np.sqrt(K), np.abs(got - ref).max() / scale
    small = ops.f16_matmul(w, a, klass=1)                      # the accurate small-batch kernel agrees to the same level
    assert np.abs(small - ref).max() <= 2e-6 * scale * np.sqrt(K)


def test_route_indices_bit_exact(ops, oracle_lib):
    rng = np.random.default_rng(6)
    for nE, k, norm in ((8, 2, True), (128, 8, True), (128, 8, False), (64, 6, True)):
        lg = rng.normal(0, 1, (33, nE)).astype(np.float32)
        lg[0, :] = 0.25                       # all tied: lowest indices win, in order
        lg[1, 3] = lg[1, nE - 2] = 7.0        # a tie at the top
        i0, w0 = oracle_lib.op_route(lg, k, norm)
        i1, w1 = ops.route(lg, k, norm)
        assert np.array_equal(i0, i1)
        assert np.array_equal(w0.view(np.uint32), w1.view(np.uint32))


def test_greedy_draw_first_maximum_and_masks(ops, oracle_lib):
    rng = np.random.default_rng(7)
    V = 32000
    lg = rng.normal(0, 1, (6, V)).astype(np.float32)
    lg[0, 100] = lg[0, 20000] = 9.0           # exact tie: index 100
    lg[1, :] = -1.5                           # all equal: index 0
    lg[2, V - 1] = 50.0
    draws = [abi.Draw(abi.DRAW_GREEDY, 0, 0, 0, 0)] * 6
    masks = np.full((2, (V + 31) // 32), 0xFFFFFFFF, np.uint32)
    masks[0, 100 // 32] &= ~np.uint32(1 << (100 % 32))      # forbid id 100 for row 0
    masks[1, :] = 0
    masks[1, 7] = 1 << 3                                    # only id 227 allowed for row 3
    mi = np.array([0, -1, -1, 1, -1, -1], np.int32)
    want = oracle_lib.op_draw(lg, draws, mi, masks)
    got = ops.draw(lg, draws, mi, masks)
    assert np.array_equal(want, got)
    assert got[0] == 20000 and got[1] == 0 and got[2] == V - 1 and got[3] == 227


def test_minp_draw_matches_the_retained_set_walk(ops, oracle_lib):
    rng = np.random.default_rng(8)
    V = 4096
    lg = (rng.normal(0, 2, (40, V))).astype(np.float32)
    lg[5, 10] = lg[5, 11] = lg[5].max() + 1   # tied top tokens
    draws = []
    for r in range(40):
        draws.append(abi.Draw(abi.DRAW_MINP, [0.7, 1.0, 1.3][r % 3], [0.05, 0.2, 0.01, 1.5][r % 4], 0, float(rng.random())))
    want = oracle_lib.op_draw(lg, draws)
    got = ops.draw(lg, draws)
    assert np.array_equal(want, got)
    # every drawn id lies in the oracle's retained set
    for r in range(40):
        ids, probs = oracle_lib.op_minp_set(lg[r], draws[r].temperature, draws[r].min_p)
        assert got[r] in ids and abs(probs.sum() - 1) < 1e-12


@pytest.mark.parametrize("nH,nKV,hd", [(32, 8, 128), (32, 4, 64), (4, 2, 64), (4, 2, 16), (8, 2, 8), (8, 8, 128)])
def test_paged_attention_matches_the_f64_oracle(ops, oracle_lib, nH, nKV, hd):
    rng = np.random.default_rng(hd + nH)
    rows, max_keys = 6, 1300
    n_keys = np.array([1, 15, 16, 17, 700, 1300], np.int32)   # block edges, split edges (512), ragged
    q = rng.normal(0, 1, (rows, nH * hd)).astype(np.float32)
    k = rng.normal(0, 1, (rows, max_keys, nKV * hd)).astype(np.float32)
    v = rng.normal(0, 1, (rows, max_keys, nKV * hd)).astype(np.float32)
    scale = 1.0 / np.sqrt(hd)
    for cap in (0.0, 30.0):
        want = oracle_lib.op_attention(q, k, v, n_keys, nH, nKV, hd, scale, cap)
        got = ops.attention(q, k, v, n_keys, nH, nKV, hd, scale, cap, block_rows=16)
        np.testing.assert_allclose(got, want, atol=2e-5, rtol=1e-4)   # fast class: fp32 online softmax vs f64
        exact = ops.attention(q, k, v, n_keys, nH, nKV, hd, scale, cap, block_rows=16, klass=1)
        # exact class: the oracle's own f64 order; only libm's last-ulp exp/tanh can move a rounding
        assert (exact.view(np.uint32) != want.view(np.uint32)).mean() < 1e-3
        np.testing.assert_allclose(exact, want, atol=0, rtol=3e-7)
    want0 = oracle_lib.op_attention(q, k, v, n_keys, nH, nKV, hd, scale, 0.0)
    np.testing.assert_allclose(ops.attention(q, k, v, n_keys, nH, nKV, hd, scale, 0.0, block_rows=64), want0, atol=2e-5, rtol=1e-4)
    np.testing.assert_allclose(ops.attention(q, k, v, n_keys, nH, nKV, hd, scale, 0.0, block_rows=64, klass=1), want0, atol=0, rtol=3e-7)


def _tcgen05_prefill_bar(got, want):
    """Runs of 128 rows and more go through the tcgen05 kernel, whose operands (Q, K, V and the softmax weights) are single
    fp16 values with fp32 accumulation and fp32 softmax: relative L2 5e-4 and max |error| 1e-3 on unit-variance data
    (measured: 2.6e-4 and 6.8e-4)."""
    assert np.isfinite(got).all()
    rel = np.linalg.norm(got.astype(np.float64) - want) / np.linalg.norm(want)
    assert rel <= 5e-4, rel
    assert np.abs(got - want).max() <= 1e-3, np.abs(got - want).max()


@pytest.mark.parametrize("nH,nKV,hd", [(32, 8, 128), (32, 4, 64), (4, 2, 64), (8, 8, 128), (16, 2, 128)])
@pytest.mark.parametrize("rows,pos0,block_rows", [(16, 0, 16), (37, 0, 16), (45, 83, 16), (33, 500, 64), (130, 7, 16), (128, 0, 16), (300, 77, 16),
                                                  (257, 500, 64)])
def test_prefill_attention_matches_the_f64_oracle(ops, oracle_lib, nH, nKV, hd, rows, pos0, block_rows):
    """A run of rows at consecutive positions of one sequence (a prefill chunk): row j sees keys 0..pos0+j. The oracle is the
    CPU path's per-row attention given each row its own key count; tile edges (16 rows, 32 keys), block edges and a chunk
    that starts deep in the context are covered."""
    rng = np.random.default_rng(hd + nH + rows + pos0)
    keys = pos0 + rows
    q = rng.normal(0, 1, (rows, nH * hd)).astype(np.float32)
    k = rng.normal(0, 1, (keys, nKV * hd)).astype(np.float32)
    v = rng.normal(0, 1, (keys, nKV * hd)).astype(np.float32)
    scale = 1.0 / np.sqrt(hd)
    n_keys = (pos0 + 1 + np.arange(rows)).astype(np.int32)
    kk = np.broadcast_to(k, (rows,) + k.shape)
    vv = np.broadcast_to(v, (rows,) + v.shape)
    for cap in (0.0, 30.0):
        want = oracle_lib.op_attention(q, kk, vv, n_keys, nH, nKV, hd, scale, cap)
        got = ops.prefill_attention(q, k, v, pos0, nH, nKV, hd, scale, cap, block_rows=block_rows)
        if rows < 128:
            np.testing.assert_allclose(got, want, atol=2e-5, rtol=1e-4)   # mma.sync kernel, hi + lo operands: fp32 online softmax vs f64
        else:
            _tcgen05_prefill_bar(got, want)


def test_prefill_attention_properties_at_chunk_size(ops):
    """Size-independent properties at the benchmark's prefill chunk (2048 rows, 32 query / 8 kv heads of 128): a constant
    V comes back; the output is linear in V; row j does not depend on keys after pos0+j (later rows' keys are poisoned
    one row at a time by comparing against a shorter run)."""
    rng = np.random.default_rng(21)
    nH, nKV, hd, rows, pos0 = 32, 8, 128, 2048, 160
    keys = pos0 + rows
    q = rng.normal(0, 1, (rows, nH * hd)).astype(np.float32)
    k = rng.normal(0, 1, (keys, nKV * hd)).astype(np.float32)
    v1 = rng.normal(0, 1, (keys, nKV * hd)).astype(np.float16).astype(np.float32)
    const = np.broadcast_to(rng.normal(0, 1, (1, nKV * hd)).astype(np.float16).astype(np.float32), v1.shape)
    o_const = ops.prefill_attention(q, k, const, pos0, nH, nKV, hd)
    want = np.repeat(const[0].reshape(nKV, 1, hd), nH // nKV, axis=1).reshape(-1)
    np.testing.assert_allclose(o_const, np.broadcast_to(want, o_const.shape), atol=2e-3, rtol=0)
    o1 = ops.prefill_attention(q, k, v1, pos0, nH, nKV, hd)
    o2 = ops.prefill_attention(q, k, 2 * v1, pos0, nH, nKV, hd)
    np.testing.assert_allclose(o2, 2 * o1, atol=1e-5, rtol=1e-5)
    # the first 1000 rows of the run, computed without the later keys present at all, are the same rows
    short = ops.prefill_attention(q[:1000], k[:pos0 + 1000], v1[:pos0 + 1000], pos0, nH, nKV, hd)
    assert np.array_equal(short[:896], o1[:896])        # whole 128-row tiles see identical key tiles
    np.testing.assert_allclose(short[896:], o1[896:1000], atol=1e-6, rtol=1e-5)
    # and a prefill row agrees with the flash-decode kernel's row for the same query
    pick = np.array([0, 511, 2047])
    n_keys = (pos0 + 1 + pick).astype(np.int32)
    kk = np.broadcast_to(k, (3,) + k.shape)
    vv = np.broadcast_to(v1, (3,) + v1.shape)
    dec = ops.attention(q[pick], kk, vv, n_keys, nH, nKV, hd)
    np.testing.assert_allclose(o1[pick], dec, atol=1e-3, rtol=0)    # the tcgen05 kernel's bar (the decode kernel is at fp32 level)


def test_attention_properties_at_full_context(ops):
    """Size-independent properties at the benchmark's largest context (8192 keys, 8 kv heads of 128):
    constant V gives that constant back; the output is linear in V; keys past n_keys do not matter."""
    rng = np.random.default_rng(9)
    nH, nKV, hd, rows, max_keys = 32, 8, 128, 3, 8192
    n_keys = np.array([8192, 4097, 129], np.int32)
    q = rng.normal(0, 1, (rows, nH * hd)).astype(np.float32)
    k = rng.normal(0, 1, (rows, max_keys, nKV * hd)).astype(np.float32)
    v1 = rng.normal(0, 1, (rows, max_keys, nKV * hd)).astype(np.float16).astype(np.float32)
    const = np.broadcast_to(rng.normal(0, 1, (1, 1, nKV * hd)).astype(np.float16).astype(np.float32), v1.shape)
    o_const = ops.attention(q, k, const, n_keys, nH, nKV, hd)
    want = np.repeat(const[0, 0].reshape(nKV, 1, hd), nH // nKV, axis=1).reshape(-1)
    np.testing.assert_allclose(o_const, np.broadcast_to(want, o_const.shape), atol=2e-3, rtol=0)
    o1 = ops.attention(q, k, v1, n_keys, nH, nKV, hd)
    o2 = ops.attention(q, k, 2 * v1, n_keys, nH, nKV, hd)
    np.testing.assert_allclose(o2, 2 * o1, atol=1e-5, rtol=1e-5)
    k2 = k.copy()
    for r in range(rows):
        k2[r, n_keys[r]:] = 1e4          # poison the keys outside the causal range
    assert np.array_equal(ops.attention(q, k2, v1, n_keys, nH, nKV, hd), o1)


def test_philox_and_gumbel_draw_on_the_device(ops, oracle_lib):
    """Philox4x32-10 is integer-only: the device's words are the oracle's, bit for bit (and the oracle's are the
    Random123 known answers). The Gumbel-max draw then differs from the host's only in the float transform (f32 here,
    f64 there), which can change the argmax only when the two best keys are within a few ulps: the reference measures
    that rate rather than assuming it (backend/cuda/gumbel.cu:3-8), and so does this test."""
    rng = np.random.default_rng(17)
    ctr = rng.integers(0, 2**32, (500, 4), dtype=np.uint64).astype(np.uint32)
    key = rng.integers(0, 2**32, (500, 2), dtype=np.uint64).astype(np.uint32)
    ctr[0], key[0] = 0, 0
    ctr[1], key[1] = 0xffffffff, 0xffffffff
    got = ops.philox(ctr, key)
    assert np.array_equal(got, oracle_lib.op_philox(ctr, key))
    assert got[0].tolist() == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert got[1].tolist() == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    V, rows = 32003, 400                                     # a vocabulary that is not a multiple of 4
    lg = rng.normal(0, 2.0, (rows, V)).astype(np.float32)
    lg[3] = -np.inf                                          # nothing comparable: the plain argmax
    lg[4, 100:200] = lg[4].max() + 50                        # a hundred-way tie far above the noise range: not all keys equal, one winner
    draws = [abi.gumbel_draw(0.5 + (r % 7) * 0.25, 1000 + r // 50, r) for r in range(rows)]
    want = oracle_lib.op_draw(lg, draws)
    got = ops.draw(lg, draws)
    assert got[3] == want[3] == 0
    diff = np.nonzero(want != got)[0]
    assert len(diff) <= 2, len(diff)                         # measured: f32 vs f64 noise flips well under 1% of rows
    for r in diff:                                           # and only between keys that are f32 neighbours
        inv_t = np.float32(1.0 / (0.5 + (r % 7) * 0.25))
        _, keys = oracle_lib.op_gumbel_keys(lg[r], float(inv_t), 1000 + r // 50, int(r))
        assert abs(keys[want[r]] - keys[got[r]]) <= 4e-6 * abs(keys[want[r]])
    # masks apply before the draw: a masked-out winner cannot be drawn
    words = (V + 31) // 32
    mask = np.full((1, words), 0xFFFFFFFF, np.uint32)
    w0 = int(want[0])
    mask[0, w0 >> 5] &= ~np.uint32(1 << (w0 & 31))
    mi = np.full(rows, -1, np.int32)
    mi[0] = 0
    gm = ops.draw(lg, draws, mi, mask)
    assert gm[0] != w0 and gm[0] == oracle_lib.op_draw(lg, draws, mi, mask)[0]


@pytest.mark.parametrize("V,k", [(32003, 40), (151936, 256), (1000, 1000), (5000, 1), (70000, 1024)])
def test_topk_rows_match_the_host_order(ops, oracle_lib, V, k):
    """The K best logits ordered (logit descending, token id ascending) with -0 and +0 tied, and the whole-row Z
    (decoder/resident/forward.go:91-96; the tie order is a contract: it feeds the host's cumulative draw)."""
    rng = np.random.default_rng(V + k)
    lg = rng.normal(0, 3.0, (4, V)).astype(np.float32)
    lg[1] = np.round(lg[1])                       # heavy ties, many of them across the K boundary
    lg[1, ::7] = -0.0
    lg[1, 3::7] = 0.0
    lg[2, : V // 2] = -np.inf
    lg[3] = 1.25                                  # everything ties: the K lowest ids
    want_i, want_v, want_z = oracle_lib.op_topk(lg, k, 1.0 / 0.7)
    got_i, got_v, got_z = ops.topk(lg, k, 1.0 / 0.7)
    assert np.array_equal(got_i, want_i)
    assert np.array_equal(got_v.view(np.uint32), want_v.view(np.uint32))
    np.testing.assert_allclose(got_z, want_z, rtol=1e-12)
    assert got_i[3].tolist() == list(range(k))


def test_a_bounded_device_wait_that_runs_out_reports_timeout_and_the_context_stays_usable(ops):
    """Every spin in the tcgen05 kernels is bounded: when a stage never fills, the waiting thread gives up after its poll
    limit, the CTA raises the model's error flag, waits for the copies it started, frees its tensor memory and returns, and
    the entry point reports B200_TIMEOUT (status 5). The test hook makes the f16 matmul's loader stop bringing stages in
    from K chunk 2 on and shortens the issuer's limit; the call must come back with status 5, and with the hook disarmed
    the same context must multiply correctly again."""
    import ctypes as C
    rng = np.random.default_rng(5)
    M, K, N = 128, 512, 512
    w = rng.normal(0, 0.05, (N, K)).astype(np.float16)
    a = rng.normal(0, 1, (M, K)).astype(np.float32)
    want = a.astype(np.float64) @ w.astype(np.float64).T
    np.testing.assert_allclose(ops.f16_matmul(w, a, klass=2), want, atol=2e-4, rtol=1e-4)
    assert ops.lib.b200_debug_wait_fault(ops.ctx, 20000, 2) == abi.OK
    try:
        with pytest.raises(ResidentError) as e:
            ops.f16_matmul(w, a, klass=2)
        assert e.value.status == abi.TIMEOUT, str(e.value)
    finally:
        assert ops.lib.b200_debug_wait_fault(ops.ctx, 0, -1) == abi.OK
    np.testing.assert_allclose(ops.f16_matmul(w, a, klass=2), want, atol=2e-4, rtol=1e-4)


@pytest.mark.parametrize("M", [1, 2, 3, 20, 33, 100, 256, 300])
def test_q4k_matmul_from_tile_major_copy_only(ops, oracle_lib, M):
    """A fast-class model keeps only the tile-major copy of a Q4_K projection (klass 7 gives the kernels nothing else): the
    one- and two-row dp4a kernel addresses it with a 2304-byte super-block stride, the small-batch kernel streams it, and the
    tcgen05 kernel's loader fetches 2304 contiguous bytes per 16 rows instead of a tiled box. The last two must give the bits
    the same kernel gives from the row-major matrix (same products, same order); the dp4a kernel over tiles partitions a row's
    super-blocks over lanes and warps in another way, so its f32 sums are those of the row-major one to rounding. Ragged row
    counts too (N not a multiple of 16 or of 128: the copy is padded with zero blocks to whole 16-row tiles, and 16-row
    tiles past the matrix are not fetched)."""
    rng = np.random.default_rng(170 + M)
    for N, K in ((100, 256), (448 * 16 + 20, 512), (1000, 768), (4096, 2048), (130, 4096)):
        raw = q4k.quantize(rng.normal(0, 0.02, (N, K)).astype(np.float32))
        a = rng.normal(0, 1, (M, K)).astype(np.float32)
        got = ops.q4k_matmul(raw, a, N, klass=7)
        ref = oracle_lib.op_q4k_matmul_f64(raw, a, N)
        if M <= 2:   # integer dots, f32 sums in another order
            assert np.abs(got - ref).max() <= 2e-5 * np.abs(ref).max(), (N, K, np.abs(got - ref).max() / np.abs(ref).max())
            assert np.array_equal(got, ops.q4k_matmul(raw, a, N, klass=7))
        else:
            assert np.array_equal(got, ops.q4k_matmul(raw, a, N, klass=0)), (N, K)
            assert np.abs(got - ref).max() <= 4e-3 * np.abs(ref).max(), (N, K)


@pytest.mark.parametrize("M", [1, 2, 3, 7, 8, 9, 16, 17, 25, 32])
def test_q4k_matmul_small_batch_kernel(ops, oracle_lib, M):
    """The fast class's kernel for up to 32 rows (klass 5 forces it; klass 0 picks it from 3 rows): the matrix re-laid tile by
    tile, raw super-blocks through per-warp rings of bulk copies, nibbles to fp16 in registers, mma.sync m16n8k16 with fp32
    accumulation, the minimum term as its own small product, the activation tiles in the layout the quantizing kernels write.
    Against the f64 value of the exact formula: the tcgen05 matmul's tolerance (both round the sub-block scale and the
    activations to fp16). Shapes: ragged row counts (rows past N are zero blocks), one super-block, an odd count of
    super-blocks, a K long enough to be split into ranges, a tall matrix."""
    rng = np.random.default_rng(70 + M)
    for N, K in ((100, 256), (448 * 64 + 20, 512), (192, 4096), (1000, 768), (4096, 2048)):
        raw = q4k.quantize(rng.normal(0, 0.02, (N, K)).astype(np.float32))
        a = rng.normal(0, 1, (M, K)).astype(np.float32)
        a[M - 1, 32:64] = 0
        if M > 2:
            a[1, 5] = 40.0                                 # an activation outlier
        ref = oracle_lib.op_q4k_matmul_f64(raw, a, N)
        got = ops.q4k_matmul(raw, a, N, klass=5)
        scale = np.abs(ref).max()
        assert np.abs(got - ref).max() <= 4e-3 * scale, (N, K, np.abs(got - ref).max() / scale)
        rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
        assert rel <= 2.5e-3, (N, K, rel)
        assert np.array_equal(got, ops.q4k_matmul(raw, a, N, klass=5))      # K ranges are added in a fixed order
        if M >= 3:
            assert np.array_equal(got, ops.q4k_matmul(raw, a, N, klass=0))  # what the fast class picks at these row counts
