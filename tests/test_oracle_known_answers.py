"""Pins the CPU oracle to the known answers held by the reference's own unit tests.

Each test names the reference test it restates (paths inside the aiis-clef tree). These run on
the CPU and must pass before the oracle is trusted as the checker for the CUDA path.
"""
import numpy as np
import pytest

from oracle import binding as orc
from util import lcg_stream, to_bf16_bits

E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


# ---- src/dequant.rs:102-131, src/model/gemm_ref.rs:141-150 ------------------------------------------------
def test_nibble_order_is_low_first():
    packed = np.zeros(8, np.uint8)
    packed[0] = 0x01
    got = orc.dequantise(packed, np.array([1.0], np.float32), 1.0, 16, 1)
    assert got.size == 16
    assert got[0] == 0.5 and got[1] == 0.0          # dequant.rs:105-111


def test_scales_apply_per_block():
    values = np.zeros(16, np.uint8)
    values[0] = 0x02
    values[8] = 0x02
    got = orc.dequantise(values, np.array([2.0, 3.0], np.float32), 1.0, 32, 1)
    assert got[0] == 2.0 and got[16] == 3.0         # dequant.rs:114-123


def test_sign_bit_and_table():
    # dequant.rs:125-131 (decode(0x9) = -0.5, 0x1 = 0.5, 0x0 = 0, 0x7 = 6) and gemm_ref.rs:141-150.
    def decode(code):
        return orc.dequantise(np.array([code] + [0] * 7, np.uint8), np.array([1.0], np.float32), 1.0, 16, 1)[0]
    assert decode(0x9) == -0.5 and decode(0x1) == 0.5 and decode(0x0) == 0.0 and decode(0x7) == 6.0
    for code, mag in enumerate(E2M1):
        assert decode(code) == mag
        assert decode(code | 8) == -mag
    low, high = orc.dequantise(np.array([0x21] + [0] * 7, np.uint8), np.array([1.0], np.float32), 1.0, 16, 1)[:2]
    assert (low, high) == (0.5, 1.0)                # unpack_nibbles(0x21) == (0.5, 1.0)
    low, high = orc.dequantise(np.array([0x71] + [0] * 7, np.uint8), np.array([1.0], np.float32), 1.0, 16, 1)[:2]
    assert (low, high) == (0.5, 6.0)


def test_global_scale_divides():
    # gemm_ref.rs:190-203
    packed = np.array([0x02, 0, 0, 0, 0, 0, 0, 0], np.uint8)
    assert orc.dequantise(packed, np.array([1.0], np.float32), 1.0, 16, 1)[0] == 1.0
    assert orc.dequantise(packed, np.array([1.0], np.float32), 2.0, 16, 1)[0] == 0.5


# ---- src/model/gemm_ref.rs:152-163, src/cuda/mod.rs:5638-5640 ------------------------------------------------
def test_e4m3_decode_points():
    assert orc.e4m3_one(0x38) == 1.0
    assert orc.e4m3_one(0x40) == 2.0
    assert orc.e4m3_one(0x30) == 0.5
    assert orc.e4m3_one(0xB8) == -1.0
    assert orc.e4m3_one(0x00) == 0.0
    assert orc.from_e4m3(0x38) == 1.0 and orc.to_e4m3(1.0) == 0x38     # the unit scale byte
    for b in range(0x7F):
        assert orc.from_e4m3(b) == orc.e4m3_one(b)                       # both decoders agree on positives


def test_e4m3_encode_rules():
    # kernels/nvfp4_quant.h:35-57: zero/negative/NaN -> 0, round half up, clamp 0x7E, subnormal rule.
    assert orc.to_e4m3(0.0) == 0 and orc.to_e4m3(-1.0) == 0 and orc.to_e4m3(float("nan")) == 0
    assert orc.to_e4m3(448.0) == 0x7E and orc.to_e4m3(1e9) == 0x7E and orc.to_e4m3(464.0) == 0x7E
    assert orc.to_e4m3(1.0625) == 0x39          # exactly half way between 1.0 and 1.125 rounds UP
    assert orc.to_e4m3(1.0624999) == 0x38
    assert orc.to_e4m3(1.96875) == 0x40         # mantissa rounds to 8 -> next exponent
    assert orc.to_e4m3(2.0 ** -9) == 1 and orc.to_e4m3(2.0 ** -10) == 1 and orc.to_e4m3(0.99 * 2.0 ** -10) == 0
    assert orc.to_e4m3(7.4 / 512) == 7 and orc.to_e4m3(7.6 / 512) == 7   # the cap at 7 below the normal range
    assert orc.to_e4m3(2.0 ** -6) == 0x08
    # every code decodes and re-encodes to itself
    for b in range(0x7F):
        assert orc.to_e4m3(orc.from_e4m3(b)) == b


def test_e2m1_ties_go_down_and_sign_rule():
    # kernels/nvfp4_quant.h:13-33 (first minimum with a strict '<'; sign = v < 0)
    assert [orc.to_e2m1(v) for v in E2M1] == list(range(8))
    ties = {0.25: 0, 0.75: 1, 1.25: 2, 1.75: 3, 2.5: 4, 3.5: 5, 5.0: 6}
    for v, code in ties.items():
        assert orc.to_e2m1(v) == code
        assert orc.to_e2m1(np.nextafter(np.float32(v), np.float32(10))) == code + 1
        assert orc.to_e2m1(-v) == (code | 8)
    assert orc.to_e2m1(-0.0) == 0 and orc.to_e2m1(-1e-30) == 8
    assert orc.to_e2m1(7.0) == 7 and orc.to_e2m1(1e6) == 7 and orc.to_e2m1(2.0 ** 24 - 1) == 7
    # far above the table the rounded differences coincide and the first entry wins
    assert orc.to_e2m1(1e29) == 0
    assert orc.to_e2m1(1e30) == 0 and orc.to_e2m1(float("inf")) == 0 and orc.to_e2m1(float("-inf")) == 8
    assert orc.to_e2m1(float("nan")) == 0


# ---- src/swizzle.rs:143-322, 372-396 ------------------------------------------------------------------------
def ramp(n):
    return (np.arange(n) % 251).astype(np.uint8)


@pytest.mark.parametrize("rows,cols", [(128, 4), (256, 8), (4096, 256), (12288, 256), (130, 6)])
def test_swizzle_round_trip(rows, cols):
    src = ramp(rows * cols)
    sw = orc.swizzle_tiled(src, rows, cols, 128, False)
    assert sw.size == orc.swizzled_len_tiled(rows, cols, 128)
    assert np.array_equal(orc.unswizzle_tiled(sw, rows, cols, 128, False), src)
    cf = orc.swizzle_tiled(src, rows, cols, 128, True)
    assert np.array_equal(orc.unswizzle_tiled(cf, rows, cols, 128, True), src)


def test_first_tile_arrangement():
    rows, cols = 128, 4
    src = np.arange(rows * cols).astype(np.uint8)
    sw = orc.swizzle_tiled(src, rows, cols, 128, False)
    for m3 in range(32):
        for m2 in range(4):
            for k2 in range(4):
                assert sw[m3 * 16 + m2 * 4 + k2] == ((m2 * 32 + m3) * 4 + k2) % 256


def test_conflict_free_tile_arrangement():
    rows, cols = 128, 4
    src = np.arange(rows * cols).astype(np.uint8)
    sw = orc.swizzle_tiled(src, rows, cols, 128, True)
    for m in range(128):
        for k2 in range(4):
            assert sw[m * 4 + k2] == (m * 4 + k2) % 256
    assert sw[4] != sw[16]


def test_padding_is_zero():
    rows, cols = 129, 5
    src = ramp(rows * cols)
    sw = orc.swizzle_tiled(src, rows, cols, 128, False)
    assert sw.size == 256 * 8
    assert np.array_equal(orc.unswizzle_tiled(sw, rows, cols, 128, False), src)
    real = set()
    for m in range(rows):
        m1, m2, m3 = m // 128, (m % 128) // 32, m % 32
        for k in range(cols):
            real.add(((m1 * 2 + k // 4) * 32 + m3) * 16 + m2 * 4 + k % 4)
    for i, b in enumerate(sw):
        if i not in real:
            assert b == 0


def test_aligned_matrix_is_not_padded():
    assert orc.swizzled_len_tiled(128, 4, 128) == 128 * 4
    assert orc.swizzled_len_tiled(4096, 256, 128) == 4096 * 256
    assert orc.swizzled_len_tiled(129, 256, 128) == 256 * 256


def test_96_row_atom():
    assert orc.blk_mn_for_tile_m(192) == 96 and orc.blk_mn_for_tile_m(128) == 128 and orc.blk_mn_for_tile_m(64) == 128
    assert orc.swizzled_index_of(0, 0, 256, 192, False) == 0
    assert orc.swizzled_index_of(0, 4, 256, 192, False) == 384
    assert orc.swizzled_index_of(96, 0, 256, 192, False) == (256 // 4) * 384
    assert orc.swizzled_len_tiled(768, 256, 192) == 768 * 256


@pytest.mark.parametrize("rows,cols", [(128, 4), (256, 8), (12288, 256), (4096, 768)])
def test_gemm_index_matches_swizzle(rows, cols):
    compact = ramp(rows * cols)
    for cf in (False, True):
        sw = orc.swizzle_tiled(compact, rows, cols, 128, cf)
        for row in range(0, rows, rows // 8 + 1):
            for block in range(0, cols, cols // 8 + 1):
                assert sw[orc.swizzled_index_of(row, block, cols, 128, cf)] == compact[row * cols + block]


# ---- src/model/norm.rs:69-121 ------------------------------------------------------------------------------
def test_norm_conventions():
    x = np.full(4, 3.0, np.float32)
    assert np.allclose(orc.model_rms_norm(np.ones(4, np.float32), np.zeros(4, np.float32), 0.0), 1.0, atol=1e-6)
    assert abs(orc.model_rms_norm(x, np.zeros(4, np.float32), 0.0)[0] - 1.0) < 1e-6
    assert abs(orc.model_rms_norm(x, np.full(4, 2.0, np.float32), 0.0)[0] - 3.0) < 1e-6      # (1 + w)
    w = np.full(4, 0.5, np.float32)
    assert abs(orc.model_rms_norm(x, w, 0.0)[0] - 1.5) < 1e-6
    assert abs(orc.model_rms_norm_gated(x, np.zeros(4, np.float32), w, 0.0)[0]) < 1e-9       # silu(0) = 0
    got = orc.model_rms_norm_gated(x, np.full(4, 2.0, np.float32), np.ones(4, np.float32), 0.0)[0]
    silu2 = 2.0 / (1.0 + np.exp(-2.0))
    assert abs(got - silu2) < 1e-5 and abs(got - 1.0) > 1e-3
    # the kernel-order restatement follows the same conventions (plain weight in the gated norm)
    f32, _ = orc.rms_norm(x[None], np.full(4, 2.0, np.float32), 1, 4, 0.0)
    assert abs(f32[0, 0] - 3.0) < 1e-6
    f32, _ = orc.rms_norm_gated(x[None], np.full((1, 4), 2.0, np.float32), np.ones(4, np.float32), 1, 4, 0.0)
    assert abs(f32[0, 0] - silu2) < 1e-5


# ---- src/model/attention.rs:263-297 ----------------------------------------------------------------------------
def test_rope_identity_norm_and_tail():
    cos, sin = orc.rope_tables([0], 64, 1e7)
    v = (np.arange(64) * 0.1).astype(np.float32)
    assert np.abs(orc.model_apply_rope(v, cos[0], sin[0]) - v).max() < 1e-6
    cos, sin = orc.rope_tables([7], 64, 1e7)
    v = np.sin(np.arange(64) * 0.37).astype(np.float32)
    after = orc.model_apply_rope(v, cos[0], sin[0])
    assert abs(np.linalg.norm(v) - np.linalg.norm(after)) < 1e-4
    cos, sin = orc.rope_tables([3], 64, 1e7)
    x = np.arange(256, dtype=np.float32)[None, None, :]
    f32, _ = orc.rope(x, cos, sin, 1, 1, 256, 64, pos_map=np.array([0], np.int32))
    assert np.array_equal(f32[0, 0, 64:], x[0, 0, 64:])          # pass-through region untouched
    # kernel formula == rotate-half formula of the model (src/cuda/mod.rs:7398-7421)
    want = orc.model_apply_rope(x[0, 0, :64], cos[0], sin[0])
    assert np.abs(f32[0, 0, :64] - want).max() < 1e-4


# ---- src/cuda/mod.rs:7310-7423 the_elementwise_kernels_match_the_cpu_oracle ------------------------------------
def test_kernel_order_restatement_matches_the_f64_model():
    rows, cols = 5, 128
    i = np.arange(rows * cols)
    x = (((i * 37 % 101).astype(np.float32) - 50.0) / 11.0).reshape(rows, cols)
    w_plain = ((np.arange(cols) % 7).astype(np.float32) - 3.0) / 8.0
    w_gated = 0.5 + (np.arange(cols) % 5).astype(np.float32) / 4.0
    gate = (((i * 13 % 61).astype(np.float32) - 30.0) / 9.0).reshape(rows, cols)
    up = (((i * 29 % 71).astype(np.float32) - 35.0) / 7.0).reshape(rows, cols)
    got, _ = orc.rms_norm(x, w_plain, rows, cols, 1e-6)
    want = np.stack([orc.model_rms_norm(x[r], w_plain, 1e-6) for r in range(rows)])
    assert np.abs(got - want).max() < 1e-4
    got, _ = orc.rms_norm_gated(x, gate, w_gated, rows, cols, 1e-6)
    want = np.stack([orc.model_rms_norm_gated(x[r], gate[r], w_gated, 1e-6) for r in range(rows)])
    assert np.abs(got - want).max() < 1e-4
    got, _ = orc.swiglu(gate, up)
    want = gate / (1.0 + np.exp(-gate.astype(np.float64))) * up
    assert np.abs(got - want).max() < 1e-5


# ---- src/cuda/mod.rs:7571-7653 the_quantiser_round_trips_through_the_cpu_dequantiser ------------------------------
def test_quantiser_round_trip_bounds():
    rows, cols = 7, 12288
    i = np.arange(rows * cols)
    block = i // 16
    within = (i % 16).astype(np.float32) / np.float32(15.0)
    base = np.float32(2.0) + (block % 5).astype(np.float32)
    x = (base * (np.float32(0.5) + within)) * np.where(i % 2 == 0, np.float32(1.0), np.float32(-1.0))
    x = x.astype(np.float32)
    amax = np.abs(x).max()
    global_scale = float(np.float32(448.0) / (amax / np.float32(6.0)))
    packed, scales = orc.quantise_nvfp4(x.reshape(rows, cols), rows, cols, global_scale)
    assert packed.size == 128 * (cols // 2) and scales.size == 128 * (cols // 16)
    compact = orc.unswizzle_tiled(scales, 128, cols // 16, 128, True)
    scale_f32 = np.array([orc.e4m3_one(int(b)) for b in compact[: rows * (cols // 16)]], np.float32)
    got = orc.dequantise(packed, scale_f32, global_scale, cols, rows)
    scale_of = np.abs(x).mean()
    err = np.abs(got - x)
    big = np.abs(x) > scale_of / 8.0
    assert (err[big] / np.abs(x[big])).max() < 0.25
    max_block_scale = (np.abs(x).reshape(-1, 16).max(axis=1) / 6.0).max()
    assert err.max() <= max_block_scale + 1e-3
    # pad rows and pad scales are zero
    assert not packed[rows * (cols // 2):].any()
    assert not np.delete(compact, np.s_[: rows * (cols // 16)]).any()
    # a zero row gives zero codes and zero scales
    p0, s0 = orc.quantise_nvfp4(np.zeros((1, 64), np.float32), 1, 64, global_scale)
    assert not p0.any() and not s0.any()


# ---- fused == chain (src/cuda/mod.rs:6866-6917, 8133-8202) on the CPU restatement ---------------------------------
def test_fused_restatements_equal_their_chains():
    cols, vh, tokens = 128, 32, 7
    rows = tokens * vh
    seq = lcg_stream(0x9E3779B9 ^ tokens, 2 * rows * cols + cols) * np.float32(1.1)
    x = seq[: rows * cols].reshape(rows, cols)
    g = seq[rows * cols: 2 * rows * cols].reshape(rows, cols)
    w = np.float32(0.5) + seq[2 * rows * cols:] * np.float32(0.1)
    gs = float(np.float32(1.0 / 12.5))
    gated, _ = orc.rms_norm_gated(x, g, w, rows, cols, 1e-6)
    pc, sc = orc.quantise_nvfp4(gated.reshape(tokens, vh * cols), tokens, vh * cols, gs)
    pf, sf = orc.rms_norm_gated_quantise_nvfp4(x, g, w, rows, cols, vh, 1e-6, gs)
    assert np.array_equal(pf, pc) and np.array_equal(sf, sc)

    rows, cols = 5, 12288
    seq = lcg_stream(0x511161, 2 * rows * cols) * np.float32(0.05)
    gate, up = seq[: rows * cols].reshape(rows, cols), seq[rows * cols:].reshape(rows, cols)
    act, _ = orc.swiglu(gate, up)
    pc, sc = orc.quantise_nvfp4(act, rows, cols, 215.0)
    pf, sf = orc.swiglu_quantise_nvfp4(gate, up, rows, cols, 215.0)
    assert np.array_equal(pf, pc) and np.array_equal(sf, sc)

    rows, cols = 9, 2048
    rng = np.random.default_rng(3)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    w = (rng.standard_normal(cols) * 0.1).astype(np.float32)
    normed, _ = orc.rms_norm(x, w, rows, cols, 1e-6)
    pc, sc = orc.quantise_nvfp4(normed, rows, cols, 64.0)
    pf, sf = orc.rms_norm_quantise_nvfp4(x, w, rows, cols, 1e-6, 64.0)
    assert np.array_equal(pf, pc) and np.array_equal(sf, sc)


def test_bf16_round_trip_helpers():
    rng = np.random.default_rng(5)
    x = rng.standard_normal(4096).astype(np.float32)
    from util import to_bf16_bits
    assert np.array_equal(orc.f32_to_bf16(x), to_bf16_bits(x))
    b = orc.f32_to_bf16(x)
    assert np.array_equal(orc.f32_to_bf16(orc.bf16_to_f32(b)), b)
    # ties to even: 1 + 2^-8 is half way between two bf16 values -> even mantissa (1.0)
    assert orc.f32_to_bf16(np.array([1.0 + 2.0 ** -8], np.float32))[0] == 0x3F80
    assert orc.f32_to_bf16(np.array([1.0 + 3 * 2.0 ** -8], np.float32))[0] == 0x3F82


# ---- the steps either side of the fused quantisers --------------------------------------------------------------------
def test_to_bf16_rows_known_answers():
    """kernels/attention_mma.cu:118-171: the offset form and the scatter form, NaN -> 0x7FFF as __float2bfloat16."""
    x = np.array([1.0, -2.0, 0.5, np.inf, 1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8, np.nan, -0.0], np.float32)
    out = np.full(24, 0xBF80, np.uint16)
    orc.to_bf16_rows(x, out, off_tokens=2, stride=8)
    assert (out[:16] == 0xBF80).all()
    assert list(out[16:]) == [0x3F80, 0xC000, 0x3F00, 0x7F80, 0x3F80, 0x3F82, 0x7FFF, 0x8000]
    rows = np.arange(32, dtype=np.float32).reshape(4, 8)
    cache = np.zeros(6 * 8, np.uint16)
    orc.to_bf16_rows(rows, cache, pos_map=[5, 0, 3, 1], stride=8)
    got = orc.bf16_to_f32(cache).reshape(6, 8)
    assert np.array_equal(got[5], rows[0]) and np.array_equal(got[0], rows[1])
    assert np.array_equal(got[3], rows[2]) and np.array_equal(got[1], rows[3])
    assert not got[2].any() and not got[4].any()


def test_sigmoid_mul_and_add_known_answers():
    """kernels/elementwise.cu:344-359 (two forms) and kernels/head.cu:117-129."""
    x = np.array([2.0, -3.0, 0.0, 1.5, 7.0, 1.0, -1.0], np.float32)
    g = np.array([0.0, 0.0, 5.0, 100.0, -100.0, 1.0, -1.0], np.float32)
    f32, _ = orc.sigmoid_mul(x, g)
    assert f32[0] == 1.0 and f32[1] == -1.5 and f32[2] == 0.0 and f32[3] == 1.5 and f32[4] < 1e-40
    # element 4 is the last of the whole quad; 5 and 6 are the tail, computed as x * (1 / (1 + e))
    e = np.exp(np.float32(-1.0))
    assert f32[5] == np.float32(1.0) * (np.float32(1.0) / (np.float32(1.0) + e))
    s, bits = orc.add(np.array([1.0, 2.5, -0.0], np.float32), np.array([2.0 ** -30, -2.5, 0.0], np.float32))
    assert s[0] == 1.0 and s[1] == 0.0 and s[2] == 0.0
    # the fused restatement equals sigmoid_mul followed by the quantiser
    rows, cols = 3, 256
    rng = np.random.default_rng(11)
    xv = rng.standard_normal((rows, cols)).astype(np.float32)
    gv = (rng.standard_normal((rows, cols)) * 3).astype(np.float32)
    act, _ = orc.sigmoid_mul(xv, gv)
    pc, sc = orc.quantise_nvfp4(act, rows, cols, 48.0)
    pf, sf = orc.sigmoid_mul_quantise_nvfp4(xv, gv, rows, cols, 48.0)
    assert np.array_equal(pf, pc) and np.array_equal(sf, sc)


def test_config_0_chain_on_the_cpu_restatement():
    """The CPU-runnable configuration: 778 rows, embedding gather (table 32768 x 2048, N(0, 0.02), 8 outlier channels
    x20) -> RMSNorm (eps 1e-6, weight 1 + N(0, 0.1)) -> NVFP4 -> dequantised check with src/dequant.rs semantics."""
    from util import to_bf16_bits
    rows, hidden, vocab = 778, 2048, 32768
    rng = np.random.default_rng(7780)
    tf = (rng.standard_normal((vocab, hidden)) * 0.02).astype(np.float32)
    tf[:, rng.choice(hidden, 8, replace=False)] *= 20.0
    table = to_bf16_bits(tf)
    ids = rng.integers(0, vocab, rows).astype(np.int32)
    w = (rng.standard_normal(hidden) * 0.1).astype(np.float32)
    h = orc.embed_gather(table, ids, rows, hidden)
    assert np.array_equal(h, table[ids])
    normed, _ = orc.rms_norm(h, w, rows, hidden, 1e-6)
    gs = float(np.float32(448.0 * 6.0) / np.abs(normed).max())
    fused_p, fused_s = orc.rms_norm_quantise_nvfp4(h, w, rows, hidden, 1e-6, gs)
    chain_p, chain_s = orc.quantise_nvfp4(normed, rows, hidden, gs)
    assert np.array_equal(fused_p, chain_p) and np.array_equal(fused_s, chain_s)
    rows_padded, blocks = 896, hidden // 16
    assert fused_p.size == rows_padded * hidden // 2 and not fused_p[rows * hidden // 2:].any()
    row_major = orc.unswizzle_tiled(fused_s, rows_padded, blocks, 128, conflict_free=True)[: rows * blocks].reshape(rows, blocks)
    scale_f32 = orc.e4m3_table()[row_major]
    deq = orc.dequantise(fused_p[: rows * hidden // 2], scale_f32, gs, hidden, rows).reshape(rows, hidden)
    unit = np.repeat(scale_f32 / np.float32(gs), 16, axis=1)
    assert (np.abs(deq - normed) <= unit + 1e-12).all()
    assert np.linalg.norm(deq - normed) / np.linalg.norm(normed) < 0.2


def test_causal_conv_silu_known_answers():
    """kernels/elementwise.cu:243-274: taps before a sequence start are skipped without history and taken from the
    slot's history with it; sequences packed in one pass do not see each other."""
    k, channels = 4, 2
    x = np.arange(1, 13, dtype=np.float32).reshape(6, 2)          # rows 0..5
    w = np.tile(np.array([[0.5, -1.0, 2.0, 1.0]], np.float32), (channels, 1))
    silu = lambda a: a / (1.0 + np.exp(-a))
    # one sequence, no history: row 0 sees only its own tap (weight 1.0), row 3 sees all four
    f32, _, acc = orc.causal_conv_silu(x, w, 6, channels, k)
    assert acc[0, 0] == 1.0 * x[0, 0]
    assert acc[3, 1] == np.float32(0.5 * x[0, 1] - 1.0 * x[1, 1] + 2.0 * x[2, 1] + 1.0 * x[3, 1])
    np.testing.assert_allclose(f32, silu(acc.astype(np.float64)), rtol=1e-6)
    # two sequences (rows 0-2 and 3-5): row 3 starts afresh
    seq_start = np.array([0, 0, 0, 3, 3, 3], np.int32)
    _, _, acc2 = orc.causal_conv_silu(x, w, 6, channels, k, seq_start=seq_start)
    assert acc2[3, 0] == 1.0 * x[3, 0] and acc2[4, 0] == np.float32(2.0 * x[3, 0] + 1.0 * x[4, 0])
    assert np.array_equal(acc2[:3], acc[:3])
    # history of slot 1 continues the second sequence: its three rows stand in for rows "before 3"
    hist = np.zeros((2, k - 1, channels), np.float32)
    hist[1] = np.array([[10, 20], [30, 40], [50, 60]], np.float32)
    slot_map = np.array([0, 0, 0, 1, 1, 1], np.int32)
    _, _, acc3 = orc.causal_conv_silu(x, w, 6, channels, k, seq_start=seq_start, history=hist, slot_map=slot_map)
    assert acc3[3, 0] == np.float32(0.5 * 10 - 1.0 * 30 + 2.0 * 50 + 1.0 * x[3, 0])
    assert acc3[4, 1] == np.float32(0.5 * 40 - 1.0 * 60 + 2.0 * x[3, 1] + 1.0 * x[4, 1])
    assert np.array_equal(acc3[:3], acc[:3])                       # slot 0's history is all zeros


def test_gdn_gates_known_answers():
    """kernels/elementwise.cu:361-377."""
    a = np.array([[0.0, 25.0]], np.float32)
    b = np.array([[0.0, -30.0]], np.float32)
    decay, beta = orc.gdn_gates(a, b, np.array([0.0, 1.0], np.float32), np.array([0.0, 0.0], np.float32), 1, 2)
    assert beta[0, 0] == 0.5 and beta[0, 1] < 1e-12
    np.testing.assert_allclose(decay[0, 0], -np.log(2.0), rtol=1e-6)       # -exp(0) * log1p(exp(0))
    np.testing.assert_allclose(decay[0, 1], -np.e * 25.0, rtol=1e-6)      # softplus(x) = x above 20


def test_gdn_prep_operand_layout_and_split():
    """kernels/gdn_chunk.cu:1176-1239 restated: unit-vector heads give 1 / sqrt(1 + 1e-6) at one position (hi = 1.0,
    lo = the remainder), the stored position follows the swizzled operand layout, k heads repeat heads / kh times,
    hi + lo reproduces the normalised value to bf16^2 precision, pad rows of the last chunk stay zero."""
    seq_len, kh, heads, kd = 70, 4, 8, 128
    conv_dim = 2 * kh * kd + heads * kd
    rng = np.random.default_rng(70)
    x = rng.standard_normal((seq_len, conv_dim)).astype(np.float32)
    x[3, :] = 0.0
    x[3, 5] = 2.0                                   # q head 0 of token 3: the unit vector e_5 times 2
    x[3, kh * kd + 2 * kd + 77] = -3.0              # k head 2 of token 3: -e_77 times 3
    out = orc.gdn_prep(x, seq_len, kh, kd, heads, conv_dim)
    nchunks, ratio = 2, heads // kh

    def word(he, t, p):
        return (((he * nchunks + t // 64) * 2 + p // 64) * 8192 + (t % 64) * 128 + ((((p % 64) // 8) ^ (t % 8)) * 16) + (p % 8) * 2) // 2

    q_scale = np.float32(1.0) / np.sqrt(np.float32(kd))
    unit = np.float32(2.0) * (np.float32(1.0) / np.sqrt(np.float32(4.0) + np.float32(1e-6)))
    want_q = np.float32(unit * q_scale)
    hi = orc.bf16_to_f32(out["q_hi"])
    lo = orc.bf16_to_f32(out["q_lo"])
    for he in (0, 1):                               # q head 0 -> expanded heads 0 and 1
        assert hi[word(he, 3, 5)] == orc.bf16_to_f32(to_bf16_bits(np.array([want_q])))[0]
        assert np.float32(hi[word(he, 3, 5)] + lo[word(he, 3, 5)]) == pytest.approx(want_q, rel=2.0 ** -15)
        assert hi[word(he, 3, 6)] == 0.0
    khi = orc.bf16_to_f32(out["k_hi"])
    assert khi[word(4, 3, 77)] == -1.0 and khi[word(5, 3, 77)] == -1.0 and khi[word(6, 3, 77)] == 0.0
    assert out["kn"][3, 4, 77] == pytest.approx(-1.0, rel=1e-6) and out["kn"][3, 5, 77] == out["kn"][3, 4, 77]
    # every value: hi + lo against float64, the whole layout at once
    t = np.arange(seq_len)[:, None, None]
    he = np.arange(heads)[None, :, None]
    p = np.arange(kd)[None, None, :]
    off = word(he, t, p)
    heads_x = x[:, kh * kd: 2 * kh * kd].reshape(seq_len, kh, kd).astype(np.float64)
    want = np.repeat(heads_x / np.sqrt((heads_x ** 2).sum(-1, keepdims=True) + 1e-6), ratio, axis=1)
    err = np.abs(khi[off].astype(np.float64) + orc.bf16_to_f32(out["k_lo"])[off] - want)
    assert (err <= np.abs(want) * 2.0 ** -16 + 1e-7).all()       # two bf16 roundings deep, plus the f32 arithmetic
    assert np.array_equal(out["v"], x[:, 2 * kh * kd:])
    pad = word(np.arange(heads)[:, None, None], np.arange(seq_len, 128)[None, :, None], np.arange(kd)[None, None, :])
    assert not out["q_hi"][pad].any() and not out["k_lo"][pad].any()
