"""Parity of the NVFP4-producing entry points, called through the C-ABI, against
  T1: the reference's own kernels (oracle/_ref cubins) on the same GPU, bf16 inputs widened to f32,
  T0: the CPU oracle (oracle/clef_oracle.cpp).
Packed codes and scale bytes must be bit-exact, padding included. For the two kernels whose GPU
arithmetic uses approximate intrinsics (SwiGLU, gated RMSNorm) the CPU comparison accepts only
differences explained by a value within 4e-6 (relative) of a rounding boundary.
"""
import numpy as np
import pytest
import torch

import aiis_clef_b200 as clef
from oracle import binding as orc
from oracle import ref_gpu
from gpu_util import (Guarded, call, dev_bf16, dev_f32_from_bits, explain_mismatches, ptr, quant_sizes, stream)
from util import assert_bytes_equal, lcg_stream, normal_bf16, to_bf16_bits

pytestmark = pytest.mark.gpu

ROWS = [1, 7, 127, 128, 129, 765, 778]
BF16, F32 = 0, 1


@pytest.fixture(autouse=True)
def _reset_choice():
    clef.set_kernel_choice(0)
    yield
    clef.set_kernel_choice(0)


def run_quant(entry, rows, cols, args_before, args_after, blk_mn=128):
    """Call a quantising entry point into poisoned, guarded outputs; return (packed, scales) bytes."""
    _, pbytes, sbytes = quant_sizes(rows, cols, blk_mn)
    packed, scales = Guarded(pbytes), Guarded(sbytes)
    st = call(entry, stream(), *args_before, packed.ptr, scales.ptr, *args_after)
    assert st == 0
    torch.cuda.synchronize()
    packed.check_guards(entry + " packed")
    scales.check_guards(entry + " scales")
    return packed.bytes(), scales.bytes()


# ---------------------------------------------------------------------------------------------------------
# quantise_nvfp4
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("rows", ROWS)
@pytest.mark.parametrize("cols", [64, 2048, 6144])
def test_quantise_nvfp4(rows, cols, choice):
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(rows * 131 + cols)
    x = normal_bf16(rng, (rows, cols), outlier_channels=8)
    gs = 448.0 * 6.0 / 90.0
    dx = dev_bf16(x)
    got_p, got_s = run_quant("clef_quantise_nvfp4", rows, cols, [ptr(dx)], [rows, cols, gs, 128, 512, BF16])
    want_p, want_s = orc.quantise_nvfp4(x, rows, cols, gs)
    assert_bytes_equal(got_p, want_p, "packed vs CPU oracle")
    assert_bytes_equal(got_s, want_s, "scales vs CPU oracle")
    ref_p, ref_s = ref_gpu.quantise_nvfp4(dev_f32_from_bits(x), rows, cols, gs)
    torch.cuda.synchronize()
    assert_bytes_equal(got_p, ref_p.cpu().numpy(), "packed vs reference kernel")
    assert_bytes_equal(got_s, ref_s.cpu().numpy(), "scales vs reference kernel")
    # f32 activations: the reference engine's own dtype
    xf = dev_f32_from_bits(x)
    f_p, f_s = run_quant("clef_quantise_nvfp4", rows, cols, [ptr(xf)], [rows, cols, gs, 128, 512, F32])
    assert_bytes_equal(f_p, want_p, "f32 input packed")
    assert_bytes_equal(f_s, want_s, "f32 input scales")


def test_quantise_round_trip_recipe_of_the_reference():
    """src/cuda/mod.rs:7571-7653 with the GPU quantiser and the CPU dequantiser."""
    rows, cols = 7, 12288
    i = np.arange(rows * cols)
    x = ((np.float32(2.0) + (i // 16 % 5).astype(np.float32)) * (np.float32(0.5) + (i % 16).astype(np.float32) / np.float32(15.0))
         * np.where(i % 2 == 0, np.float32(1.0), np.float32(-1.0))).astype(np.float32)
    gs = float(np.float32(448.0) / (np.abs(x).max() / np.float32(6.0)))
    xd = torch.from_numpy(x).cuda()
    got_p, got_s = run_quant("clef_quantise_nvfp4", rows, cols, [ptr(xd)], [rows, cols, gs, 128, 512, F32])
    compact = orc.unswizzle_tiled(got_s, 128, cols // 16, 128, True)
    scale_f32 = orc.e4m3_table()[compact[: rows * (cols // 16)]]
    deq = orc.dequantise(got_p, scale_f32, gs, cols, rows)
    err = np.abs(deq - x)
    big = np.abs(x) > np.abs(x).mean() / 8.0
    assert (err[big] / np.abs(x[big])).max() < 0.25
    assert err.max() <= (np.abs(x).reshape(-1, 16).max(axis=1) / 6.0).max() + 1e-3
    z = torch.zeros(64, device="cuda")
    zp, zs = run_quant("clef_quantise_nvfp4", 1, 64, [ptr(z)], [1, 64, gs, 128, 512, F32])
    assert not zp.any() and not zs.any()


# ---------------------------------------------------------------------------------------------------------
# rms_norm_quantise_nvfp4
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("rows", ROWS)
@pytest.mark.parametrize("cols", [2048, 4096, 128, 1024, 6144])
def test_rms_norm_quantise_nvfp4(rows, cols, choice):
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(rows * 17 + cols)
    x = normal_bf16(rng, (rows, cols), outlier_channels=8)
    w = (rng.standard_normal(cols) * 0.1).astype(np.float32)
    eps, gs = 1e-6, 448.0 * 6.0 / 30.0
    dx, dw = dev_bf16(x), torch.from_numpy(w).cuda()
    got_p, got_s = run_quant("clef_rms_norm_quantise_nvfp4", rows, cols, [ptr(dx), ptr(dw)],
                             [rows, cols, eps, gs, 128, 512, BF16])
    want_p, want_s = orc.rms_norm_quantise_nvfp4(x, w, rows, cols, eps, gs)
    assert_bytes_equal(got_s, want_s, "scales vs CPU oracle")
    assert_bytes_equal(got_p, want_p, "packed vs CPU oracle")
    # reference chain on the same GPU: rms_norm_kernel -> quantise_nvfp4_kernel
    xf = dev_f32_from_bits(x)
    normed = ref_gpu.rms_norm(xf, dw, rows, cols, eps)
    ref_p, ref_s = ref_gpu.quantise_nvfp4(normed, rows, cols, gs)
    torch.cuda.synchronize()
    assert_bytes_equal(got_s, ref_s.cpu().numpy(), "scales vs reference chain")
    assert_bytes_equal(got_p, ref_p.cpu().numpy(), "packed vs reference chain")
    if cols == 4096:   # the shape the reference's fused kernel accepts
        fp, fs = ref_gpu.rms_norm_quantise_nvfp4(xf, dw, rows, cols, eps, gs)
        torch.cuda.synchronize()
        assert_bytes_equal(got_s, fs.cpu().numpy(), "scales vs reference fused kernel")
        assert_bytes_equal(got_p, fp.cpu().numpy(), "packed vs reference fused kernel")
    # f32 activations, the reference engine's own dtype (tuned f32 kernel at cols 2048 / 4096, shape-general elsewhere)
    f_p, f_s = run_quant("clef_rms_norm_quantise_nvfp4", rows, cols, [ptr(xf), ptr(dw)],
                         [rows, cols, eps, gs, 128, 512, F32])
    assert_bytes_equal(f_p, want_p, "f32 input packed")
    assert_bytes_equal(f_s, want_s, "f32 input scales")


@pytest.mark.parametrize("rows", [1, 65, 300])
@pytest.mark.parametrize("cols", [1088, 1536, 1792])
def test_widths_whose_reference_team_does_not_divide_the_cta(rows, cols):
    """cols in (1024, 1792]: the reference assigns 160, 192 or 224 threads to a row, which does not divide its
    256-thread block; its surplus threads then work on the next block's row as a partial team and race with that
    block, so the reference kernels are not an arbiter here. The CPU oracle (one team per row) is, and the result
    must be the same on every call."""
    rng = np.random.default_rng(rows + cols)
    x = normal_bf16(rng, (rows, cols), outlier_channels=4)
    w = (rng.standard_normal(cols) * 0.1).astype(np.float32)
    eps, gs = 1e-6, 64.0
    dx, dw = dev_bf16(x), torch.from_numpy(w).cuda()
    want_p, want_s = orc.rms_norm_quantise_nvfp4(x, w, rows, cols, eps, gs)
    for trial in range(3):
        got_p, got_s = run_quant("clef_rms_norm_quantise_nvfp4", rows, cols, [ptr(dx), ptr(dw)],
                                 [rows, cols, eps, gs, 128, 512, BF16])
        assert_bytes_equal(got_s, want_s, f"scales vs CPU oracle (call {trial})")
        assert_bytes_equal(got_p, want_p, f"packed vs CPU oracle (call {trial})")
    dev = clef.Device(0)
    _, want = orc.rms_norm(x, w, rows, cols, eps)
    out = dev.rms_norm_dev(dx, dw, rows, cols, eps)
    torch.cuda.synchronize()
    d = np.abs(orc.bf16_bits(out.cpu()).astype(np.int32).reshape(-1) - want.astype(np.int32).reshape(-1))
    assert d.max() <= 1


def test_rms_norm_quantise_96_row_atom():
    rows, cols = 200, 2048
    rng = np.random.default_rng(5)
    x = normal_bf16(rng, (rows, cols))
    w = (rng.standard_normal(cols) * 0.1).astype(np.float32)
    blk_mn, chunk = clef.sf_atom_for_tile_m(192)
    assert (blk_mn, chunk) == (96, 384)
    dx, dw = dev_bf16(x), torch.from_numpy(w).cuda()   # keep the inputs alive across the call
    got_p, got_s = run_quant("clef_rms_norm_quantise_nvfp4", rows, cols, [ptr(dx), ptr(dw)],
                             [rows, cols, 1e-6, 64.0, blk_mn, chunk, BF16], blk_mn=96)
    want_p, want_s = orc.rms_norm_quantise_nvfp4(x, w, rows, cols, 1e-6, 64.0, blk_mn, chunk)
    assert_bytes_equal(got_p, want_p, "packed (96-row atom)")
    assert_bytes_equal(got_s, want_s, "scales (96-row atom)")


def test_sum_of_squares_contraction_matches_the_reference_build():
    """Which FMA contraction the reference build applies to (x*x + y*y) + (z*z + w*w): the mode the CPU
    oracle uses (oracle.binding.SUMSQ_FMA) must reproduce the reference kernel's f32 output exactly."""
    rows, cols = 4096, 2048
    rng = np.random.default_rng(99)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    w = (rng.standard_normal(cols) * 0.1).astype(np.float32)
    ref = ref_gpu.rms_norm(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), rows, cols, 1e-6).cpu().numpy()
    matches = {}
    for mode in (0, 1, 2):
        f32, _ = orc.rms_norm(x, w, rows, cols, 1e-6, fma_mode=mode)
        matches[mode] = int((f32.view(np.uint32) != ref.view(np.uint32)).sum())
    assert matches[orc.SUMSQ_FMA] == 0, f"f32 words differing per contraction mode: {matches}"


# ---------------------------------------------------------------------------------------------------------
# swiglu_quantise_nvfp4
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("rows", ROWS)
@pytest.mark.parametrize("cols", [6144, 64, 12288])
def test_swiglu_quantise_nvfp4(rows, cols, choice):
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(rows * 29 + cols)
    gate = normal_bf16(rng, (rows, cols))
    up = normal_bf16(rng, (rows, cols), outlier_channels=8)
    gs = 448.0 * 6.0 / 60.0
    dg, du = dev_bf16(gate), dev_bf16(up)
    got_p, got_s = run_quant("clef_swiglu_quantise_nvfp4", rows, cols, [ptr(dg), ptr(du)], [rows, cols, gs, 128, 512, BF16])
    # T1: the reference's fused kernel, and its unfused chain, on the same GPU -- exact
    gf, uf = dev_f32_from_bits(gate), dev_f32_from_bits(up)
    ref_p, ref_s = ref_gpu.swiglu_quantise_nvfp4(gf, uf, rows, cols, gs)
    act = ref_gpu.swiglu(gf, uf, rows * cols)
    ch_p, ch_s = ref_gpu.quantise_nvfp4(act, rows, cols, gs)
    torch.cuda.synchronize()
    assert_bytes_equal(got_s, ref_s.cpu().numpy(), "scales vs reference fused kernel")
    assert_bytes_equal(got_p, ref_p.cpu().numpy(), "packed vs reference fused kernel")
    assert_bytes_equal(got_s, ch_s.cpu().numpy(), "scales vs reference chain")
    assert_bytes_equal(got_p, ch_p.cpu().numpy(), "packed vs reference chain")
    # T0: CPU oracle, boundary-aware
    want_p, want_s, pre = orc.swiglu_quantise_nvfp4(gate, up, rows, cols, gs, want_pre=True)
    n_scale, n_code, bad = explain_mismatches(pre, gs, got_p, got_s, want_p, want_s, rows, cols)
    assert bad == 0, f"{bad} differences from the CPU oracle are not at a rounding boundary ({n_scale} scales, {n_code} codes differ)"
    assert n_scale + n_code <= max(4, rows * cols // 2000)
    if choice == 1:
        f_p, f_s = run_quant("clef_swiglu_quantise_nvfp4", rows, cols, [ptr(gf), ptr(uf)], [rows, cols, gs, 128, 512, F32])
        assert_bytes_equal(f_p, got_p, "f32 input packed")
        assert_bytes_equal(f_s, got_s, "f32 input scales")


def test_swiglu_quantise_recipe_of_the_reference():
    """src/cuda/mod.rs:8133-8202: 765 and 769 rows x 12288, LCG inputs * 0.05, global 215."""
    cols, gs = 12288, 215.0
    for rows in (765, 769):
        seq = lcg_stream(0x511161, 2 * rows * cols) * np.float32(0.05)
        gate, up = to_bf16_bits(seq[: rows * cols]).reshape(rows, cols), to_bf16_bits(seq[rows * cols:]).reshape(rows, cols)
        dg, du = dev_bf16(gate), dev_bf16(up)
        got_p, got_s = run_quant("clef_swiglu_quantise_nvfp4", rows, cols, [ptr(dg), ptr(du)], [rows, cols, gs, 128, 512, BF16])
        ref_p, ref_s = ref_gpu.swiglu_quantise_nvfp4(dev_f32_from_bits(gate), dev_f32_from_bits(up), rows, cols, gs)
        torch.cuda.synchronize()
        assert_bytes_equal(got_p, ref_p.cpu().numpy(), f"{rows} rows packed")
        assert_bytes_equal(got_s, ref_s.cpu().numpy(), f"{rows} rows scales")


# ---------------------------------------------------------------------------------------------------------
# rms_norm_gated_quantise_nvfp4
# ---------------------------------------------------------------------------------------------------------
def run_gated(x, g, w, tokens, vh, cols, eps, gs, dtype=BF16, blk_mn=128):
    rows_live = tokens * vh
    tokens_padded = (tokens + blk_mn - 1) // blk_mn * blk_mn
    rows = tokens_padded * vh
    packed, scales = Guarded(rows * (cols // 2)), Guarded(tokens_padded * (vh * cols // 16))
    st = call("clef_rms_norm_gated_quantise_nvfp4", stream(), ptr(x), ptr(g), ptr(w), packed.ptr, scales.ptr, rows, cols,
              eps, gs, blk_mn, blk_mn * 4, vh, rows_live, dtype)
    assert st == 0
    torch.cuda.synchronize()
    packed.check_guards("gated packed")
    scales.check_guards("gated scales")
    return packed.bytes(), scales.bytes()


@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("tokens", [1, 7, 127, 129, 300, 778])
@pytest.mark.parametrize("vh", [16, 32])
def test_rms_norm_gated_quantise_nvfp4(tokens, vh, choice):
    clef.set_kernel_choice(choice)
    cols, eps, gs = 128, 1e-6, 448.0 * 6.0 / 40.0
    rows = tokens * vh
    rng = np.random.default_rng(tokens * 7 + vh)
    x = normal_bf16(rng, (rows, cols))
    g = normal_bf16(rng, (rows, cols))
    w = (1.0 + rng.standard_normal(cols) * 0.1).astype(np.float32)
    dx, dg, dw = dev_bf16(x), dev_bf16(g), torch.from_numpy(w).cuda()
    got_p, got_s = run_gated(dx, dg, dw, tokens, vh, cols, eps, gs)
    xf, gf = dev_f32_from_bits(x), dev_f32_from_bits(g)
    ref_p, ref_s = ref_gpu.rms_norm_gated_quantise_nvfp4(xf, gf, dw, rows, cols, vh, eps, gs)
    torch.cuda.synchronize()
    assert_bytes_equal(got_s, ref_s.cpu().numpy(), "scales vs reference fused kernel")
    assert_bytes_equal(got_p, ref_p.cpu().numpy(), "packed vs reference fused kernel")
    # reference chain: rms_norm_gated_kernel -> quantise_nvfp4_kernel over [tokens, vh*cols]
    gated = ref_gpu.rms_norm_gated(xf, gf, dw, rows, cols, eps)
    ch_p, ch_s = ref_gpu.quantise_nvfp4(gated, tokens, vh * cols, gs)
    torch.cuda.synchronize()
    assert_bytes_equal(got_s, ch_s.cpu().numpy(), "scales vs reference chain")
    assert_bytes_equal(got_p, ch_p.cpu().numpy(), "packed vs reference chain")
    want_p, want_s, pre = orc.rms_norm_gated_quantise_nvfp4(x, g, w, rows, cols, vh, eps, gs, want_pre=True)
    n_scale, n_code, bad = explain_mismatches(pre.reshape(tokens, vh * cols), gs, got_p, got_s, want_p, want_s, tokens, vh * cols, rel=8e-6)
    assert bad == 0, f"{bad} differences from the CPU oracle are not at a rounding boundary ({n_scale} scales, {n_code} codes)"
    # f32 activations, the reference engine's own dtype (tuned f32 kernel or the shape-general one)
    f_p, f_s = run_gated(xf, gf, dw, tokens, vh, cols, eps, gs, dtype=F32)
    assert_bytes_equal(f_p, got_p, "f32 input packed")
    assert_bytes_equal(f_s, got_s, "f32 input scales")


def test_gated_recipe_of_the_reference():
    """src/cuda/mod.rs:6866-6917: 7 and 300 tokens x 32 heads x 128, LCG inputs * 1.1, global 1/12.5."""
    cols, vh, eps = 128, 32, 1e-6
    gs = float(np.float32(1.0 / 12.5))
    for tokens in (7, 300):
        rows = tokens * vh
        seq = lcg_stream(0x9E3779B9 ^ tokens, 2 * rows * cols + cols) * np.float32(1.1)
        x = to_bf16_bits(seq[: rows * cols]).reshape(rows, cols)
        g = to_bf16_bits(seq[rows * cols: 2 * rows * cols]).reshape(rows, cols)
        w = (np.float32(0.5) + seq[2 * rows * cols:] * np.float32(0.1)).astype(np.float32)
        dw = torch.from_numpy(w).cuda()
        got_p, got_s = run_gated(dev_bf16(x), dev_bf16(g), dw, tokens, vh, cols, eps, gs)
        ref_p, ref_s = ref_gpu.rms_norm_gated_quantise_nvfp4(dev_f32_from_bits(x), dev_f32_from_bits(g), dw, rows, cols, vh, eps, gs)
        torch.cuda.synchronize()
        assert_bytes_equal(got_p, ref_p.cpu().numpy(), f"{tokens} tokens packed")
        assert_bytes_equal(got_s, ref_s.cpu().numpy(), f"{tokens} tokens scales")


# ---------------------------------------------------------------------------------------------------------
# determinism, argument checks
# ---------------------------------------------------------------------------------------------------------
def test_same_call_twelve_times():
    """src/gpu.rs:5885-5985: every op answers the same twelve times."""
    rows, cols = 300, 2048
    rng = np.random.default_rng(1)
    x, w = dev_bf16(normal_bf16(rng, (rows, cols))), torch.from_numpy((rng.standard_normal(cols) * 0.1).astype(np.float32)).cuda()
    gate, up = dev_bf16(normal_bf16(rng, (rows, 6144))), dev_bf16(normal_bf16(rng, (rows, 6144)))
    first = None
    for _ in range(12):
        a = run_quant("clef_rms_norm_quantise_nvfp4", rows, cols, [ptr(x), ptr(w)], [rows, cols, 1e-6, 64.0, 128, 512, BF16])
        b = run_quant("clef_swiglu_quantise_nvfp4", rows, 6144, [ptr(gate), ptr(up)], [rows, 6144, 64.0, 128, 512, BF16])
        cur = [a[0], a[1], b[0], b[1]]
        if first is None:
            first = cur
        else:
            for u, v in zip(first, cur):
                assert np.array_equal(u, v)


def test_bad_arguments_are_refused_without_a_launch():
    lib = clef.load()
    x = torch.zeros(2048 * 4, dtype=torch.bfloat16, device="cuda")
    out = Guarded(1 << 16)
    sc = Guarded(1 << 12)
    w = torch.zeros(2048, device="cuda")
    s = stream()
    assert lib.clef_quantise_nvfp4(s, ptr(x), out.ptr, sc.ptr, 4, 100, 1.0, 128, 512, BF16) == -1      # cols % 64
    assert lib.clef_quantise_nvfp4(s, None, out.ptr, sc.ptr, 4, 2048, 1.0, 128, 512, BF16) == -1        # null
    assert lib.clef_quantise_nvfp4(s, ptr(x), out.ptr, sc.ptr, 4, 2048, 1.0, 128, 500, BF16) == -1      # chunk
    assert lib.clef_quantise_nvfp4(s, ptr(x), out.ptr, sc.ptr, 4, 2048, 1.0, 128, 512, 7) == -1         # dtype
    assert lib.clef_rms_norm_quantise_nvfp4(s, x.data_ptr() + 2, ptr(w), out.ptr, sc.ptr, 2, 2048, 1e-6, 1.0, 128, 512, BF16) == -1
    assert lib.clef_rms_norm_gated_quantise_nvfp4(s, ptr(x), ptr(x), ptr(w), out.ptr, sc.ptr, 100, 128, 1e-6, 1.0, 128, 512, 16, 64, BF16) == -1
    assert b"rows" in lib.clef_last_error()
    torch.cuda.synchronize()
    assert (out.bytes() == 0xA5).all() and (sc.bytes() == 0xA5).all()
