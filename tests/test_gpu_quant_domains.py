"""The tuned quantising kernels at the edges of their block quantiser's fast domain, and at the exact shapes of
the benchmark step, against the reference's own kernels (oracle/_ref cubins) on the same GPU.

The tuned kernels quantise a block on a short path when its scale argument lies in [2^-6, 2^30) (a normal E4M3 code,
clamped from 448 up) or the block is all zeros, and recompute it literally otherwise. These tests drive whole
launches to both sides of those edges (subnormal scale codes, clamped codes, scale arguments beyond 2^30, zero and
non-finite blocks, global scales outside the tuned range) and compare bytes with the reference kernels, padding
included.
"""
import numpy as np
import pytest
import torch

import aiis_clef_b200 as clef
from oracle import binding as orc
from oracle import ref_gpu
from gpu_util import Guarded, call, dev_bf16, dev_f32_from_bits, f32_to_bf16_bits_gpu, ptr, quant_sizes, stream
from util import assert_bytes_equal, normal_bf16, to_bf16_bits

pytestmark = pytest.mark.gpu
BF16 = 0


@pytest.fixture(autouse=True)
def _tuned_kernels():
    clef.set_kernel_choice(0)
    yield
    clef.set_kernel_choice(0)


def run_quant(entry, rows, cols, args_before, args_after):
    _, pbytes, sbytes = quant_sizes(rows, cols, 128)
    packed, scales = Guarded(pbytes), Guarded(sbytes)
    assert call(entry, stream(), *args_before, packed.ptr, scales.ptr, *args_after) == 0
    torch.cuda.synchronize()
    packed.check_guards(entry + " packed")
    scales.check_guards(entry + " scales")
    return packed.bytes(), scales.bytes()


def adversarial_bf16_matrix(rng, rows, cols):
    """[rows, cols] bf16 bits whose 16-value blocks cover: zeros, negative zeros, exact E2M1 ties at several
    magnitudes, values spanning 10^-12 .. 10^12, bf16 denormals, the largest bf16, infinities and NaN."""
    blocks = rows * cols // 16
    x = rng.standard_normal((blocks, 16)).astype(np.float32)
    x *= np.float32(10.0) ** rng.integers(-12, 13, (blocks, 1)).astype(np.float32)
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0], np.float32)
    kind = rng.integers(0, 16, blocks)
    x[kind == 0] = 0.0
    x[kind == 1] = -0.0
    tie_rows = np.flatnonzero(kind == 2)
    for i in tie_rows:
        amax = np.float32(2.0) ** rng.integers(-8, 9)
        v = np.concatenate([ties, -ties]) * (amax / np.float32(6.0))
        x[i] = v
    x[kind == 3, 0] = 0.0                                  # one zero inside a normal block
    bits = to_bf16_bits(x)
    bits[kind == 4, 3] = 0x0001                            # a bf16 denormal
    bits[kind == 5] = 0x0040                               # only denormals
    special = np.flatnonzero(kind == 6)
    for n, i in enumerate(special):
        bits[i, n % 16] = [0x7F80, 0xFF80, 0x7FC0, 0x7F7F, 0xFF7F][n % 5]   # +inf, -inf, NaN, +max, -max
    return bits.reshape(rows, cols)


@pytest.mark.parametrize("global_scale", [1.0, 64.0, 1.0 / 12.5, 2688.0, 1e-6, 1e6, 3e-20, 5e19, 1e-30, 1e30, 0.0, -3.0])
def test_plain_quantiser_on_adversarial_blocks(global_scale):
    rows, cols = 130, 2048
    rng = np.random.default_rng(41)
    x = adversarial_bf16_matrix(rng, rows, cols)
    dx = dev_bf16(x)
    got_p, got_s = run_quant("clef_quantise_nvfp4", rows, cols, [ptr(dx)], [rows, cols, global_scale, 128, 512, BF16])
    ref_p, ref_s = ref_gpu.quantise_nvfp4(dev_f32_from_bits(x), rows, cols, global_scale)
    torch.cuda.synchronize()
    assert_bytes_equal(got_s, ref_s.cpu().numpy(), f"scales vs reference kernel (global scale {global_scale})")
    assert_bytes_equal(got_p, ref_p.cpu().numpy(), f"packed vs reference kernel (global scale {global_scale})")
    want_p, want_s = orc.quantise_nvfp4(x, rows, cols, global_scale)
    assert_bytes_equal(got_s, want_s, "scales vs CPU oracle")
    assert_bytes_equal(got_p, want_p, "packed vs CPU oracle")
    # f32 activations (the engine's own dtype) through the tuned f32 kernel
    xf = dev_f32_from_bits(x)
    f_p, f_s = run_quant("clef_quantise_nvfp4", rows, cols, [ptr(xf)], [rows, cols, global_scale, 128, 512, 1])
    assert_bytes_equal(f_s, ref_s.cpu().numpy(), f"f32 activations: scales vs reference kernel (global scale {global_scale})")
    assert_bytes_equal(f_p, ref_p.cpu().numpy(), f"f32 activations: packed vs reference kernel (global scale {global_scale})")


def _with_zero_rows(bits, rng, every=7):
    bits = bits.copy()
    bits[::every] = 0
    bits[3::every * 3] = 0x8000
    return bits


@pytest.mark.parametrize("global_scale", [2e-3, 0.02, 3e4, 1e7, 3e9, 1e10, 1e-25])
@pytest.mark.parametrize("cols", [2048, 4096])
def test_rms_norm_quantise_outside_the_fast_domain(cols, global_scale):
    """Normalised values are O(1), so the global scale alone decides the code range: 2e-3 gives subnormal scale codes,
    0.02 a mix of subnormal and normal ones, 3e4 and 1e7 clamped ones, 3e9 scale arguments around 2^30 (the end of the
    short path), 1e10 beyond it, 1e-25 the shape-general kernel."""
    rows = 300
    rng = np.random.default_rng(cols + 5)
    x = _with_zero_rows(normal_bf16(rng, (rows, cols), outlier_channels=8), rng)
    w = (rng.standard_normal(cols) * 0.1).astype(np.float32)
    dx, dw = dev_bf16(x), torch.from_numpy(w).cuda()
    got_p, got_s = run_quant("clef_rms_norm_quantise_nvfp4", rows, cols, [ptr(dx), ptr(dw)],
                             [rows, cols, 1e-6, global_scale, 128, 512, BF16])
    xf = dev_f32_from_bits(x)
    normed = ref_gpu.rms_norm(xf, dw, rows, cols, 1e-6)
    ref_p, ref_s = ref_gpu.quantise_nvfp4(normed, rows, cols, global_scale)
    torch.cuda.synchronize()
    assert_bytes_equal(got_s, ref_s.cpu().numpy(), "scales vs reference chain")
    assert_bytes_equal(got_p, ref_p.cpu().numpy(), "packed vs reference chain")
    # the tuned f32 kernel (the engine's own dtype) on the same rows
    f_p, f_s = run_quant("clef_rms_norm_quantise_nvfp4", rows, cols, [ptr(xf), ptr(dw)], [rows, cols, 1e-6, global_scale, 128, 512, 1])
    assert_bytes_equal(f_s, ref_s.cpu().numpy(), "f32 activations: scales vs reference chain")
    assert_bytes_equal(f_p, ref_p.cpu().numpy(), "f32 activations: packed vs reference chain")


@pytest.mark.parametrize("rows,cols", [(2568, 2048), (1484, 4096), (3700, 2048), (2368, 2048), (8192, 2048), (1185, 4096)])
def test_rms_norm_quantise_tail_round_shared_by_warp_pairs(rows, cols):
    """Row counts that leave the tuned kernel a last round for at most half of its warps (the grid has 148 x 16 warps
    at 2,048 columns, 148 x 8 at 4,096): that round's rows are split between two warps each. With full rounds in front
    (2,568 = 2,368 + 200 rows; 1,484 = 1,184 + 300), pad rows inside the tail (rows not a multiple of 128), exactly
    full rounds (2,368: no tail), and a tail too long for pairs (3,700); blocks outside the quantiser's short path and
    zero rows land in the tail too. Bytes against the reference chain."""
    rng = np.random.default_rng(rows + cols)
    x = _with_zero_rows(normal_bf16(rng, (rows, cols), outlier_channels=8), rng)
    x[-3] = adversarial_bf16_matrix(rng, 1, cols)[0]          # non-finite, denormal and tie blocks in the last rows
    x[-40] = adversarial_bf16_matrix(rng, 1, cols)[0]
    w = (rng.standard_normal(cols) * 0.1).astype(np.float32)
    dx, dw, xf32 = dev_bf16(x), torch.from_numpy(w).cuda(), dev_f32_from_bits(x)
    for gs in (80.0, 0.02):                                    # 0.02: subnormal scale codes, the literal path
        got_p, got_s = run_quant("clef_rms_norm_quantise_nvfp4", rows, cols, [ptr(dx), ptr(dw)], [rows, cols, 1e-6, gs, 128, 512, BF16])
        normed = ref_gpu.rms_norm(dev_f32_from_bits(x), dw, rows, cols, 1e-6)
        ref_p, ref_s = ref_gpu.quantise_nvfp4(normed, rows, cols, gs)
        torch.cuda.synchronize()
        assert_bytes_equal(got_s, ref_s.cpu().numpy(), f"scales vs reference chain (global scale {gs})")
        assert_bytes_equal(got_p, ref_p.cpu().numpy(), f"packed vs reference chain (global scale {gs})")
        # the tuned f32 kernel has the same tail round
        f_p, f_s = run_quant("clef_rms_norm_quantise_nvfp4", rows, cols, [ptr(xf32), ptr(dw)], [rows, cols, 1e-6, gs, 128, 512, 1])
        assert_bytes_equal(f_s, ref_s.cpu().numpy(), f"f32 activations: scales vs reference chain (global scale {gs})")
        assert_bytes_equal(f_p, ref_p.cpu().numpy(), f"f32 activations: packed vs reference chain (global scale {gs})")


def test_rms_norm_quantise_f32_on_arbitrary_f32_rows():
    """f32 rows that are not bf16 values (the engine's residual stream), 4096 columns: the reference's own fused kernel
    serves this shape, and the chain must agree with it too; 8,192 rows cover the tuned kernel's tail."""
    for rows, cols in ((8192, 2048), (777, 4096)):
        gen = torch.Generator(device="cuda").manual_seed(rows)
        x = torch.randn(rows, cols, device="cuda", generator=gen) * 3.0
        x[:, 5] *= 30.0
        x[17] = 0.0
        w = torch.randn(cols, device="cuda", generator=gen) * 0.1
        got_p, got_s = run_quant("clef_rms_norm_quantise_nvfp4", rows, cols, [ptr(x), ptr(w)], [rows, cols, 1e-6, 80.0, 128, 512, 1])
        normed = ref_gpu.rms_norm(x, w, rows, cols, 1e-6)
        ref_p, ref_s = ref_gpu.quantise_nvfp4(normed, rows, cols, 80.0)
        torch.cuda.synchronize()
        assert_bytes_equal(got_s, ref_s.cpu().numpy(), "scales vs reference chain")
        assert_bytes_equal(got_p, ref_p.cpu().numpy(), "packed vs reference chain")
        if cols == 4096:
            fp, fs = ref_gpu.rms_norm_quantise_nvfp4(x, w, rows, cols, 1e-6, 80.0)
            torch.cuda.synchronize()
            assert_bytes_equal(got_s, fs.cpu().numpy(), "scales vs reference fused kernel")
            assert_bytes_equal(got_p, fp.cpu().numpy(), "packed vs reference fused kernel")


@pytest.mark.parametrize("global_scale", [2e-3, 0.05, 3e4, 4e9, 1e11, 1e-25])
def test_swiglu_quantise_outside_the_fast_domain(global_scale):
    rows, cols = 129, 6144
    rng = np.random.default_rng(77)
    gate = _with_zero_rows(normal_bf16(rng, (rows, cols)), rng)
    up = normal_bf16(rng, (rows, cols), outlier_channels=8)
    up[5] = 0
    dg, du = dev_bf16(gate), dev_bf16(up)
    got_p, got_s = run_quant("clef_swiglu_quantise_nvfp4", rows, cols, [ptr(dg), ptr(du)], [rows, cols, global_scale, 128, 512, BF16])
    ref_p, ref_s = ref_gpu.swiglu_quantise_nvfp4(dev_f32_from_bits(gate), dev_f32_from_bits(up), rows, cols, global_scale)
    torch.cuda.synchronize()
    assert_bytes_equal(got_s, ref_s.cpu().numpy(), "scales vs reference fused kernel")
    assert_bytes_equal(got_p, ref_p.cpu().numpy(), "packed vs reference fused kernel")
    gf, uf = dev_f32_from_bits(gate), dev_f32_from_bits(up)
    f_p, f_s = run_quant("clef_swiglu_quantise_nvfp4", rows, cols, [ptr(gf), ptr(uf)], [rows, cols, global_scale, 128, 512, 1])
    assert_bytes_equal(f_s, ref_s.cpu().numpy(), "f32 activations: scales vs reference fused kernel")
    assert_bytes_equal(f_p, ref_p.cpu().numpy(), "f32 activations: packed vs reference fused kernel")


def test_unit_quantisers_f32_on_arbitrary_f32_values():
    """f32 gate / up values that are not bf16 values (GEMM accumulators): the tuned f32 SwiGLU + NVFP4 and plain NVFP4
    kernels against the reference's own kernels, bit for bit. Gates beyond +-44, infinities and NaN take the literal
    path; 8,192 x 6144 covers the grid-stride tail and a padded last row tile."""
    for rows, cols in ((8192, 6144), (333, 1024)):
        gen = torch.Generator(device="cuda").manual_seed(rows + 1)
        gate = torch.randn(rows, cols, device="cuda", generator=gen) * 4.0
        up = torch.randn(rows, cols, device="cuda", generator=gen) * 2.0
        gate[:, 7] *= 20.0                      # |g| beyond the short form's range in every row
        gate[3, 40:56] = 0.0
        gate[4, 64] = float("inf")
        gate[5, 80] = float("-inf")
        gate[6, 96] = float("nan")
        up[7, 100] = float("inf")
        up[8, 120] = float("nan")
        up[9] = 0.0
        gate[10] = -0.0
        for gs in (48.0, 1e-3, 1e6):
            got_p, got_s = run_quant("clef_swiglu_quantise_nvfp4", rows, cols, [ptr(gate), ptr(up)], [rows, cols, gs, 128, 512, 1])
            ref_p, ref_s = ref_gpu.swiglu_quantise_nvfp4(gate, up, rows, cols, gs)
            torch.cuda.synchronize()
            assert_bytes_equal(got_s, ref_s.cpu().numpy(), f"SwiGLU scales vs reference fused kernel (global scale {gs})")
            assert_bytes_equal(got_p, ref_p.cpu().numpy(), f"SwiGLU packed vs reference fused kernel (global scale {gs})")
            got_p, got_s = run_quant("clef_quantise_nvfp4", rows, cols, [ptr(gate)], [rows, cols, gs, 128, 512, 1])
            ref_p, ref_s = ref_gpu.quantise_nvfp4(gate, rows, cols, gs)
            torch.cuda.synchronize()
            assert_bytes_equal(got_s, ref_s.cpu().numpy(), f"plain scales vs reference kernel (global scale {gs})")
            assert_bytes_equal(got_p, ref_p.cpu().numpy(), f"plain packed vs reference kernel (global scale {gs})")


@pytest.mark.parametrize("global_scale", [2e-3, 0.05, 3e4, 4e9, 1e11, 1e-25])
def test_gated_norm_quantise_outside_the_fast_domain(global_scale):
    tokens, vh, cols = 130, 16, 128
    rows = tokens * vh
    rng = np.random.default_rng(78)
    x = _with_zero_rows(normal_bf16(rng, (rows, cols)), rng)
    g = normal_bf16(rng, (rows, cols))
    g[11] = 0
    w = (1.0 + rng.standard_normal(cols) * 0.1).astype(np.float32)
    dw = torch.from_numpy(w).cuda()
    tokens_padded = (tokens + 127) // 128 * 128
    packed, scales = Guarded(tokens_padded * vh * cols // 2), Guarded(tokens_padded * vh * cols // 16)
    dx, dg = dev_bf16(x), dev_bf16(g)
    assert call("clef_rms_norm_gated_quantise_nvfp4", stream(), ptr(dx), ptr(dg), ptr(dw), packed.ptr,
                scales.ptr, tokens_padded * vh, cols, 1e-6, global_scale, 128, 512, vh, rows, BF16) == 0
    torch.cuda.synchronize()
    packed.check_guards("gated packed")
    scales.check_guards("gated scales")
    ref_p, ref_s = ref_gpu.rms_norm_gated_quantise_nvfp4(dev_f32_from_bits(x), dev_f32_from_bits(g), dw, rows, cols, vh, 1e-6,
                                                         global_scale)
    torch.cuda.synchronize()
    assert_bytes_equal(scales.bytes(), ref_s.cpu().numpy(), "scales vs reference fused kernel")
    assert_bytes_equal(packed.bytes(), ref_p.cpu().numpy(), "packed vs reference fused kernel")
    # the tuned f32 kernel on the same rows
    xf, gf = dev_f32_from_bits(x), dev_f32_from_bits(g)
    p2, s2 = Guarded(tokens_padded * vh * cols // 2), Guarded(tokens_padded * vh * cols // 16)
    assert call("clef_rms_norm_gated_quantise_nvfp4", stream(), ptr(xf), ptr(gf), ptr(dw), p2.ptr, s2.ptr, tokens_padded * vh, cols, 1e-6,
                global_scale, 128, 512, vh, rows, 1) == 0
    torch.cuda.synchronize()
    p2.check_guards("gated packed, f32")
    s2.check_guards("gated scales, f32")
    assert_bytes_equal(s2.bytes(), ref_s.cpu().numpy(), "f32 activations: scales vs reference fused kernel")
    assert_bytes_equal(p2.bytes(), ref_p.cpu().numpy(), "f32 activations: packed vs reference fused kernel")


def test_gated_norm_quantise_f32_on_arbitrary_f32_rows():
    """f32 head rows and gates that are not bf16 values (8,192 tokens x 16 heads: the tuned f32 kernel's tail; and a
    ragged token count with 32 heads), with gates beyond the short silu form's range: the reference's fused kernel."""
    for tokens, vh in ((8192, 16), (301, 32)):
        rows, cols = tokens * vh, 128
        gen = torch.Generator(device="cuda").manual_seed(tokens)
        x = torch.randn(rows, cols, device="cuda", generator=gen) * 2.0
        g = torch.randn(rows, cols, device="cuda", generator=gen) * 3.0
        g[5, :16] = 50.0
        g[6, 16:32] = -95.0
        x[9] = 0.0
        w = 1.0 + torch.randn(cols, device="cuda", generator=gen) * 0.1
        tp = (tokens + 127) // 128 * 128
        packed, scales = Guarded(tp * vh * cols // 2), Guarded(tp * vh * cols // 16)
        assert call("clef_rms_norm_gated_quantise_nvfp4", stream(), ptr(x), ptr(g), ptr(w), packed.ptr, scales.ptr, tp * vh, cols, 1e-6,
                    96.0, 128, 512, vh, rows, 1) == 0
        ref_p, ref_s = ref_gpu.rms_norm_gated_quantise_nvfp4(x, g, w, rows, cols, vh, 1e-6, 96.0)
        torch.cuda.synchronize()
        packed.check_guards("gated packed")
        scales.check_guards("gated scales")
        assert_bytes_equal(scales.bytes(), ref_s.cpu().numpy(), "scales vs reference fused kernel")
        assert_bytes_equal(packed.bytes(), ref_p.cpu().numpy(), "packed vs reference fused kernel")


# ---------------------------------------------------------------------------------------------------------
# the benchmark step's own shapes: 8,192 rows (3.46 rows per resident warp: its own tail geometry)
# ---------------------------------------------------------------------------------------------------------
STEP_ROWS = 8192


def test_step_shape_rms_norm_quantise():
    rows, cols = STEP_ROWS, 2048
    rng = np.random.default_rng(8192)
    x = normal_bf16(rng, (rows, cols), outlier_channels=8)
    w = (rng.standard_normal(cols) * 0.1).astype(np.float32)
    dx, dw = dev_bf16(x), torch.from_numpy(w).cuda()
    got_p, got_s = run_quant("clef_rms_norm_quantise_nvfp4", rows, cols, [ptr(dx), ptr(dw)], [rows, cols, 1e-6, 64.0, 128, 512, BF16])
    normed = ref_gpu.rms_norm(dev_f32_from_bits(x), dw, rows, cols, 1e-6)
    ref_p, ref_s = ref_gpu.quantise_nvfp4(normed, rows, cols, 64.0)
    torch.cuda.synchronize()
    assert_bytes_equal(got_s, ref_s.cpu().numpy(), "scales vs reference chain")
    assert_bytes_equal(got_p, ref_p.cpu().numpy(), "packed vs reference chain")
    want_p, want_s = orc.rms_norm_quantise_nvfp4(x, w, rows, cols, 1e-6, 64.0)
    assert_bytes_equal(got_s, want_s, "scales vs CPU oracle")
    assert_bytes_equal(got_p, want_p, "packed vs CPU oracle")


def test_step_shape_swiglu_quantise():
    rows, cols = STEP_ROWS, 6144
    rng = np.random.default_rng(8193)
    gate, up = normal_bf16(rng, (rows, cols)), normal_bf16(rng, (rows, cols), outlier_channels=8)
    dg, du = dev_bf16(gate), dev_bf16(up)
    got_p, got_s = run_quant("clef_swiglu_quantise_nvfp4", rows, cols, [ptr(dg), ptr(du)], [rows, cols, 48.0, 128, 512, BF16])
    ref_p, ref_s = ref_gpu.swiglu_quantise_nvfp4(dev_f32_from_bits(gate), dev_f32_from_bits(up), rows, cols, 48.0)
    torch.cuda.synchronize()
    assert_bytes_equal(got_s, ref_s.cpu().numpy(), "scales vs reference fused kernel")
    assert_bytes_equal(got_p, ref_p.cpu().numpy(), "packed vs reference fused kernel")


def test_step_shape_rope_qk():
    """clef_rope_qk on 16 q and 2 kv heads x 128 (rotary 64, theta 1e7, cpos = 0..8191): within 2 bf16 ulp of the
    reference rope_kernel's f32 result, pass-through dims byte-exact."""
    from util import bf16_ulp_distance

    rows, qh, kh, hd, rot = STEP_ROWS, 16, 2, 128, 64
    rng = np.random.default_rng(8194)
    q, k = normal_bf16(rng, (rows, qh, hd)), normal_bf16(rng, (rows, kh, hd))
    dev = clef.Device(0)
    pos = torch.arange(rows, dtype=torch.int32, device="cuda")
    cos, sin = dev.rope_tables_dev(pos, rows, rot, 1e7)
    got_q, got_k = dev.rope_qk_dev(dev_bf16(q), dev_bf16(k), cos, sin, rows, qh, kh, hd, rot, pos_map=pos)
    torch.cuda.synchronize()
    for got, bits, heads in ((got_q, q, qh), (got_k, k, kh)):
        ref = ref_gpu.rope(dev_f32_from_bits(bits), cos, sin, rows, heads, hd, rot, pos_map=pos)
        torch.cuda.synchronize()
        want = f32_to_bf16_bits_gpu(ref).reshape(rows, heads, hd)
        have = orc.bf16_bits(got.cpu()).reshape(rows, heads, hd)
        assert bf16_ulp_distance(have[..., :rot], want[..., :rot]).max() <= 2
        assert np.array_equal(have[..., rot:], bits[..., rot:]), "pass-through dims must be copied byte for byte"
