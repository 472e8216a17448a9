"""Parity of the FP8 (E4M3) activation quantisers through the C-ABI against the reference's own kernels run on
the same GPU (oracle/_ref/quantise.cubin; bf16 inputs widened exactly to the f32 those kernels take) and against
the CPU oracle. Codes, row scale words and the bf16 twin output must be byte-identical to the reference kernels;
against the CPU oracle the two kernels without approximate intrinsics must be byte-identical as well."""
import numpy as np
import pytest
import torch

import aiis_clef_b200 as clef
from oracle import binding as orc
from oracle import ref_gpu
from gpu_util import Guarded, call, dev_bf16, dev_f32_from_bits, ptr, stream
from util import assert_bytes_equal, normal_bf16, to_bf16_bits

pytestmark = pytest.mark.gpu
BF16, F32 = 0, 1


@pytest.fixture(autouse=True)
def _cleanup():
    yield
    torch.cuda.empty_cache()


def special_rows(xb, rows, cols):
    """Rows the recipe treats specially: all zero, a single huge value, tiny values only, an infinity, a NaN."""
    if rows < 12:
        return
    xb[2, :] = 0
    xb[3, 5] = to_bf16_bits(np.array([3.0e38], np.float32))[0]
    xb[4, :] = to_bf16_bits((np.ones(cols) * 1e-39).astype(np.float32))
    xb[4, 7] = to_bf16_bits(np.array([-3e-39], np.float32))[0]
    xb[5, 9] = to_bf16_bits(np.array([np.inf], np.float32))[0]
    xb[6, 11] = to_bf16_bits(np.array([np.nan], np.float32))[0]
    xb[7, :] = to_bf16_bits((np.ones(cols) * 1e-30).astype(np.float32))
    xb[8, :64] = to_bf16_bits(np.linspace(-448, 448, 64).astype(np.float32))       # exact code points and ties
    xb[9, :] = to_bf16_bits(np.full(cols, -0.0, np.float32))
    xb[10, :16] = to_bf16_bits((448.0 * np.array([2 ** -6, 2 ** -7, 2 ** -9, 2 ** -10, 1.5 * 2 ** -9, 2.5 * 2 ** -9,
                                                   15.5 * 2 ** -10, 7.5 * 2 ** -9, 2 ** -6 * 0.97, 1, 0.5, 0.25, 17 / 32, 19 / 32,
                                                   21 / 32, 1 / 3]) / 448.0 * 448.0).astype(np.float32))
    xb[10, 16] = to_bf16_bits(np.array([448.0], np.float32))[0]


def as_u16(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


@pytest.mark.parametrize("dtype", [BF16, F32], ids=["bf16", "f32"])
@pytest.mark.parametrize("rows,cols", [(1, 2048), (778, 2048), (129, 4096), (33, 6144), (20, 12288), (300, 2560)])
def test_quantise_fp8_matches_the_reference_kernel(rows, cols, dtype):
    rng = np.random.default_rng(rows + cols)
    xb = normal_bf16(rng, (rows, cols), outlier_channels=3)
    special_rows(xb, rows, cols)
    xf = dev_f32_from_bits(xb)
    ref_q, ref_s = ref_gpu.quantise_fp8(xf, rows, cols)
    out, scales = Guarded(rows * cols), Guarded(rows * 2)
    src = dev_bf16(xb) if dtype == BF16 else xf
    assert call("clef_quantise_fp8", stream(), ptr(src), out.ptr, scales.ptr, rows, cols, dtype) == 0
    torch.cuda.synchronize()
    out.check_guards("codes")
    scales.check_guards("scales")
    assert_bytes_equal(scales.bytes().view(np.uint16), as_u16(ref_s), "row scales vs reference kernel")
    assert_bytes_equal(out.bytes(), ref_q.cpu().numpy().reshape(-1), "codes vs reference kernel")
    want_q, want_s = orc.quantise_fp8(xb, rows, cols)
    assert_bytes_equal(scales.bytes().view(np.uint16), want_s, "row scales vs CPU oracle")
    assert_bytes_equal(out.bytes(), want_q.reshape(-1), "codes vs CPU oracle")


@pytest.mark.parametrize("rows,cols", [(5, 64), (300, 512), (65, 1000), (40, 1792)])
def test_quantise_fp8_narrow_rows_against_the_cpu_oracle(rows, cols):
    """Rows narrower than a reference CTA: the reference kernel reads the wrong source row there, so the
    arbiter is the CPU restatement of the intended recipe."""
    rng = np.random.default_rng(rows * cols)
    xb = normal_bf16(rng, (rows, cols), outlier_channels=2)
    out, scales = Guarded(rows * cols), Guarded(rows * 2)
    dx = dev_bf16(xb)
    assert call("clef_quantise_fp8", stream(), ptr(dx), out.ptr, scales.ptr, rows, cols, BF16) == 0
    torch.cuda.synchronize()
    out.check_guards("codes")
    want_q, want_s = orc.quantise_fp8(xb, rows, cols)
    assert_bytes_equal(scales.bytes().view(np.uint16), want_s, "row scales vs CPU oracle")
    assert_bytes_equal(out.bytes(), want_q.reshape(-1), "codes vs CPU oracle")


@pytest.mark.parametrize("dtype", [BF16, F32], ids=["bf16", "f32"])
@pytest.mark.parametrize("rows,cols", [(1, 6144), (778, 6144), (129, 12288), (65, 1024), (40, 4000)])
def test_swiglu_quantise_fp8_matches_the_reference_kernel(rows, cols, dtype):
    rng = np.random.default_rng(rows + cols + 1)
    gb = to_bf16_bits((rng.standard_normal((rows, cols)) * 2).astype(np.float32))
    ub = normal_bf16(rng, (rows, cols))
    if rows >= 12:
        gb[3, :8] = to_bf16_bits(np.array([60, -60, 88.5, -88.5, 20, -20, 0, -0.0], np.float32))
        ub[4, :] = 0
        ub[5, :] = to_bf16_bits((np.ones(cols) * 1e-30).astype(np.float32))
    gf, uf = dev_f32_from_bits(gb), dev_f32_from_bits(ub)
    ref_q, ref_s = ref_gpu.swiglu_quantise_fp8(gf, uf, rows, cols)
    out, scales = Guarded(rows * cols), Guarded(rows * 2)
    g_in, u_in = (dev_bf16(gb), dev_bf16(ub)) if dtype == BF16 else (gf, uf)
    assert call("clef_swiglu_quantise_fp8", stream(), ptr(g_in), ptr(u_in), out.ptr, scales.ptr, rows, cols, dtype) == 0
    torch.cuda.synchronize()
    out.check_guards("codes")
    scales.check_guards("scales")
    assert_bytes_equal(scales.bytes().view(np.uint16), as_u16(ref_s), "row scales vs reference kernel")
    assert_bytes_equal(out.bytes(), ref_q.cpu().numpy().reshape(-1), "codes vs reference kernel")
    # CPU oracle (expf in place of __expf): scale words equal or adjacent, codes within one step
    want_q, want_s = orc.swiglu_quantise_fp8(gb, ub, rows, cols)
    got_s = scales.bytes().view(np.uint16).astype(np.int32)
    assert np.abs(got_s - want_s.astype(np.int32)).max() <= 1
    same = got_s == want_s
    got_q = out.bytes().reshape(rows, cols)[same].astype(np.int32)
    dq = np.abs((got_q & 0x7F) - (want_q[same].astype(np.int32) & 0x7F))
    assert dq.max() <= 1 and (dq > 0).mean() < 0.01


@pytest.mark.parametrize("dtype", [BF16, F32], ids=["bf16", "f32"])
@pytest.mark.parametrize("rows", [1, 7, 300, 1280])
def test_rms_norm_fp8_bf16_matches_the_reference_kernel(rows, dtype):
    """src/cuda/mod.rs:6925-6960 (the fused norm equals the chain) at the reference's own row counts, cols 4096."""
    cols = 4096
    rng = np.random.default_rng(rows)
    xb = normal_bf16(rng, (rows, cols), outlier_channels=4)
    special_rows(xb, rows, cols)
    w = (rng.standard_normal(cols) * 0.3).astype(np.float32)
    dw, xf = torch.from_numpy(w).cuda(), dev_f32_from_bits(xb)
    ref_q, ref_s, ref_bf = ref_gpu.rms_norm_fp8_bf16(xf, dw, rows, cols, 1e-6)
    q, qs, bf = Guarded(rows * cols), Guarded(rows * 2), Guarded(rows * cols * 2)
    src = dev_bf16(xb) if dtype == BF16 else xf
    assert call("clef_rms_norm_fp8_bf16", stream(), ptr(src), ptr(dw), q.ptr, qs.ptr, bf.ptr, rows, cols, 1e-6, dtype) == 0
    torch.cuda.synchronize()
    for g, name in ((q, "codes"), (qs, "scales"), (bf, "bf16")):
        g.check_guards(name)
    finite_rows = np.ones(rows, bool)
    if rows >= 12:
        finite_rows[[5, 6]] = False          # inf / NaN rows: the bf16 twin's NaN pattern is not part of the contract
    assert_bytes_equal(qs.bytes().view(np.uint16), as_u16(ref_s), "row scales vs reference kernel")
    assert_bytes_equal(q.bytes(), ref_q.cpu().numpy().reshape(-1), "codes vs reference kernel")
    assert_bytes_equal(bf.bytes().view(np.uint16).reshape(rows, cols)[finite_rows], as_u16(ref_bf).reshape(rows, cols)[finite_rows],
                       "bf16 twin vs reference kernel")
    # the chain of this library's own entry points gives the same bytes
    dev = clef.Device(0)
    normed = dev.rms_norm_dev(xf, dw, rows, cols, 1e-6)
    cq, cs = dev.quantise_fp8_dev(normed, rows, cols)
    assert_bytes_equal(q.bytes(), cq.cpu().numpy().reshape(-1), "codes vs rms_norm -> quantise_fp8")
    assert_bytes_equal(qs.bytes().view(np.uint16), as_u16(cs), "scales vs rms_norm -> quantise_fp8")
    want_q, want_s, want_bf = orc.rms_norm_fp8_bf16(xb, w, rows, cols, 1e-6)
    assert_bytes_equal(qs.bytes().view(np.uint16), want_s, "row scales vs CPU oracle")
    assert_bytes_equal(q.bytes(), want_q.reshape(-1), "codes vs CPU oracle")
    assert_bytes_equal(bf.bytes().view(np.uint16).reshape(rows, cols)[finite_rows], want_bf[finite_rows], "bf16 twin vs CPU oracle")


@pytest.mark.parametrize("rows,cols", [(65, 2048), (40, 1024), (9, 8192)])
def test_rms_norm_fp8_bf16_other_widths_equal_the_chain(rows, cols):
    """Widths the reference declines: the arbiter is rms_norm_kernel (reference, f32) -> quantise_fp8 recipe."""
    rng = np.random.default_rng(cols)
    xb = normal_bf16(rng, (rows, cols), outlier_channels=2)
    w = (rng.standard_normal(cols) * 0.1).astype(np.float32)
    dw, dx = torch.from_numpy(w).cuda(), dev_bf16(xb)
    q, qs, bf = Guarded(rows * cols), Guarded(rows * 2), Guarded(rows * cols * 2)
    assert call("clef_rms_norm_fp8_bf16", stream(), ptr(dx), ptr(dw), q.ptr, qs.ptr, bf.ptr, rows, cols, 1e-6, BF16) == 0
    torch.cuda.synchronize()
    normed = ref_gpu.rms_norm(dev_f32_from_bits(xb), dw, rows, cols, 1e-6)
    want_q, want_s = orc.quantise_fp8(normed.cpu().numpy(), rows, cols)
    assert_bytes_equal(qs.bytes().view(np.uint16), want_s, "row scales vs reference norm + recipe")
    assert_bytes_equal(q.bytes(), want_q.reshape(-1), "codes vs reference norm + recipe")
    assert_bytes_equal(bf.bytes().view(np.uint16), as_u16(normed.to(torch.bfloat16)).reshape(-1), "bf16 twin")
    # without the twin output
    q2, qs2 = Guarded(rows * cols), Guarded(rows * 2)
    assert call("clef_rms_norm_fp8_bf16", stream(), ptr(dx), ptr(dw), q2.ptr, qs2.ptr, None, rows, cols, 1e-6, BF16) == 0
    torch.cuda.synchronize()
    assert_bytes_equal(q2.bytes(), q.bytes(), "codes without the bf16 twin")


@pytest.mark.parametrize("dtype", [BF16, F32], ids=["bf16", "f32"])
@pytest.mark.parametrize("tokens,vh", [(1, 32), (300, 32), (778, 32), (65, 16), (33, 5)])
def test_rms_norm_gated_quantise_fp8_matches_the_reference_kernel(tokens, vh, dtype):
    cols = 128
    rows = tokens * vh
    rng = np.random.default_rng(tokens * vh)
    xb = normal_bf16(rng, (rows, cols), outlier_channels=2)
    gb = to_bf16_bits((rng.standard_normal((rows, cols)) * 2).astype(np.float32))
    if tokens >= 33:
        xb[vh * 2: vh * 3] = 0                     # a token of zeros
        gb[vh * 3, :4] = to_bf16_bits(np.array([70, -70, 30, -30], np.float32))
    w = (1.0 + rng.standard_normal(cols) * 0.1).astype(np.float32)
    dw, xf, gf = torch.from_numpy(w).cuda(), dev_f32_from_bits(xb), dev_f32_from_bits(gb)
    ref_q, ref_s = ref_gpu.rms_norm_gated_quantise_fp8(xf, gf, dw, rows, cols, vh, 1e-6)
    out, scales = Guarded(rows * cols), Guarded(tokens * 2)
    x_in, g_in = (dev_bf16(xb), dev_bf16(gb)) if dtype == BF16 else (xf, gf)
    assert call("clef_rms_norm_gated_quantise_fp8", stream(), ptr(x_in), ptr(g_in), ptr(dw), out.ptr, scales.ptr, rows, cols,
                1e-6, vh, rows, dtype) == 0
    torch.cuda.synchronize()
    out.check_guards("codes")
    scales.check_guards("scales")
    assert_bytes_equal(scales.bytes().view(np.uint16), as_u16(ref_s), "token scales vs reference kernel")
    assert_bytes_equal(out.bytes(), ref_q.cpu().numpy().reshape(-1), "codes vs reference kernel")
    # CPU oracle (expf and IEEE division in place of the intrinsics): adjacent at most
    want_q, want_s = orc.rms_norm_gated_quantise_fp8(xb, gb, w, rows, cols, vh, 1e-6)
    got_s = scales.bytes().view(np.uint16).astype(np.int32)
    assert np.abs(got_s - want_s.astype(np.int32)).max() <= 1
    same = np.repeat(got_s == want_s, vh)
    dq = np.abs((out.bytes().reshape(rows, cols)[same].astype(np.int32) & 0x7F) - (want_q[same].astype(np.int32) & 0x7F))
    assert dq.max() <= 1 and (dq > 0).mean() < 0.01


def test_rms_norm_gated_quantise_fp8_ragged_tail_and_errors():
    """rows_live below rows: the dead head rows add nothing to the amax and their bytes stay untouched."""
    cols, vh, tokens = 128, 8, 5
    rows, live = tokens * vh, tokens * vh - 11
    rng = np.random.default_rng(9)
    xb, gb = normal_bf16(rng, (rows, cols)), normal_bf16(rng, (rows, cols))
    w = np.ones(cols, np.float32)
    out, scales = Guarded(rows * cols), Guarded(tokens * 2)
    dx, dg, dw = dev_bf16(xb), dev_bf16(gb), torch.from_numpy(w).cuda()
    assert call("clef_rms_norm_gated_quantise_fp8", stream(), ptr(dx), ptr(dg), ptr(dw), out.ptr, scales.ptr, rows, cols, 1e-6, vh,
                live, BF16) == 0
    torch.cuda.synchronize()
    out.check_guards("codes")
    got = out.bytes().reshape(rows, cols)
    assert (got[live:] == 0xA5).all()                      # the poison of the guarded buffer: never written
    want_q, want_s = orc.rms_norm_gated_quantise_fp8(xb, gb, w, rows, cols, vh, 1e-6, rows_live=live)
    assert np.abs(scales.bytes().view(np.uint16).astype(np.int32) - want_s.astype(np.int32)).max() <= 1
    lib = clef.load()
    assert lib.clef_rms_norm_gated_quantise_fp8(stream(), ptr(dx), ptr(dg), ptr(dw), out.ptr, scales.ptr, rows, 512, 1e-6, vh, rows, BF16) == -3
    assert lib.clef_rms_norm_gated_quantise_fp8(stream(), ptr(dx), ptr(dg), ptr(dw), out.ptr, scales.ptr, rows + 1, cols, 1e-6, vh, rows, BF16) == -1
    assert lib.clef_quantise_fp8(stream(), ptr(dx), out.ptr, scales.ptr, 4, 100, BF16) == -1
    assert lib.clef_quantise_fp8(stream(), ptr(dx), out.ptr, scales.ptr, 4, 32768, BF16) == -3


def test_fp8_quantisers_on_arbitrary_f32_values():
    """f32 activations that are not bf16 values (GEMM accumulators), at the widths the tuned f32 kernels serve and
    8,192 rows (grid-stride loops, ragged last CTA): codes, scales and the bf16 twin against the reference's own
    kernels, bit for bit. Gates beyond +-44, infinities, NaN, zero rows and tiny rows take the literal paths."""
    dev = clef.Device(0)

    def general(fn, *args):
        """The same entry point on the shape-general kernels (each compared with the reference kernels elsewhere)."""
        clef.set_kernel_choice(1)
        try:
            got = fn(*args)
            torch.cuda.synchronize()
        finally:
            clef.set_kernel_choice(0)
        return got

    def spoil(t):
        t[2] = 0.0
        t[3, 5] = 3.0e38
        t[4] = 1e-39
        t[5, 9] = float("inf")
        t[6, 11] = float("nan")
        t[7] = 1e-30
        t[9] = -0.0

    for rows in (8192, 333):
        gen = torch.Generator(device="cuda").manual_seed(rows + 17)
        # plain and SwiGLU: one width per blocks-per-lane / warps-per-row shape
        for cols in (512, 1536, 2048, 4096, 6144, 12288):
            if rows == 8192 and cols not in (2048, 6144):
                continue
            gate = torch.randn(rows, cols, device="cuda", generator=gen) * 3.0
            up = torch.randn(rows, cols, device="cuda", generator=gen) * 2.0
            gate[:, 7] *= 25.0                      # |g| beyond the short form's range in every row
            spoil(gate)
            up[8, 100] = float("inf")
            up[10, 120] = float("nan")
            up[11] = 0.0
            q, s = dev.quantise_fp8_dev(gate, rows, cols)
            # the reference's launch is one row per CTA above 1792 columns only
            rq, rs = ref_gpu.quantise_fp8(gate, rows, cols) if cols > 1792 else general(dev.quantise_fp8_dev, gate, rows, cols)
            assert torch.equal(s, rs) and torch.equal(q, rq), f"plain, {rows} x {cols}"
            q, s = dev.swiglu_quantise_fp8_dev(gate, up, rows, cols)
            rq, rs = ref_gpu.swiglu_quantise_fp8(gate, up, rows, cols)
            assert torch.equal(s, rs) and torch.equal(q, rq), f"SwiGLU, {rows} x {cols}"
        # RMSNorm with the bf16 twin: the reference kernel at 4096, the chain of the general kernels at 2048
        for cols in (2048, 4096):
            x = torch.randn(rows, cols, device="cuda", generator=gen) * 1.5
            x[:, 3] *= 40.0
            spoil(x)
            w = torch.randn(cols, device="cuda", generator=gen) * 0.3
            q, s, bf = Guarded(rows * cols), Guarded(rows * 2), Guarded(rows * cols * 2)
            assert call("clef_rms_norm_fp8_bf16", stream(), ptr(x), ptr(w), q.ptr, s.ptr, bf.ptr, rows, cols, 1e-6, F32) == 0
            torch.cuda.synchronize()
            for g, name in ((q, "codes"), (s, "scales"), (bf, "bf16")):
                g.check_guards(name)
            finite = np.ones(rows, bool)
            finite[[5, 6]] = False
            if cols == 4096:
                rq, rs, rbf = ref_gpu.rms_norm_fp8_bf16(x, w, rows, cols, 1e-6)
                want_q, want_s, want_bf = rq.cpu().numpy().reshape(-1), as_u16(rs), as_u16(rbf).reshape(rows, cols)
            else:
                g_q, g_s, g_bf = Guarded(rows * cols), Guarded(rows * 2), Guarded(rows * cols * 2)
                assert general(call, "clef_rms_norm_fp8_bf16", stream(), ptr(x), ptr(w), g_q.ptr, g_s.ptr, g_bf.ptr, rows,
                               cols, 1e-6, F32) == 0
                want_q, want_s, want_bf = g_q.bytes(), g_s.bytes().view(np.uint16), g_bf.bytes().view(np.uint16).reshape(rows, cols)
            assert_bytes_equal(s.bytes().view(np.uint16), want_s, f"norm scales, {rows} x {cols}")
            assert_bytes_equal(q.bytes(), want_q, f"norm codes, {rows} x {cols}")
            assert_bytes_equal(bf.bytes().view(np.uint16).reshape(rows, cols)[finite], want_bf[finite], f"bf16 twin, {rows} x {cols}")
        # gated norm: 128-wide heads, every team shape
        for vh in (8, 16, 32, 64):
            tokens = rows if vh <= 32 else rows // 4
            hr = tokens * vh
            x = torch.randn(hr, 128, device="cuda", generator=gen) * 1.5
            g = torch.randn(hr, 128, device="cuda", generator=gen) * 3.0
            g[:, 7] *= 25.0
            spoil(x)
            g[vh * 3 + 1, 40] = float("inf")
            g[vh * 4 + 1, 41] = float("nan")
            x[vh * 5: vh * 6] = 0.0               # a token of zeros
            w = 1.0 + torch.randn(128, device="cuda", generator=gen) * 0.1
            out, scales = Guarded(hr * 128), Guarded(tokens * 2)
            assert call("clef_rms_norm_gated_quantise_fp8", stream(), ptr(x), ptr(g), ptr(w), out.ptr, scales.ptr, hr, 128,
                        1e-6, vh, hr, F32) == 0
            torch.cuda.synchronize()
            out.check_guards("codes")
            scales.check_guards("scales")
            if vh <= 32:
                rq, rs = ref_gpu.rms_norm_gated_quantise_fp8(x, g, w, hr, 128, vh, 1e-6)
                want_q, want_s = rq.cpu().numpy().reshape(-1), as_u16(rs)
            else:                                  # beyond the reference's launch: the general kernel
                g_out, g_scales = Guarded(hr * 128), Guarded(tokens * 2)
                assert general(call, "clef_rms_norm_gated_quantise_fp8", stream(), ptr(x), ptr(g), ptr(w), g_out.ptr,
                               g_scales.ptr, hr, 128, 1e-6, vh, hr, F32) == 0
                want_q, want_s = g_out.bytes(), g_scales.bytes().view(np.uint16)
            assert_bytes_equal(scales.bytes().view(np.uint16), want_s, f"gated scales, {tokens} tokens x {vh}")
            assert_bytes_equal(out.bytes(), want_q, f"gated codes, {tokens} tokens x {vh}")
            del x, g, out, scales


def test_fp8_full_size():
    """130,712 rows: codes and scales of the plain and the SwiGLU quantiser against the reference kernels."""
    rows = 130712
    gen = torch.Generator(device="cuda")
    gen.manual_seed(rows)
    dev = clef.Device(0)
    x = torch.randn(rows, 2048, device="cuda", generator=gen).to(torch.bfloat16)
    q, s = dev.quantise_fp8_dev(x, rows, 2048)
    rq, rs = ref_gpu.quantise_fp8(x.float(), rows, 2048)
    assert torch.equal(q, rq) and torch.equal(s, rs)
    del x, q, s, rq, rs
    gate = torch.randn(rows, 6144, device="cuda", generator=gen).to(torch.bfloat16)
    up = torch.randn(rows, 6144, device="cuda", generator=gen).to(torch.bfloat16)
    q, s = dev.swiglu_quantise_fp8_dev(gate, up, rows, 6144)
    rq, rs = ref_gpu.swiglu_quantise_fp8(gate.float(), up.float(), rows, 6144)
    assert torch.equal(q, rq) and torch.equal(s, rs)
