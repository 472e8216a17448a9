"""Parity of the steps either side of the fused quantisers through the C-ABI: the bf16 KV-cache write (alone and
fused behind the key-side RoPE / qk-norm RoPE), sigmoid_mul with and without the NVFP4 quantiser, the residual add
with and without the next RMSNorm + quantiser.

Each fused entry point must give the bytes of the reference's own kernel CHAIN run on the same GPU
(oracle/_ref: rope_kernel -> to_bf16(_scatter)_kernel, sigmoid_mul_kernel -> quantise_nvfp4_kernel, add_kernel ->
rms_norm_kernel -> quantise_nvfp4_kernel), with bf16 inputs widened exactly to the f32 the reference kernels take,
and agree with the CPU oracle (exactly where the arithmetic has no approximate intrinsic).
"""
import numpy as np
import pytest
import torch

import aiis_clef_b200 as clef
from oracle import binding as orc
from oracle import ref_gpu
from gpu_util import Guarded, call, dev_bf16, dev_f32_from_bits, explain_mismatches, f32_to_bf16_bits_gpu, ptr, stream
from util import assert_bytes_equal, bf16_ulp_distance, normal_bf16, to_bf16_bits

pytestmark = pytest.mark.gpu
BF16, F32 = 0, 1
FILL = -16512          # bf16 -1.0 (0xBF80) as int16: what an untouched cache element holds


@pytest.fixture(autouse=True)
def _reset_choice():
    clef.set_kernel_choice(0)
    yield
    clef.set_kernel_choice(0)
    torch.cuda.empty_cache()


def i32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()


def cache_case(rng, tokens, slots_rows):
    """A position map as the engine builds it: distinct cache rows, not monotonic."""
    return rng.permutation(slots_rows)[:tokens].astype(np.int32)


# ---- to_bf16 / to_bf16_scatter --------------------------------------------------------------------------------
@pytest.mark.parametrize("n,off,stride", [(8, None, 0), (4096 + 5, None, 0), (778 * 256, 3, 256), (130712 * 8, 0, 8)])
def test_to_bf16_matches_the_reference_kernel(n, off, stride):
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 3).astype(np.float32)
    x[:4] = [np.inf, -np.inf, np.nan, -0.0][: min(4, n)]
    dx = torch.from_numpy(x).cuda()
    cap = n + (off or 0) * stride
    off_dev = None if off is None else i32([off])
    want = torch.full((cap + 16,), -1.0, dtype=torch.bfloat16, device="cuda")
    ref_gpu.to_bf16(dx, want, n, off_dev, stride)
    got = Guarded((cap + 16) * 2)
    got.payload().view(torch.int16)[:] = FILL
    assert call("clef_to_bf16", stream(), got.ptr, ptr(dx), n, ptr(off_dev), stride, F32) == 0
    torch.cuda.synchronize()
    got.check_guards("to_bf16")
    assert_bytes_equal(got.as_bf16_bits(), want.cpu().view(torch.int16).numpy().view(np.uint16), "to_bf16 vs reference kernel")
    # bf16 input: a copy to the offset
    xb = to_bf16_bits(x)
    got2 = Guarded((cap + 16) * 2)
    got2.payload().view(torch.int16)[:] = FILL
    dxb = dev_bf16(xb)
    assert call("clef_to_bf16", stream(), got2.ptr, ptr(dxb), n, ptr(off_dev), stride, BF16) == 0
    torch.cuda.synchronize()
    base = (off or 0) * stride
    assert_bytes_equal(got2.as_bf16_bits()[base:base + n], xb, "to_bf16 of bf16 input")
    # CPU oracle
    cpu = np.full(cap + 16, 0xBF80, np.uint16)
    orc.to_bf16_rows(x, cpu, off_tokens=off, stride=stride)
    assert_bytes_equal(got.as_bf16_bits(), cpu, "to_bf16 vs CPU oracle")


@pytest.mark.parametrize("dtype", [BF16, F32], ids=["bf16", "f32"])
@pytest.mark.parametrize("tokens,stride", [(1, 8), (778, 256), (129, 2 * 128), (8192, 256), (300, 1024)])
def test_to_bf16_scatter_matches_the_reference_kernel(tokens, stride, dtype):
    rng = np.random.default_rng(tokens + stride)
    cache_rows = tokens + 37
    xb = normal_bf16(rng, (tokens, stride))
    xf = dev_f32_from_bits(xb)
    pm = cache_case(rng, tokens, cache_rows)
    dpm = i32(pm)
    want = torch.full((cache_rows * stride,), -1.0, dtype=torch.bfloat16, device="cuda")
    ref_gpu.to_bf16_scatter(xf, want, tokens * stride, dpm, stride)
    got = Guarded(cache_rows * stride * 2)
    got.payload().view(torch.int16)[:] = FILL
    src = dev_bf16(xb) if dtype == BF16 else xf
    assert call("clef_to_bf16_scatter", stream(), got.ptr, ptr(src), tokens * stride, ptr(dpm), stride, dtype) == 0
    torch.cuda.synchronize()
    assert_bytes_equal(got.as_bf16_bits(), want.cpu().view(torch.int16).numpy().view(np.uint16), "scatter vs reference kernel")
    cpu = np.full(cache_rows * stride, 0xBF80, np.uint16)
    orc.to_bf16_rows(xb, cpu, pos_map=pm, stride=stride)
    assert_bytes_equal(got.as_bf16_bits(), cpu, "scatter vs CPU oracle")


def test_to_bf16_argument_errors():
    x = torch.zeros(64, device="cuda")
    out = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    pm = i32([0, 1])
    lib = clef.load()
    assert lib.clef_to_bf16_scatter(stream(), ptr(out), ptr(x), 64, ptr(pm), 12, F32) == -1      # stride % 8
    assert lib.clef_to_bf16_scatter(stream(), ptr(out), ptr(x), 60, ptr(pm), 32, F32) == -1      # n % stride
    assert lib.clef_to_bf16_scatter(stream(), ptr(out), ptr(x), 64, None, 32, F32) == -1         # no map
    assert lib.clef_to_bf16(stream(), None, ptr(x), 64, None, 0, F32) == -1
    assert lib.clef_to_bf16(stream(), ptr(out), ptr(x), 0, None, 0, F32) == 0


# ---- RoPE + KV-cache write ---------------------------------------------------------------------------------------
def rope_setup(rng, tokens, rot, table_rows):
    pos = rng.integers(0, table_rows, tokens).astype(np.int32)
    dev = clef.Device(0)
    cos, sin = dev.rope_tables_dev(i32(np.arange(table_rows)), table_rows, rot, 1e7)
    return pos, cos, sin


@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("dtype", [BF16, F32], ids=["bf16", "f32"])
@pytest.mark.parametrize("mode", ["map", "len", "plain"])
@pytest.mark.parametrize("tokens,heads,hd,rot", [(1, 2, 128, 64), (778, 2, 128, 64), (129, 2, 256, 64), (65, 4, 64, 64), (300, 1, 96, 32), (33, 2, 40, 16)])
def test_rope_kv_write_equals_the_reference_chain(tokens, heads, hd, rot, mode, dtype, choice):
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(tokens * 7 + hd + rot)
    kb, vb = normal_bf16(rng, (tokens, heads, hd)), normal_bf16(rng, (tokens, heads, hd))
    kf, vf = dev_f32_from_bits(kb), dev_f32_from_bits(vb)
    pos, cos, sin = rope_setup(rng, tokens, rot, 512)
    dpos = i32(pos)
    stride = heads * hd
    cache_rows = tokens + 21
    cmap = clen = None
    if mode == "map":
        cmap = i32(cache_case(rng, tokens, cache_rows))
    elif mode == "len":
        clen = i32([17])
    # reference chain: rope_kernel (f32) -> to_bf16(_scatter)_kernel for k; to_bf16(_scatter)_kernel for v
    k_rot = ref_gpu.rope(kf, cos, sin, tokens, heads, hd, rot, None, None, dpos)
    want_k = torch.full((cache_rows * stride,), -1.0, dtype=torch.bfloat16, device="cuda")
    want_v = torch.full((cache_rows * stride,), -1.0, dtype=torch.bfloat16, device="cuda")
    for src, dst in ((k_rot.reshape(-1), want_k), (vf.reshape(-1), want_v)):
        if cmap is not None:
            ref_gpu.to_bf16_scatter(src, dst, tokens * stride, cmap, stride)
        else:
            ref_gpu.to_bf16(src, dst, tokens * stride, clen, stride)
    got_k, got_v = Guarded(cache_rows * stride * 2), Guarded(cache_rows * stride * 2)
    got_k.payload().view(torch.int16)[:] = FILL
    got_v.payload().view(torch.int16)[:] = FILL
    k_in, v_in = (dev_bf16(kb), dev_bf16(vb)) if dtype == BF16 else (kf, vf)
    assert call("clef_rope_kv_write", stream(), got_k.ptr, got_v.ptr, ptr(k_in), ptr(v_in), ptr(cos), ptr(sin), tokens, heads,
                hd, rot, None, None, ptr(dpos), ptr(cmap), ptr(clen), dtype) == 0
    torch.cuda.synchronize()
    got_k.check_guards("cache_k")
    got_v.check_guards("cache_v")
    wk = want_k.cpu().view(torch.int16).numpy().view(np.uint16)
    wv = want_v.cpu().view(torch.int16).numpy().view(np.uint16)
    assert_bytes_equal(got_v.as_bf16_bits(), wv, "value cache vs reference chain")
    assert_bytes_equal(got_k.as_bf16_bits(), wk, "key cache vs reference chain")


@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("dtype", [BF16, F32], ids=["bf16", "f32"])
@pytest.mark.parametrize("mode", ["map", "len"])
@pytest.mark.parametrize("tokens,heads,hd,rot", [(4, 2, 128, 64), (778, 2, 128, 64), (129, 2, 256, 64), (776, 2, 256, 64), (4, 2, 256, 64), (65, 3, 128, 64), (40, 4, 64, 32)])
def test_qk_norm_rope_kv_write_equals_the_unfused_calls(tokens, heads, hd, rot, mode, dtype, choice):
    """k_raw -> clef_qk_norm_rope (itself checked against the reference kernels elsewhere) -> to_bf16(_scatter)
    must equal the one-launch entry point byte for byte; the f32 path is additionally the reference chain."""
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(tokens * 11 + hd)
    kb, vb = normal_bf16(rng, (tokens * heads, hd)), normal_bf16(rng, (tokens * heads, hd))
    w = (rng.standard_normal(hd) * 0.1).astype(np.float32)
    dw = torch.from_numpy(w).cuda()
    pos, cos, sin = rope_setup(rng, tokens, rot, 300)
    dpos = i32(pos)
    stride = heads * hd
    cache_rows = tokens + 9
    cmap = i32(cache_case(rng, tokens, cache_rows)) if mode == "map" else None
    clen = i32([5]) if mode == "len" else None
    dev = clef.Device(0)
    k_in, v_in = (dev_bf16(kb), dev_bf16(vb)) if dtype == BF16 else (dev_f32_from_bits(kb), dev_f32_from_bits(vb))
    k_rot, _ = dev.qk_norm_rope_dev(k_in, dw, cos, sin, tokens * heads, heads, hd, rot, 1e-6, pos_map=dpos)
    want_k = torch.full((cache_rows * stride,), -1.0, dtype=torch.bfloat16, device="cuda")
    want_v = torch.full((cache_rows * stride,), -1.0, dtype=torch.bfloat16, device="cuda")
    for src, dst in ((k_rot.float().reshape(-1), want_k), (v_in.float().reshape(-1), want_v)):
        if cmap is not None:
            ref_gpu.to_bf16_scatter(src, dst, tokens * stride, cmap, stride)
        else:
            ref_gpu.to_bf16(src, dst, tokens * stride, clen, stride)
    got_k, got_v = Guarded(cache_rows * stride * 2), Guarded(cache_rows * stride * 2)
    got_k.payload().view(torch.int16)[:] = FILL
    got_v.payload().view(torch.int16)[:] = FILL
    assert call("clef_qk_norm_rope_kv_write", stream(), got_k.ptr, got_v.ptr, ptr(k_in), ptr(v_in), ptr(dw), ptr(cos), ptr(sin),
                tokens, heads, hd, rot, 1e-6, None, None, ptr(dpos), ptr(cmap), ptr(clen), dtype) == 0
    torch.cuda.synchronize()
    got_k.check_guards("cache_k")
    got_v.check_guards("cache_v")
    assert_bytes_equal(got_v.as_bf16_bits(), want_v.cpu().view(torch.int16).numpy().view(np.uint16), "value cache")
    assert_bytes_equal(got_k.as_bf16_bits(), want_k.cpu().view(torch.int16).numpy().view(np.uint16), "key cache")


# ---- sigmoid_mul ---------------------------------------------------------------------------------------------------
def test_sigmoid_mul_short_form_is_exact_for_every_bf16_pair_of_its_domain():
    """Every (gate, x) pair of bf16 values with |gate| <= 44 and x zero or 2^-60 <= |x| < inf, on the device."""
    all_pairs, domain = ref_gpu.probe_sigmoid_mul_bf16()
    assert domain["checked"] > 1_500_000_000 and domain["mismatches"] == 0, domain
    assert all_pairs["mismatches"] > 0     # outside the domain the short form does differ: the gate is needed


@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("total", [3, 16, 4099, 778 * 4096, 129 * 4096 + 2])
def test_sigmoid_mul(total, choice):
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(total)
    xb = normal_bf16(rng, (total,))
    gb = to_bf16_bits((rng.standard_normal(total) * 4).astype(np.float32))
    if total > 100:
        gb[:8] = to_bf16_bits(np.array([50, -50, 88.5, -88.5, np.inf, -np.inf, np.nan, 0], np.float32))
        xb[8:14] = to_bf16_bits(np.array([0.0, -0.0, 1e-30, -1e-25, np.inf, np.nan], np.float32))
        gb[40:48] = to_bf16_bits(np.array([-43, -40, -30, 43, 12, -12, 1, -1], np.float32))
        xb[40:44] = to_bf16_bits(np.array([1e-20, -3e-19, 1e-38, 9e-41], np.float32))
    xf, gf = dev_f32_from_bits(xb), dev_f32_from_bits(gb)
    ref = ref_gpu.sigmoid_mul(xf, gf, total)
    # f32: bit-exact against the reference kernel (NaN payloads aside: compare as bits where both are not NaN)
    outf = Guarded(total * 4)
    assert call("clef_sigmoid_mul", stream(), outf.ptr, ptr(xf), ptr(gf), total, F32) == 0
    torch.cuda.synchronize()
    outf.check_guards("sigmoid_mul f32")
    got, want = outf.as_f32(), ref.cpu().numpy()
    nan = np.isnan(want)
    assert (np.isnan(got) == nan).all()
    assert_bytes_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan], "f32 sigmoid_mul vs reference kernel")
    # bf16: the reference f32 result rounded to nearest even, zero signs aside
    out = Guarded(total * 2)
    dxb, dgb = dev_bf16(xb), dev_bf16(gb)
    assert call("clef_sigmoid_mul", stream(), out.ptr, ptr(dxb), ptr(dgb), total, BF16) == 0
    torch.cuda.synchronize()
    out.check_guards("sigmoid_mul bf16")
    d = bf16_ulp_distance(out.as_bf16_bits()[~nan], f32_to_bf16_bits_gpu(ref)[~nan])
    assert d.max() == 0, f"{int((d > 0).sum())} bf16 results differ from the rounded reference result"
    # CPU oracle (expf in place of __expf): within 1 bf16 ulp
    _, cpu = orc.sigmoid_mul(xb, gb)
    finite = ~nan & np.isfinite(want)
    assert bf16_ulp_distance(out.as_bf16_bits()[finite], cpu[finite]).max() <= 1


@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("dtype", [BF16, F32], ids=["bf16", "f32"])
@pytest.mark.parametrize("rows,cols", [(1, 64), (778, 4096), (129, 2048), (300, 512), (65, 1088), (8192, 4096)])
def test_sigmoid_mul_quantise_equals_the_reference_chain(rows, cols, dtype, choice):
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(rows + cols)
    xb = normal_bf16(rng, (rows, cols), outlier_channels=2)
    gb = to_bf16_bits((rng.standard_normal((rows, cols)) * 4).astype(np.float32))
    if rows >= 65:
        gb[3, :16] = to_bf16_bits(np.linspace(-60, 60, 16).astype(np.float32))     # outside the short form
        xb[5, 16:32] = 0                                                              # an all-zero block
        xb[7, 32:40] = to_bf16_bits(np.array([1e-30, -1e-25, 3e-39, 0, -0.0, 1e-19, -1e-18, 1], np.float32))
        xb[9, :] = 0                                                                  # a zero row
        xb[11, 48:64] = to_bf16_bits((np.ones(16) * 1e-30).astype(np.float32))      # a block of tiny values only
    gs = 448.0 * 6.0 / 8.0
    xf, gf = dev_f32_from_bits(xb), dev_f32_from_bits(gb)
    act = ref_gpu.sigmoid_mul(xf, gf, rows * cols)
    ref_p, ref_s = ref_gpu.quantise_nvfp4(act, rows, cols, gs)
    rp, pbytes, sbytes = rows + (-rows % 128), (rows + (-rows % 128)) * cols // 2, (rows + (-rows % 128)) * cols // 16
    packed, scales = Guarded(pbytes), Guarded(sbytes)
    x_in, g_in = (dev_bf16(xb), dev_bf16(gb)) if dtype == BF16 else (xf, gf)
    assert call("clef_sigmoid_mul_quantise_nvfp4", stream(), ptr(x_in), ptr(g_in), packed.ptr, scales.ptr, rows, cols, gs, 128,
                512, dtype) == 0
    torch.cuda.synchronize()
    packed.check_guards("packed")
    scales.check_guards("scales")
    assert_bytes_equal(scales.bytes(), ref_s.cpu().numpy(), "scales vs reference chain")
    assert_bytes_equal(packed.bytes(), ref_p.cpu().numpy(), "packed codes vs reference chain")
    if rows <= 778:
        # CPU oracle, boundary-aware (expf in place of __expf)
        want_p, want_s, pre = orc.sigmoid_mul_quantise_nvfp4(xb, gb, rows, cols, gs, want_pre=True)
        n_scale, n_code, unexplained = explain_mismatches(pre, gs, packed.bytes(), scales.bytes(), want_p, want_s, rows, cols)
        assert unexplained == 0, (n_scale, n_code, unexplained)
        assert n_scale + n_code <= max(4, rows * cols // 2000)


# ---- add, add + RMSNorm + NVFP4 ----------------------------------------------------------------------------------------
@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("total", [1, 16, 4099, 778 * 2048, 129 * 2048 + 3])
def test_add(total, choice):
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(total)
    ab, bb = normal_bf16(rng, (total,)), normal_bf16(rng, (total,))
    af, bf = dev_f32_from_bits(ab), dev_f32_from_bits(bb)
    ref = ref_gpu.add(af, bf, total)
    outf = Guarded(total * 4)
    assert call("clef_add", stream(), outf.ptr, ptr(af), ptr(bf), total, F32) == 0
    out = Guarded(total * 2)
    da, db = dev_bf16(ab), dev_bf16(bb)
    assert call("clef_add", stream(), out.ptr, ptr(da), ptr(db), total, BF16) == 0
    torch.cuda.synchronize()
    outf.check_guards("add f32")
    out.check_guards("add bf16")
    assert_bytes_equal(outf.as_f32().view(np.uint32), ref.cpu().numpy().view(np.uint32), "f32 add vs reference kernel")
    assert_bytes_equal(out.as_bf16_bits(), f32_to_bf16_bits_gpu(ref), "bf16 add vs rounded reference result")
    f32, cpu = orc.add(ab, bb)
    assert_bytes_equal(out.as_bf16_bits(), cpu, "bf16 add vs CPU oracle")
    # in place: out aliases a
    assert call("clef_add", stream(), ptr(da), ptr(da), ptr(db), total, BF16) == 0
    torch.cuda.synchronize()
    assert_bytes_equal(orc.bf16_bits(da.cpu()), cpu, "in-place add")


@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("dtype", [BF16, F32], ids=["bf16", "f32"])
@pytest.mark.parametrize("rows,cols", [(1, 2048), (778, 2048), (129, 4096), (300, 512), (8192, 2048)])
def test_add_rms_norm_quantise_equals_the_chain(rows, cols, dtype, choice):
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(rows * 3 + cols)
    ab = normal_bf16(rng, (rows, cols), outlier_channels=4)
    bb = normal_bf16(rng, (rows, cols))
    if rows >= 129:
        bb[5] = ab[5] ^ 0x8000          # a row that sums to exact zeros
        ab[7, :64] = 0
        bb[7, :64] = 0
    w = (rng.standard_normal(cols) * 0.1).astype(np.float32)
    dw = torch.from_numpy(w).cuda()
    gs = 448.0 * 6.0 / 30.0
    af, bf = dev_f32_from_bits(ab), dev_f32_from_bits(bb)
    rp = rows + (-rows % 128)
    packed, scales = Guarded(rp * cols // 2), Guarded(rp * cols // 16)
    if dtype == F32:
        # the reference chain itself: add_kernel -> rms_norm_kernel -> quantise_nvfp4_kernel
        total = ref_gpu.add(af, bf, rows * cols)
        normed = ref_gpu.rms_norm(total, dw, rows, cols, 1e-6)
        ref_p, ref_s = ref_gpu.quantise_nvfp4(normed, rows, cols, gs)
        sum_out = Guarded(rows * cols * 4)
        assert call("clef_add_rms_norm_quantise_nvfp4", stream(), sum_out.ptr, ptr(af), ptr(bf), ptr(dw), packed.ptr, scales.ptr,
                    rows, cols, 1e-6, gs, 128, 512, F32) == 0
        torch.cuda.synchronize()
        assert_bytes_equal(sum_out.as_f32().view(np.uint32), total.cpu().numpy().view(np.uint32), "f32 sum vs reference add_kernel")
    else:
        # bf16 residual stream: the stored (rounded) sum is what the norm sees
        total = ref_gpu.add(af, bf, rows * cols).to(torch.bfloat16)
        normed = ref_gpu.rms_norm(total.float(), dw, rows, cols, 1e-6)
        ref_p, ref_s = ref_gpu.quantise_nvfp4(normed, rows, cols, gs)
        sum_out = Guarded(rows * cols * 2)
        da, db = dev_bf16(ab), dev_bf16(bb)
        assert call("clef_add_rms_norm_quantise_nvfp4", stream(), sum_out.ptr, ptr(da), ptr(db), ptr(dw), packed.ptr, scales.ptr,
                    rows, cols, 1e-6, gs, 128, 512, BF16) == 0
        torch.cuda.synchronize()
        assert_bytes_equal(sum_out.as_bf16_bits(), orc.bf16_bits(total.cpu()).reshape(-1), "bf16 sum vs rounded reference add")
    sum_out.check_guards("sum_out")
    packed.check_guards("packed")
    scales.check_guards("scales")
    assert_bytes_equal(scales.bytes(), ref_s.cpu().numpy(), "scales vs reference chain")
    assert_bytes_equal(packed.bytes(), ref_p.cpu().numpy(), "packed codes vs reference chain")
    if dtype == BF16 and rows <= 778:
        # CPU oracle: add, then rms_norm_quantise on the stored sum; no approximate intrinsic on this path -> exact
        _, cpu_sum = orc.add(ab, bb)
        want_p, want_s = orc.rms_norm_quantise_nvfp4(cpu_sum.reshape(rows, cols), w, rows, cols, 1e-6, gs)
        assert_bytes_equal(scales.bytes(), want_s, "scales vs CPU oracle")
        assert_bytes_equal(packed.bytes(), want_p, "packed codes vs CPU oracle")
        # in place: sum_out aliases a
        packed2, scales2 = Guarded(rp * cols // 2), Guarded(rp * cols // 16)
        assert call("clef_add_rms_norm_quantise_nvfp4", stream(), ptr(da), ptr(da), ptr(db), ptr(dw), packed2.ptr, scales2.ptr,
                    rows, cols, 1e-6, gs, 128, 512, BF16) == 0
        torch.cuda.synchronize()
        assert_bytes_equal(orc.bf16_bits(da.cpu()).reshape(-1), cpu_sum.reshape(-1), "in-place residual")
        assert_bytes_equal(packed2.bytes(), want_p, "packed codes, in-place residual")
    if dtype == F32:
        # in place: sum_out aliases a
        packed2, scales2 = Guarded(rp * cols // 2), Guarded(rp * cols // 16)
        a2 = af.clone()
        assert call("clef_add_rms_norm_quantise_nvfp4", stream(), ptr(a2), ptr(a2), ptr(bf), ptr(dw), packed2.ptr, scales2.ptr,
                    rows, cols, 1e-6, gs, 128, 512, F32) == 0
        torch.cuda.synchronize()
        assert torch.equal(a2.reshape(-1).view(torch.int32), total.reshape(-1).view(torch.int32)), "in-place f32 residual"
        assert_bytes_equal(packed2.bytes(), ref_p.cpu().numpy(), "packed codes, in-place f32 residual")
        assert_bytes_equal(scales2.bytes(), ref_s.cpu().numpy(), "scales, in-place f32 residual")


# ---- q and k (and the KV-cache write) in one launch ---------------------------------------------------------------
@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("dtype", [BF16, F32], ids=["bf16", "f32"])
@pytest.mark.parametrize("rows,q_heads,kv_heads,hd,rot", [(1, 16, 2, 128, 64), (778, 16, 2, 128, 64), (129, 8, 2, 256, 64),
                                                           (65, 4, 4, 64, 64), (33, 3, 1, 40, 16), (8192, 16, 2, 128, 64)])
def test_rope_qk_and_rope_qkv_write_equal_the_separate_calls(rows, q_heads, kv_heads, hd, rot, dtype, choice):
    """clef_rope_qk == clef_rope(q), clef_rope(k); clef_rope_qkv_write == clef_rope(q), clef_rope_kv_write(k, v): byte for
    byte (the separate calls are compared with the reference kernels above and in test_gpu_parity_elem.py)."""
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(rows * 13 + hd + q_heads)
    tdt = torch.bfloat16 if dtype == BF16 else torch.float32
    mk = (lambda b: dev_bf16(b)) if dtype == BF16 else (lambda b: dev_f32_from_bits(b))
    q, k, v = (mk(normal_bf16(rng, (rows, h, hd))) for h in (q_heads, kv_heads, kv_heads))
    pos, cos, sin = rope_setup(rng, rows, rot, 700)
    dpos = i32(pos)
    dev = clef.Device(0)
    want_q = dev.rope_apply_dev(q, cos, sin, rows, q_heads, hd, rot, pos_map=dpos)
    want_k = dev.rope_apply_dev(k, cos, sin, rows, kv_heads, hd, rot, pos_map=dpos)
    got_q, got_k = dev.rope_qk_dev(q, k, cos, sin, rows, q_heads, kv_heads, hd, rot, pos_map=dpos)
    torch.cuda.synchronize()
    assert got_q.dtype == tdt and torch.equal(got_q, want_q) and torch.equal(got_k, want_k)
    cache_rows = rows + 11
    cmap = i32(cache_case(rng, rows, cache_rows))
    caches = [torch.full((cache_rows, kv_heads, hd), -1.0, dtype=torch.bfloat16, device="cuda") for _ in range(4)]
    dev.rope_kv_write_dev(caches[0], caches[1], k, v, cos, sin, rows, kv_heads, hd, rot, pos_map=dpos, cache_map=cmap)
    got_q2 = dev.rope_qkv_write_dev(q, caches[2], caches[3], k, v, cos, sin, rows, q_heads, kv_heads, hd, rot, pos_map=dpos,
                                    cache_map=cmap)
    torch.cuda.synchronize()
    assert torch.equal(got_q2, want_q) and torch.equal(caches[2], caches[0]) and torch.equal(caches[3], caches[1])
    # without a map: rows land at *cache_len + t
    clen = i32([7])
    c2 = [torch.full((cache_rows, kv_heads, hd), -1.0, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    dev.rope_qkv_write_dev(q, c2[0], c2[1], k, v, cos, sin, min(rows, 4), q_heads, kv_heads, hd, rot, pos_map=dpos, cache_len=clen)
    torch.cuda.synchronize()
    n = min(rows, 4)
    assert torch.equal(c2[0][7:7 + n], want_k[:n].to(torch.bfloat16)) and torch.equal(c2[1][7:7 + n], v[:n].to(torch.bfloat16))
    assert (c2[0][:7].float() == -1.0).all() and (c2[0][7 + n:].float() == -1.0).all()


# ---- the first layer's gather and norm + quantiser in one pass ------------------------------------------------------------
@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("dtype", [BF16, F32], ids=["bf16", "f32"])
@pytest.mark.parametrize("tokens,hidden,vocab", [(1, 2048, 50), (778, 2048, 32768), (129, 4096, 1000), (8192, 2048, 32768), (65, 1024, 300)])
def test_embed_rms_norm_quantise_equals_the_two_calls(tokens, hidden, vocab, dtype, choice):
    """clef_embed_rms_norm_quantise_nvfp4 == clef_embed_gather, then clef_rms_norm_quantise_nvfp4 on the gathered rows
    (each compared with the reference kernels in test_gpu_parity_*.py), byte for byte, h included; and against the CPU
    oracle of the 778-row configuration's chain."""
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(tokens + hidden)
    tbits = normal_bf16(rng, (vocab, hidden), scale=0.02, outlier_channels=8)
    table = dev_bf16(tbits) if dtype == BF16 else dev_f32_from_bits(tbits)
    ids_np = rng.integers(0, vocab, tokens).astype(np.int32)
    ids_np[-1] = vocab - 1
    ids = i32(ids_np)
    w_np = (rng.standard_normal(hidden) * 0.1).astype(np.float32)
    w = torch.from_numpy(w_np).cuda()
    dev = clef.Device(0)
    gs = 448.0 * 6.0 / 30.0
    want_h = dev.embed_gather_dev(table, ids, tokens, hidden)
    want_p, want_s = dev.rms_norm_quantise_nvfp4_dev(want_h, w, tokens, hidden, 1e-6, gs, 128)
    got_h, got_p, got_s = dev.embed_rms_norm_quantise_nvfp4_dev(table, ids, w, tokens, hidden, 1e-6, gs, 128)
    torch.cuda.synchronize()
    assert got_h.dtype == want_h.dtype and torch.equal(got_h, want_h)
    assert torch.equal(got_p, want_p) and torch.equal(got_s, want_s)
    cpu_p, cpu_s = orc.rms_norm_quantise_nvfp4(tbits[ids_np], w_np, tokens, hidden, 1e-6, gs)
    assert_bytes_equal(got_s.cpu().numpy(), cpu_s, "scales vs CPU oracle")
    assert_bytes_equal(got_p.cpu().numpy().reshape(-1), cpu_p, "packed vs CPU oracle")
    # interleaved scale-tile order per call
    rp = (tokens + 127) // 128 * 128
    pk, sc, h2 = Guarded(rp * hidden // 2), Guarded(rp * hidden // 16), torch.empty_like(want_h)
    assert call("clef_embed_rms_norm_quantise_nvfp4_ex", stream(), ptr(table), ptr(ids), ptr(h2), ptr(w), pk.ptr, sc.ptr, tokens,
                hidden, 1e-6, gs, 128, 512, dtype, 1) == 0
    pk2, sc2 = Guarded(rp * hidden // 2), Guarded(rp * hidden // 16)
    assert call("clef_rms_norm_quantise_nvfp4_ex", stream(), ptr(want_h), ptr(w), pk2.ptr, sc2.ptr, tokens, hidden, 1e-6, gs, 128,
                512, dtype, 1) == 0
    torch.cuda.synchronize()
    pk.check_guards("packed")
    sc.check_guards("scales")
    assert np.array_equal(pk.bytes(), pk2.bytes()) and np.array_equal(sc.bytes(), sc2.bytes()) and torch.equal(h2, want_h)


# ---- device-to-device copies inside a pass (copy_kernel, copy_u8_kernel, copy_range_u8_kernel) -------------------------
@pytest.mark.parametrize("nbytes", [0, 1, 31, 32, 33, 4096, 100003, 8192 * 2048 * 2])
@pytest.mark.parametrize("dst_off,src_off", [(0, 0), (32, 64), (5, 37), (7, 8), (1, 0), (16, 48)])
def test_copy_bytes(nbytes, dst_off, src_off):
    """clef_copy_bytes against a plain slice copy, for offsets that are congruent modulo 32 (the 32-byte path with a
    ragged head and tail) and that are not (the byte path); the bytes either side of the destination range stay."""
    gen = torch.Generator(device="cuda").manual_seed(nbytes + dst_off * 64 + src_off)
    src = torch.randint(0, 256, (nbytes + src_off + 64,), device="cuda", generator=gen, dtype=torch.uint8)
    dst = torch.full((nbytes + dst_off + 64,), 0xA5, device="cuda", dtype=torch.uint8)
    clef.Device(0).copy_bytes_dev(dst, dst_off, src, src_off, nbytes)
    torch.cuda.synchronize()
    assert torch.equal(dst[dst_off:dst_off + nbytes], src[src_off:src_off + nbytes])
    assert (dst[:dst_off] == 0xA5).all() and (dst[dst_off + nbytes:] == 0xA5).all()


def test_copy_bytes_refuses_overlap():
    buf = torch.zeros(1024, device="cuda", dtype=torch.uint8)
    assert clef.load().clef_copy_bytes(stream(), ptr(buf), 0, ptr(buf), 16, 64) == -1
    assert clef.load().clef_copy_bytes(stream(), ptr(buf), 0, ptr(buf), 64, 64) == 0
