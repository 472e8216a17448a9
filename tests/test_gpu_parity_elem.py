"""Parity of the non-quantising entry points (bf16 or f32 in, same dtype out) through the C-ABI.

bf16: the output must be within 1 bf16 ulp (RoPE: 2) of the reference kernel's f32 result rounded
to bf16 (T1, same GPU) and of the CPU oracle's; pass-through data and gathers are bit-exact.
f32 (the reference engine's own dtype): bit-exact against the reference kernels.
"""
import numpy as np
import pytest
import torch

import aiis_clef_b200 as clef
from oracle import binding as orc
from oracle import ref_gpu
from gpu_util import Guarded, call, dev_bf16, dev_f32_from_bits, f32_to_bf16_bits_gpu, ptr, stream
from util import assert_bytes_equal, bf16_ulp_distance, normal_bf16, to_bf16_bits

pytestmark = pytest.mark.gpu
BF16, F32 = 0, 1


@pytest.fixture(autouse=True)
def _reset_choice():
    clef.set_kernel_choice(0)
    yield
    clef.set_kernel_choice(0)


def out_buffer(n_elems, dtype):
    return Guarded(n_elems * (2 if dtype == BF16 else 4))


def check_ulp(got_bits, want_bits, tol, what):
    d = bf16_ulp_distance(got_bits.reshape(-1), want_bits.reshape(-1))
    assert d.max() <= tol, f"{what}: {int((d > tol).sum())} values beyond {tol} bf16 ulp (max {int(d.max())})"


# ---- embed_gather -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("tokens,hidden", [(1, 2048), (778, 2048), (129, 4096), (65, 136), (8192, 2048)])
def test_embed_gather(tokens, hidden, choice):
    clef.set_kernel_choice(choice)
    vocab = 4099
    rng = np.random.default_rng(tokens + hidden)
    table = to_bf16_bits((rng.standard_normal((vocab, hidden)) * 0.02).astype(np.float32))
    ids = rng.integers(0, vocab, tokens).astype(np.int32)
    ids[0], ids[-1] = vocab - 1, 0
    dt, di = dev_bf16(table), torch.from_numpy(ids).cuda()
    out = out_buffer(tokens * hidden, BF16)
    assert call("clef_embed_gather", stream(), ptr(dt), ptr(di), out.ptr, tokens, hidden, BF16) == 0
    torch.cuda.synchronize()
    out.check_guards("embed")
    want = orc.embed_gather(table, ids, tokens, hidden)
    assert_bytes_equal(out.as_bf16_bits(), want, "embedding rows vs CPU oracle")
    tf = dev_f32_from_bits(table)
    ref = ref_gpu.embed_gather(tf, di, tokens, hidden)
    outf = out_buffer(tokens * hidden, F32)
    assert call("clef_embed_gather", stream(), ptr(tf), ptr(di), outf.ptr, tokens, hidden, F32) == 0
    torch.cuda.synchronize()
    assert_bytes_equal(outf.as_f32().view(np.uint32), ref.cpu().numpy().view(np.uint32), "f32 gather vs reference kernel")


# ---- rms_norm -------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("rows,cols", [(5, 128), (778, 2048), (129, 4096), (300, 256), (64, 1000), (33, 6144)])
def test_rms_norm(rows, cols, choice):
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(rows + cols)
    x = normal_bf16(rng, (rows, cols), outlier_channels=4)
    w = (rng.standard_normal(cols) * 0.1).astype(np.float32)
    dx, dw, xf = dev_bf16(x), torch.from_numpy(w).cuda(), dev_f32_from_bits(x)
    ref = ref_gpu.rms_norm(xf, dw, rows, cols, 1e-6)
    out = out_buffer(rows * cols, BF16)
    assert call("clef_rms_norm", stream(), ptr(dx), ptr(dw), out.ptr, rows, cols, 1e-6, BF16) == 0
    torch.cuda.synchronize()
    out.check_guards("rms_norm")
    check_ulp(out.as_bf16_bits(), f32_to_bf16_bits_gpu(ref), 1, "rms_norm vs reference kernel")
    want_f32, want = orc.rms_norm(x, w, rows, cols, 1e-6)
    check_ulp(out.as_bf16_bits(), want, 1, "rms_norm vs CPU oracle")
    # f32: bit-exact against the reference kernel and the CPU oracle
    outf = out_buffer(rows * cols, F32)
    assert call("clef_rms_norm", stream(), ptr(xf), ptr(dw), outf.ptr, rows, cols, 1e-6, F32) == 0
    torch.cuda.synchronize()
    assert_bytes_equal(outf.as_f32().view(np.uint32), ref.cpu().numpy().view(np.uint32), "f32 rms_norm vs reference kernel")
    assert_bytes_equal(outf.as_f32().view(np.uint32), want_f32.view(np.uint32), "f32 rms_norm vs CPU oracle")
    # no weight
    outn = out_buffer(rows * cols, F32)
    assert call("clef_rms_norm", stream(), ptr(xf), None, outn.ptr, rows, cols, 1e-6, F32) == 0
    refn = ref_gpu.rms_norm(xf, None, rows, cols, 1e-6)
    torch.cuda.synchronize()
    assert_bytes_equal(outn.as_f32().view(np.uint32), refn.cpu().numpy().view(np.uint32), "f32 rms_norm without weight")


def test_rms_norm_reference_recipe():
    """src/cuda/mod.rs:7319-7334: 5 x 128 ramps against the f64 model, 1e-4."""
    rows, cols = 5, 128
    i = np.arange(rows * cols)
    x = (((i * 37 % 101).astype(np.float32) - 50.0) / 11.0).reshape(rows, cols)
    w = ((np.arange(cols) % 7).astype(np.float32) - 3.0) / 8.0
    out = out_buffer(rows * cols, F32)
    dx, dw = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    assert call("clef_rms_norm", stream(), ptr(dx), ptr(dw), out.ptr, rows, cols, 1e-6, F32) == 0
    torch.cuda.synchronize()
    want = np.stack([orc.model_rms_norm(x[r], w, 1e-6) for r in range(rows)])
    assert np.abs(out.as_f32().reshape(rows, cols) - want).max() < 1e-4


# ---- rms_norm_gated ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("rows,cols", [(5, 128), (778 * 16, 128), (77, 2048), (300, 256)])
def test_rms_norm_gated(rows, cols, choice):
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(rows + cols)
    x, g = normal_bf16(rng, (rows, cols)), normal_bf16(rng, (rows, cols))
    w = (1.0 + rng.standard_normal(cols) * 0.1).astype(np.float32)
    dx, dg, dw = dev_bf16(x), dev_bf16(g), torch.from_numpy(w).cuda()
    xf, gf = dev_f32_from_bits(x), dev_f32_from_bits(g)
    ref = ref_gpu.rms_norm_gated(xf, gf, dw, rows, cols, 1e-6)
    out = out_buffer(rows * cols, BF16)
    assert call("clef_rms_norm_gated", stream(), ptr(dx), ptr(dg), ptr(dw), out.ptr, rows, cols, 1e-6, BF16) == 0
    torch.cuda.synchronize()
    out.check_guards("rms_norm_gated")
    check_ulp(out.as_bf16_bits(), f32_to_bf16_bits_gpu(ref), 1, "gated norm vs reference kernel")
    _, want = orc.rms_norm_gated(x, g, w, rows, cols, 1e-6)
    check_ulp(out.as_bf16_bits(), want, 1, "gated norm vs CPU oracle")
    outf = out_buffer(rows * cols, F32)
    assert call("clef_rms_norm_gated", stream(), ptr(xf), ptr(gf), ptr(dw), outf.ptr, rows, cols, 1e-6, F32) == 0
    torch.cuda.synchronize()
    assert_bytes_equal(outf.as_f32().view(np.uint32), ref.cpu().numpy().view(np.uint32), "f32 gated norm vs reference kernel")
    # null weight / null gate variants of the reference kernel
    for wt, gt in ((None, gf), (dw, None)):
        o = out_buffer(rows * cols, F32)
        assert call("clef_rms_norm_gated", stream(), ptr(xf), ptr(gt), ptr(wt), o.ptr, rows, cols, 1e-6, F32) == 0
        r = ref_gpu.rms_norm_gated(xf, gt, wt, rows, cols, 1e-6)
        torch.cuda.synchronize()
        assert_bytes_equal(o.as_f32().view(np.uint32), r.cpu().numpy().view(np.uint32), "f32 gated norm, optional operand absent")


def test_norms_f32_on_arbitrary_f32_rows():
    """f32 rows that are not bf16 values (the engine's residual stream and accumulators) through the tuned f32 kernels,
    bit for bit against the reference kernels: 8,192 rows cover the grid-stride tails; gates beyond +-44, infinities
    and NaN take the literal silu."""
    clef.set_kernel_choice(0)
    for rows, cols in ((8192, 2048), (1111, 4096)):
        gen = torch.Generator(device="cuda").manual_seed(cols)
        x = torch.randn(rows, cols, device="cuda", generator=gen) * 3.0
        x[:, 9] *= 50.0
        x[21] = 0.0
        x[22, 5] = float("inf")
        x[23, 6] = float("nan")
        w = torch.randn(cols, device="cuda", generator=gen) * 0.1
        for wt in (w, None):
            out = out_buffer(rows * cols, F32)
            assert call("clef_rms_norm", stream(), ptr(x), ptr(wt), out.ptr, rows, cols, 1e-6, F32) == 0
            ref = ref_gpu.rms_norm(x, wt, rows, cols, 1e-6)
            torch.cuda.synchronize()
            out.check_guards("rms_norm f32")
            assert_bytes_equal(out.as_f32().view(np.uint32), ref.cpu().numpy().view(np.uint32), "f32 rms_norm vs reference kernel")
    rows, cols = 8192 * 16 + 37, 128
    gen = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(rows, cols, device="cuda", generator=gen) * 2.0
    g = torch.randn(rows, cols, device="cuda", generator=gen) * 5.0
    g[:, 3] *= 15.0
    g[40, 8] = float("inf")
    g[41, 9] = float("-inf")
    g[42, 10] = float("nan")
    x[43] = 0.0
    g[44] = -0.0
    w = 1.0 + torch.randn(cols, device="cuda", generator=gen) * 0.1
    out = out_buffer(rows * cols, F32)
    assert call("clef_rms_norm_gated", stream(), ptr(x), ptr(g), ptr(w), out.ptr, rows, cols, 1e-6, F32) == 0
    ref = ref_gpu.rms_norm_gated(x, g, w, rows, cols, 1e-6)
    torch.cuda.synchronize()
    out.check_guards("rms_norm_gated f32")
    assert_bytes_equal(out.as_f32().view(np.uint32), ref.cpu().numpy().view(np.uint32), "f32 gated norm vs reference kernel")


# ---- swiglu --------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("total", [5 * 128, 5 * 128 - 1, 778 * 6144, 1, 3, 4099, 16, 17])
def test_swiglu(total, choice):
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(total)
    pad = (total + 7) // 8 * 8
    g, u = normal_bf16(rng, (pad,), scale=3.0), normal_bf16(rng, (pad,))
    dg, du = dev_bf16(g), dev_bf16(u)
    gf, uf = dev_f32_from_bits(g), dev_f32_from_bits(u)
    ref = ref_gpu.swiglu(gf, uf, total)
    out = out_buffer(total, BF16)
    assert call("clef_swiglu", stream(), ptr(dg), ptr(du), out.ptr, total, BF16) == 0
    torch.cuda.synchronize()
    out.check_guards("swiglu")
    check_ulp(out.as_bf16_bits(), f32_to_bf16_bits_gpu(ref), 1, "swiglu vs reference kernel")
    _, want = orc.swiglu(g[:total], u[:total])
    check_ulp(out.as_bf16_bits(), want, 1, "swiglu vs CPU oracle")
    outf = out_buffer(total, F32)
    assert call("clef_swiglu", stream(), ptr(gf), ptr(uf), outf.ptr, total, F32) == 0
    torch.cuda.synchronize()
    outf.check_guards("swiglu f32")
    assert_bytes_equal(outf.as_f32().view(np.uint32), ref.cpu().numpy().view(np.uint32), "f32 swiglu vs reference kernel")


# ---- rope tables / rope ------------------------------------------------------------------------------------------------
def test_rope_tables():
    positions = np.array([0, 1, 2, 3, 7, 100, 8191, 130711], np.int32)
    dp = torch.from_numpy(positions).cuda()
    cos, sin = clef.Device(0).rope_tables_dev(dp, positions.size, 64, 1e7)
    rc, rs = ref_gpu.rope_tables(dp, positions.size, 64, 1e7)
    torch.cuda.synchronize()
    assert torch.equal(cos, rc) and torch.equal(sin, rs)            # same formula, same libdevice
    wc, ws = orc.rope_tables(positions, 64, 1e7)
    # libm vs libdevice and the f32 argument: the reference's own tolerance is 1e-5 at small positions
    assert np.abs(cos.cpu().numpy()[:5] - wc[:5]).max() < 1e-5 and np.abs(sin.cpu().numpy()[:5] - ws[:5]).max() < 1e-5


def _rope_case(rows, heads, head_dim, rot, mode, rng):
    x = normal_bf16(rng, (rows, heads, head_dim))
    table_len = 4096
    positions = torch.arange(table_len, dtype=torch.int32, device="cuda")
    cos, sin = clef.Device(0).rope_tables_dev(positions, table_len, rot, 1e7)
    seq_start = pos_base = pos_map = None
    if mode == "pos_map":
        pos_map = torch.from_numpy(rng.integers(0, table_len, rows).astype(np.int32)).cuda()
    elif mode == "seq_start":
        half = rows // 2
        seq_start = torch.from_numpy(np.concatenate([np.zeros(half), np.full(rows - half, half)]).astype(np.int32)).cuda()
        pos_base = torch.tensor([17], dtype=torch.int32, device="cuda")
    return x, cos, sin, seq_start, pos_base, pos_map


@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("mode", ["pos_map", "seq_start", "row"])
@pytest.mark.parametrize("rows,heads,head_dim,rot", [(778, 16, 128, 64), (301, 2, 128, 64), (5, 3, 256, 64), (64, 4, 256, 256), (33, 2, 64, 32), (17, 3, 72, 24)])
def test_rope(rows, heads, head_dim, rot, mode, choice):
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(rows + heads + head_dim)
    x, cos, sin, seq_start, pos_base, pos_map = _rope_case(rows, heads, head_dim, rot, mode, rng)
    dx, xf = dev_bf16(x), dev_f32_from_bits(x)
    ref = ref_gpu.rope(xf, cos, sin, rows, heads, head_dim, rot, seq_start, pos_base, pos_map)
    n = rows * heads * head_dim
    out = out_buffer(n, BF16)
    assert call("clef_rope", stream(), out.ptr, ptr(dx), ptr(cos), ptr(sin), rows, heads, head_dim, rot,
                ptr(seq_start), ptr(pos_base), ptr(pos_map), BF16) == 0
    torch.cuda.synchronize()
    out.check_guards("rope")
    got = out.as_bf16_bits().reshape(rows, heads, head_dim)
    check_ulp(got, f32_to_bf16_bits_gpu(ref), 2, "rope vs reference kernel")
    assert_bytes_equal(got[:, :, rot:], x[:, :, rot:], "pass-through dims")
    _, want = orc.rope(x, cos.cpu().numpy(), sin.cpu().numpy(), rows, heads, head_dim, rot,
                       None if seq_start is None else seq_start.cpu().numpy(),
                       None if pos_base is None else pos_base.cpu().numpy(),
                       None if pos_map is None else pos_map.cpu().numpy())
    check_ulp(got, want, 2, "rope vs CPU oracle")
    outf = out_buffer(n, F32)
    assert call("clef_rope", stream(), outf.ptr, ptr(xf), ptr(cos), ptr(sin), rows, heads, head_dim, rot,
                ptr(seq_start), ptr(pos_base), ptr(pos_map), F32) == 0
    torch.cuda.synchronize()
    assert_bytes_equal(outf.as_f32().view(np.uint32), ref.cpu().numpy().view(np.uint32), "f32 rope vs reference kernel")


@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("with_gate", [False, True])
@pytest.mark.parametrize("tokens,heads,head_dim,rot", [(7, 16, 256, 64), (300, 4, 256, 256), (64, 16, 128, 64), (33, 2, 128, 64), (9, 2, 512, 64), (778, 16, 128, 64), (1, 1, 128, 64)])
def test_qk_norm_rope(tokens, heads, head_dim, rot, with_gate, choice):
    """src/cuda/mod.rs:6743-6806: the fused kernel equals split -> per-head rms_norm -> rope."""
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(tokens + head_dim + int(with_gate))
    rows = tokens * heads
    stride = 2 * head_dim if with_gate else head_dim
    x = normal_bf16(rng, (rows, stride))
    w = (rng.standard_normal(head_dim) * 0.1).astype(np.float32)
    table_len = 1024
    cos, sin = clef.Device(0).rope_tables_dev(torch.arange(table_len, dtype=torch.int32, device="cuda"), table_len, rot, 1e7)
    pos_map_np = rng.integers(0, table_len, tokens).astype(np.int32)
    pos_map = torch.from_numpy(pos_map_np).cuda()
    dw, xf = torch.from_numpy(w).cuda(), dev_f32_from_bits(x)
    # reference chain on the GPU in f32: (split) -> rms_norm over head rows -> rope
    q_f = xf.view(rows, stride)[:, :head_dim].contiguous()
    normed = ref_gpu.rms_norm(q_f, dw, rows, head_dim, 1e-6)
    chain = ref_gpu.rope(normed, cos, sin, tokens, heads, head_dim, rot, None, None, pos_map)
    for dtype, xin in ((F32, xf), (BF16, dev_bf16(x))):
        out = out_buffer(rows * head_dim, dtype)
        gate = out_buffer(rows * head_dim, dtype) if with_gate else None
        assert call("clef_qk_norm_rope", stream(), ptr(xin), ptr(dw), ptr(cos), ptr(sin), out.ptr,
                    gate.ptr if gate else None, rows, heads, head_dim, rot, 1e-6, None, None, ptr(pos_map), dtype) == 0
        torch.cuda.synchronize()
        out.check_guards("qk_norm_rope")
        if dtype == F32:
            assert_bytes_equal(out.as_f32().view(np.uint32), chain.cpu().numpy().view(np.uint32), "f32 qk_norm_rope vs reference chain")
            if head_dim == 256:
                fused, fgate = ref_gpu.qk_norm_rope(xf, dw, cos, sin, rows, heads, head_dim, rot, 1e-6, None, None, pos_map, with_gate)
                torch.cuda.synchronize()
                assert_bytes_equal(out.as_f32().view(np.uint32), fused.cpu().numpy().view(np.uint32), "f32 qk_norm_rope vs reference fused kernel")
            if with_gate:
                assert_bytes_equal(gate.as_f32().view(np.uint32), xf.view(rows, stride)[:, head_dim:].contiguous().cpu().numpy().view(np.uint32), "gate half")
        else:
            check_ulp(out.as_bf16_bits(), f32_to_bf16_bits_gpu(chain), 2, "bf16 qk_norm_rope vs reference chain")
            _, want, want_gate = orc.qk_norm_rope(x, w, cos.cpu().numpy(), sin.cpu().numpy(), rows, heads, head_dim, rot, 1e-6,
                                                  pos_map=pos_map_np, with_gate=with_gate)
            check_ulp(out.as_bf16_bits(), want, 2, "bf16 qk_norm_rope vs CPU oracle")
            if with_gate:
                gate.check_guards("qk gate")
                assert_bytes_equal(gate.as_bf16_bits(), want_gate, "gate half")


@pytest.mark.parametrize("with_gate", [False, True])
@pytest.mark.parametrize("tokens,heads,head_dim", [(4099, 16, 256), (8192, 2, 256), (4099, 16, 128)])
def test_qk_norm_rope_and_rope_f32_on_arbitrary_f32_rows(tokens, heads, head_dim, with_gate):
    """f32 rows that are not bf16 values through the tuned f32 kernels at sizes with grid-stride tails, bit for bit
    against the reference kernels (the fused one serves head_dim 256, the chain both)."""
    clef.set_kernel_choice(0)
    rot, rows = 64, tokens * heads
    stride = 2 * head_dim if with_gate else head_dim
    gen = torch.Generator(device="cuda").manual_seed(tokens + head_dim)
    x = torch.randn(rows, stride, device="cuda", generator=gen) * 2.0
    x[5] = 0.0
    w = torch.randn(head_dim, device="cuda", generator=gen) * 0.1
    table_len = 4096
    cos, sin = clef.Device(0).rope_tables_dev(torch.arange(table_len, dtype=torch.int32, device="cuda"), table_len, rot, 1e7)
    pos_map = torch.randint(0, table_len, (tokens,), device="cuda", generator=gen, dtype=torch.int32)
    q_f = x[:, :head_dim].contiguous()
    normed = ref_gpu.rms_norm(q_f, w, rows, head_dim, 1e-6)
    chain = ref_gpu.rope(normed, cos, sin, tokens, heads, head_dim, rot, None, None, pos_map)
    out = out_buffer(rows * head_dim, F32)
    gate = out_buffer(rows * head_dim, F32) if with_gate else None
    assert call("clef_qk_norm_rope", stream(), ptr(x), ptr(w), ptr(cos), ptr(sin), out.ptr, gate.ptr if gate else None, rows,
                heads, head_dim, rot, 1e-6, None, None, ptr(pos_map), F32) == 0
    torch.cuda.synchronize()
    out.check_guards("qk_norm_rope f32")
    assert_bytes_equal(out.as_f32().view(np.uint32), chain.cpu().numpy().view(np.uint32), "f32 qk_norm_rope vs reference chain")
    if head_dim == 256:
        fused, _ = ref_gpu.qk_norm_rope(x, w, cos, sin, rows, heads, head_dim, rot, 1e-6, None, None, pos_map, with_gate)
        torch.cuda.synchronize()
        assert_bytes_equal(out.as_f32().view(np.uint32), fused.cpu().numpy().view(np.uint32), "f32 qk_norm_rope vs reference fused kernel")
    if with_gate:
        gate.check_guards("gate f32")
        assert_bytes_equal(gate.as_f32().view(np.uint32), x[:, head_dim:].contiguous().cpu().numpy().view(np.uint32), "gate half")
    # the plain rotation of the same rows (q alone, then q and k in one launch)
    ro = out_buffer(rows * head_dim, F32)
    assert call("clef_rope", stream(), ro.ptr, ptr(q_f), ptr(cos), ptr(sin), tokens, heads, head_dim, rot, None, None, ptr(pos_map), F32) == 0
    want = ref_gpu.rope(q_f, cos, sin, tokens, heads, head_dim, rot, None, None, pos_map)
    torch.cuda.synchronize()
    ro.check_guards("rope f32")
    assert_bytes_equal(ro.as_f32().view(np.uint32), want.cpu().numpy().view(np.uint32), "f32 rope vs reference kernel")
    kv_heads = 2
    k_f = normed.view(tokens, heads, head_dim)[:, :kv_heads].contiguous()
    qo, ko = out_buffer(rows * head_dim, F32), out_buffer(tokens * kv_heads * head_dim, F32)
    assert call("clef_rope_qk", stream(), qo.ptr, ptr(q_f), heads, ko.ptr, ptr(k_f), kv_heads, ptr(cos), ptr(sin), tokens, head_dim, rot,
                None, None, ptr(pos_map), F32) == 0
    want_k = ref_gpu.rope(k_f, cos, sin, tokens, kv_heads, head_dim, rot, None, None, pos_map)
    torch.cuda.synchronize()
    qo.check_guards("rope_qk q f32")
    ko.check_guards("rope_qk k f32")
    assert_bytes_equal(qo.as_f32().view(np.uint32), want.cpu().numpy().view(np.uint32), "f32 rope_qk q vs reference kernel")
    assert_bytes_equal(ko.as_f32().view(np.uint32), want_k.cpu().numpy().view(np.uint32), "f32 rope_qk k vs reference kernel")


@pytest.mark.parametrize("with_gate", [False, True])
@pytest.mark.parametrize("tokens,heads,head_dim", [(778, 16, 256), (4099, 16, 256), (129, 2, 256), (1, 1, 256), (4099, 16, 128), (65, 3, 128)])
def test_qk_norm_rope_bf16_rounds_the_reference_f32_result(tokens, heads, head_dim, with_gate):
    """bf16 in and out: the tuned kernels (head_dim 128 and 256, rotary 64) and the general kernel must both give
    the reference fused f32 kernel's result rounded once to bf16, byte for byte (bf16 widens to f32 exactly)."""
    rot = 64
    rng = np.random.default_rng(tokens * 3 + head_dim + int(with_gate))
    rows = tokens * heads
    stride = 2 * head_dim if with_gate else head_dim
    x = normal_bf16(rng, (rows, stride))
    x[rng.integers(0, rows, 8)] = 0                      # all-zero head rows
    w = (rng.standard_normal(head_dim) * 0.1).astype(np.float32)
    table_len = 2048
    dev = clef.Device(0)
    cos, sin = dev.rope_tables_dev(torch.arange(table_len, dtype=torch.int32, device="cuda"), table_len, rot, 1e7)
    pos_map = torch.from_numpy(rng.integers(0, table_len, tokens).astype(np.int32)).cuda()
    dw, xf = torch.from_numpy(w).cuda(), dev_f32_from_bits(x)
    if head_dim == 256:
        fused, _ = ref_gpu.qk_norm_rope(xf, dw, cos, sin, rows, heads, head_dim, rot, 1e-6, None, None, pos_map, with_gate)
    else:   # the reference gates its fused kernel on head_dim 256; the chain it replaces is the arbiter elsewhere
        q_f = xf.view(rows, stride)[:, :head_dim].contiguous()
        fused = ref_gpu.rope(ref_gpu.rms_norm(q_f, dw, rows, head_dim, 1e-6), cos, sin, tokens, heads, head_dim, rot, None, None, pos_map)
    want = f32_to_bf16_bits_gpu(fused)
    for choice in (0, 1):
        clef.set_kernel_choice(choice)
        out = out_buffer(rows * head_dim, BF16)
        gate = out_buffer(rows * head_dim, BF16) if with_gate else None
        assert call("clef_qk_norm_rope", stream(), ptr(dev_bf16(x)), ptr(dw), ptr(cos), ptr(sin), out.ptr,
                    gate.ptr if gate else None, rows, heads, head_dim, rot, 1e-6, None, None, ptr(pos_map), BF16) == 0
        torch.cuda.synchronize()
        out.check_guards("qk_norm_rope")
        assert_bytes_equal(out.as_bf16_bits(), want, f"bf16 qk_norm_rope, kernel choice {choice}")
        if with_gate:
            gate.check_guards("qk gate")
            assert_bytes_equal(gate.as_bf16_bits(), x.reshape(rows, stride)[:, head_dim:], "gate half")


def test_rope_contraction_matches_the_reference_build():
    """Which FMA contraction the reference build applies to lo*c - hi*s and to hi*c + lo*s (each
    expression on its own): the modes the CPU oracle uses must reproduce rope_kernel's f32 output."""
    rows, heads, head_dim, rot = 512, 4, 128, 64
    half = rot // 2
    rng = np.random.default_rng(3)
    x = rng.standard_normal((rows, heads, head_dim)).astype(np.float32)
    cos, sin = clef.Device(0).rope_tables_dev(torch.arange(rows, dtype=torch.int32, device="cuda"), rows, rot, 1e7)
    ref = ref_gpu.rope(torch.from_numpy(x).cuda(), cos, sin, rows, heads, head_dim, rot).cpu().numpy()
    diffs = {}
    for mode in (0, 1, 2):
        f32, _ = orc.rope(x, cos.cpu().numpy(), sin.cpu().numpy(), rows, heads, head_dim, rot, rope_fma=mode + 3 * mode)
        bad = f32.view(np.uint32) != ref.view(np.uint32)
        diffs[mode] = (int(bad[:, :, :half].sum()), int(bad[:, :, half:rot].sum()))
    lo_mode, hi_mode = orc.ROPE_FMA % 3, orc.ROPE_FMA // 3
    assert diffs[lo_mode][0] == 0 and diffs[hi_mode][1] == 0, f"(lo, hi) f32 words differing per contraction mode: {diffs}"
