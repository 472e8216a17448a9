"""Parity of the elementwise kernels in front of the Gated-DeltaNet scan through the C-ABI against the reference's
own kernels on the same GPU (oracle/_ref/elementwise.cubin; bf16 inputs widened exactly to the f32 those kernels
take) and against the CPU oracle: causal convolution + silu with sequence starts, history and slot maps built by
the pass maps, the history save, the gate transform, the splitting copies."""
import numpy as np
import pytest
import torch

import aiis_clef_b200 as clef
from oracle import binding as orc
from oracle import ref_gpu
from gpu_util import dev_bf16, dev_f32_from_bits, ptr, stream
from util import bf16_ulp_distance, normal_bf16, to_bf16_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _cleanup():
    clef.set_kernel_choice(0)
    yield
    clef.set_kernel_choice(0)
    torch.cuda.empty_cache()


def i32(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.int32)).cuda()


def bits(t):
    return orc.bf16_bits(t.cpu())


def packed_sequences(rng, rows, n_seq):
    """seq_start per row for n_seq sequences packed back to back, and a slot per row."""
    cuts = np.sort(rng.choice(np.arange(1, rows), n_seq - 1, replace=False)) if n_seq > 1 else np.array([], int)
    starts = np.concatenate([[0], cuts]).astype(np.int32)
    seq_start = np.zeros(rows, np.int32)
    slot_map = np.zeros(rows, np.int32)
    for i, s in enumerate(starts):
        e = starts[i + 1] if i + 1 < len(starts) else rows
        seq_start[s:e] = s
        slot_map[s:e] = (i * 3 + 1) % n_seq
    return seq_start, slot_map


@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("mode", ["plain", "sequences", "history"])
@pytest.mark.parametrize("rows,channels,k", [(1, 64, 4), (7, 128, 4), (778, 1024, 4), (300, 8192, 4), (65, 96, 3), (40, 40, 2), (129, 256, 5)])
def test_causal_conv_silu(rows, channels, k, mode, choice):
    clef.set_kernel_choice(choice)
    rng = np.random.default_rng(rows * 31 + channels + k)
    xb = normal_bf16(rng, (rows, channels))
    w = (rng.standard_normal((channels, k)) * 0.5).astype(np.float32)
    n_seq = min(4, rows)
    seq_start = slot_map = hist = None
    if mode != "plain":
        seq_start, slot_map = packed_sequences(rng, rows, n_seq)
    if mode == "history":
        hist = normal_bf16(rng, (n_seq, k - 1, channels))
    dw = torch.from_numpy(w).cuda()
    d_ss = None if seq_start is None else i32(seq_start)
    d_sm = None if slot_map is None or hist is None else i32(slot_map)
    dev = clef.Device(0)
    ref = ref_gpu.causal_conv_silu(dev_f32_from_bits(xb), dw, rows, channels, k, d_ss,
                                   None if hist is None else dev_f32_from_bits(hist), d_sm)
    # f32: bit-exact against the reference kernel
    out_f = dev.causal_conv_silu_dev(dev_f32_from_bits(xb), dw, rows, channels, k, d_ss,
                                     None if hist is None else dev_f32_from_bits(hist), d_sm)
    torch.cuda.synchronize()
    assert torch.equal(out_f.view(torch.int32), ref.view(torch.int32))
    # bf16: the reference f32 result rounded to nearest even
    out_b = dev.causal_conv_silu_dev(dev_bf16(xb), dw, rows, channels, k, d_ss, None if hist is None else dev_bf16(hist), d_sm)
    torch.cuda.synchronize()
    assert np.array_equal(bits(out_b), bits(ref.to(torch.bfloat16)))
    # CPU oracle: the pre-activation sums are exact arithmetic; the silu differs by the exp approximation only
    f32, cpu_b, acc = orc.causal_conv_silu(xb, w, rows, channels, k, seq_start, hist, slot_map if hist is not None else None)
    assert bf16_ulp_distance(bits(out_b).reshape(-1), cpu_b.reshape(-1)).max() <= 1
    np.testing.assert_allclose(out_f.cpu().numpy(), f32, rtol=2e-6, atol=1e-30)


def test_causal_conv_silu_accumulators_outside_the_short_silu_domain():
    """One tap with weight 1 makes the accumulator the input itself: the two f32 values the short silu form misses,
    values beyond |44|, infinities, NaN, zeros of both signs and subnormals must all come out as the reference
    kernel's literal expression gives them (f32 storage, bit for bit)."""
    rows, channels, k = 64, 64, 4
    special = np.array([0x3E609AF2, 0x3E24A9BF, 0xBE609AF2, 0x42300000, 0x42300001, 0xC2300001, 0x42B00000, 0xC2B00000,
                        0x7F800000, 0xFF800000, 0x7FC00000, 0x00000000, 0x80000000, 0x00000001, 0x80000001, 0x007FFFFF,
                        0x00800000, 0x3F800000, 0xC1200000, 0x41A00000], np.uint32)
    rng = np.random.default_rng(44)
    xb = rng.standard_normal((rows, channels)).astype(np.float32)
    flat = xb.reshape(-1)
    flat[rng.choice(flat.size, special.size * 8, replace=False)] = np.tile(special, 8).view(np.float32)
    w = np.zeros((channels, k), np.float32)
    w[:, k - 1] = 1.0
    dx, dw = torch.from_numpy(xb).cuda(), torch.from_numpy(w).cuda()
    seq_start = i32(np.arange(rows))                 # every row starts a sequence: only the last tap is live
    ref = ref_gpu.causal_conv_silu(dx, dw, rows, channels, k, seq_start, None, None)
    for choice in (0, 1):
        clef.set_kernel_choice(choice)
        got = clef.Device(0).causal_conv_silu_dev(dx, dw, rows, channels, k, seq_start, None, None)
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int32), ref.view(torch.int32)), choice


@pytest.mark.parametrize("offset", [0, 1, 2])
def test_causal_conv_silu_sequence_starts_at_any_alignment(offset):
    """The tuned kernel reads the 8 sequence starts of a strip as two 16-byte loads when the array allows it: the
    same map at a 16-byte aligned address and 4 and 8 bytes off it, many short sequences, ragged row count."""
    rows, channels, k = 1003, 256, 4
    rng = np.random.default_rng(9 + offset)
    xb = normal_bf16(rng, (rows, channels))
    w = (rng.standard_normal((channels, k)) * 0.5).astype(np.float32)
    seq_start, slot_map = packed_sequences(rng, rows, 37)
    hist = normal_bf16(rng, (37, k - 1, channels))
    holder = torch.zeros(rows + 8, dtype=torch.int32, device="cuda")
    d_ss = holder[offset:offset + rows]
    d_ss.copy_(i32(seq_start))
    dw, d_sm = torch.from_numpy(w).cuda(), i32(slot_map)
    ref = ref_gpu.causal_conv_silu(dev_f32_from_bits(xb), dw, rows, channels, k, d_ss.clone(), dev_f32_from_bits(hist), d_sm)
    got = clef.Device(0).causal_conv_silu_dev(dev_bf16(xb), dw, rows, channels, k, d_ss, dev_bf16(hist), d_sm)
    torch.cuda.synchronize()
    assert np.array_equal(bits(got), bits(ref.to(torch.bfloat16)))


def test_causal_conv_silu_with_pass_maps_and_history_round_trip():
    """Two passes over the same requests: the first pass saves each request's last k - 1 rows as its history
    (hist_save of the pass maps), the second continues the requests; a request continued this way must equal the
    same request run in one piece."""
    k, channels, capacity = 4, 512, 4096
    rng = np.random.default_rng(5)
    lens = [192, 128, 320]
    first = [128, 64, 192]
    reqs = [rng.integers(0, 1000, n).astype(np.uint32) for n in lens]
    xs = [normal_bf16(rng, (n, channels)) for n in lens]
    w = (rng.standard_normal((channels, k)) * 0.5).astype(np.float32)
    dw = torch.from_numpy(w).cuda()
    dev = clef.Device(0)
    whole = [dev.causal_conv_silu_dev(dev_bf16(x), dw, x.shape[0], channels, k) for x in xs]
    hist = torch.zeros(len(lens), k - 1, channels, dtype=torch.bfloat16, device="cuda")
    # pass 1: the first part of every request, coalesced
    m1 = clef.pass_maps([(reqs[i], 0, i, first[i]) for i in range(3)], capacity)
    x1 = dev_bf16(np.concatenate([xs[i][: first[i]] for i in range(3)]))
    rows1 = int(m1["total"])
    out1 = dev.causal_conv_silu_dev(x1, dw, rows1, channels, k, i32(m1["seq_start"]), hist, i32(m1["slot_map"]))
    saves = i32(m1["hist_save"].astype(np.int32).reshape(-1))
    dev.conv_hist_save_dev(x1, hist, saves, 3, rows1, k, channels)
    ref_hist = ref_gpu.conv_hist_save(x1.float(), torch.zeros(3, k - 1, channels, device="cuda"), saves, 3, rows1, k, channels)
    assert torch.equal(hist.float(), ref_hist)
    # pass 2: the rest of every request
    rest = [lens[i] - first[i] for i in range(3)]
    m2 = clef.pass_maps([(reqs[i], first[i], i, rest[i]) for i in range(3)], capacity)
    x2 = dev_bf16(np.concatenate([xs[i][first[i]:] for i in range(3)]))
    out2 = dev.causal_conv_silu_dev(x2, dw, int(m2["total"]), channels, k, i32(m2["seq_start"]), hist, i32(m2["slot_map"]))
    torch.cuda.synchronize()
    for i in range(3):
        o1, o2 = int(m1["offs"][i]), int(m2["offs"][i])
        assert torch.equal(out1[o1:o1 + first[i]], whole[i][: first[i]])
        assert torch.equal(out2[o2:o2 + rest[i]], whole[i][first[i]:])


@pytest.mark.parametrize("tokens,heads", [(1, 32), (778, 32), (8192, 16), (65, 5)])
def test_gdn_gates(tokens, heads):
    rng = np.random.default_rng(tokens + heads)
    ab = to_bf16_bits((rng.standard_normal((tokens, heads)) * 6).astype(np.float32))
    bb = to_bf16_bits((rng.standard_normal((tokens, heads)) * 3).astype(np.float32))
    ab.reshape(-1)[:4] = to_bf16_bits(np.array([30.0, 19.9, -60.0, 0.0], np.float32))[: min(4, ab.size)]
    a_log = (rng.standard_normal(heads) * 0.5).astype(np.float32)
    dt_bias = (rng.standard_normal(heads) * 0.5).astype(np.float32)
    dal, ddt = torch.from_numpy(a_log).cuda(), torch.from_numpy(dt_bias).cuda()
    dev = clef.Device(0)
    rd, rb = ref_gpu.gdn_gates(dev_f32_from_bits(ab), dev_f32_from_bits(bb), dal, ddt, tokens, heads)
    for a_in, b_in in ((dev_f32_from_bits(ab), dev_f32_from_bits(bb)), (dev_bf16(ab), dev_bf16(bb))):
        decay, beta = dev.gdn_gates_dev(a_in, b_in, dal, ddt, tokens, heads)
        torch.cuda.synchronize()
        assert torch.equal(decay.view(torch.int32), rd.view(torch.int32)) and torch.equal(beta.view(torch.int32), rb.view(torch.int32))
    cd, cb = orc.gdn_gates(ab, bb, a_log, dt_bias, tokens, heads)
    np.testing.assert_allclose(decay.cpu().numpy(), cd, rtol=3e-6, atol=1e-30)
    np.testing.assert_allclose(beta.cpu().numpy(), cb, rtol=3e-6, atol=1e-30)


@pytest.mark.parametrize("seq_len,kh,heads,extra", [(1, 16, 32, 0), (64, 16, 32, 0), (130, 4, 8, 8), (778, 16, 32, 0), (65, 4, 4, 24),
                                                   (2048, 16, 32, 0)])
def test_gdn_prep_operands_of_the_chunked_scan(seq_len, kh, heads, extra):
    """clef_gdn_prep against the reference's gdn_prep_kernel on the same GPU: the four hi / lo operand buffers (the
    whole buffers, pad rows of the last chunk included), the f32 normalised k and the f32 v, byte for byte, from f32
    and from bf16 rows; and against a plain numpy restatement of the normalisation and of the operand layout.
    (The reference kernel gives each of its four row warps kh / 4 heads, so it serves kh % 4 == 0 only.)"""
    kd = 128
    conv_dim = 2 * kh * kd + heads * kd + extra
    rng = np.random.default_rng(seq_len + kh)
    xb = normal_bf16(rng, (seq_len, conv_dim))
    xb[rng.integers(0, seq_len, 2), : kd] = 0                      # an all-zero q head: rsqrt(1e-6) * 0
    dev = clef.Device(0)
    ref = ref_gpu.gdn_prep(dev_f32_from_bits(xb), seq_len, kh, kd, heads, conv_dim)
    for mixed in (dev_f32_from_bits(xb), dev_bf16(xb)):
        got = dev.gdn_prep_dev(mixed, seq_len, kh, kd, heads, conv_dim)
        torch.cuda.synchronize()
        for name in ("q_hi", "q_lo", "k_hi", "k_lo"):
            assert torch.equal(got[name], ref[name]), name
        assert torch.equal(got["kn"].view(-1).view(torch.int32), ref["kn"].view(torch.int32))
        assert torch.equal(got["v"].view(-1).view(torch.int32), ref["v"].view(torch.int32))
    # numpy restatement: value(t, he, p) = x / sqrt(sum x^2 + 1e-6) (* kd^-0.5 for q) = hi + lo up to bf16^2 precision,
    # stored at ((he * nchunks + t // 64) * 2 + p // 64) * 8192 + (t % 64) * 128 + (((p % 64) // 8) ^ (t % 8)) * 16 + (p % 8) * 2
    x = orc.bf16_to_f32(xb).astype(np.float64)
    nchunks = (seq_len + 63) // 64
    ratio = heads // kh
    t = np.arange(seq_len)[:, None, None]
    he = np.arange(heads)[None, :, None]
    p = np.arange(kd)[None, None, :]
    off = (((he * nchunks + t // 64) * 2 + p // 64) * 8192 + (t % 64) * 128 + (((p % 64) // 8) ^ (t % 8)) * 16 + (p % 8) * 2) // 2
    for name, base, scale in (("q", 0, kd ** -0.5), ("k", kh * kd, 1.0)):
        heads_x = x[:, base: base + kh * kd].reshape(seq_len, kh, kd)
        want = heads_x / np.sqrt((heads_x ** 2).sum(-1, keepdims=True) + 1e-6) * scale
        want = np.repeat(want, ratio, axis=1)
        hi = orc.bf16_to_f32(got[name + "_hi"].cpu().numpy().view(np.uint16))[off].astype(np.float64)
        lo = orc.bf16_to_f32(got[name + "_lo"].cpu().numpy().view(np.uint16))[off].astype(np.float64)
        assert np.abs(hi + lo - want).max() <= 2e-6                  # rsqrtf is good to 2 ulp; |value| <= 1
        assert (np.abs(lo) <= np.abs(hi) * 2.0 ** -8 + 1e-30).all()  # lo is the rounding remainder of hi
        if name == "k":
            assert np.abs(got["kn"].cpu().numpy() - want).max() <= 2e-6
    assert np.array_equal(got["v"].cpu().numpy(), orc.bf16_to_f32(xb)[:, 2 * kh * kd: 2 * kh * kd + heads * kd])
    # the CPU oracle (1 / sqrtf for rsqrtf): same layout, the f32 values within the 2 ulp of rsqrtf plus one rounding,
    # the hi words equal except where that difference crosses a bf16 rounding boundary
    if seq_len <= 778:
        cpu = orc.gdn_prep(xb, seq_len, kh, kd, heads, conv_dim)
        np.testing.assert_allclose(got["kn"].cpu().numpy(), cpu["kn"], rtol=4e-7, atol=1e-30)
        for name in ("q_hi", "k_hi"):
            g = got[name].cpu().numpy().view(np.uint16)
            assert bf16_ulp_distance(g, cpu[name]).max() <= 1 and (g != cpu[name]).mean() < 1e-3
            assert np.array_equal(g == 0, cpu[name] == 0)            # the same words are written


def test_gdn_prep_argument_errors():
    lib = clef.load()
    from gpu_util import ptr, stream
    b = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    args = lambda **kw: [kw.get(k, d) for k, d in (("seq_len", 4), ("heads", 4), ("kh", 2), ("kd", 128), ("conv_dim", 1024))]
    call = lambda **kw: lib.clef_gdn_prep(stream(), ptr(b), ptr(b), ptr(b), ptr(b), ptr(b), ptr(b), ptr(b), *args(**kw), 0.1, 0)
    assert call(kd=64) == -1              # the operand layout is built for 128
    assert call(heads=3) == -1            # not a multiple of kh
    assert call(conv_dim=1016) == -1      # too narrow for q, k and v
    assert call(seq_len=0) == 0


@pytest.mark.parametrize("mode", ["plain", "sequences", "history"])
@pytest.mark.parametrize("seq_len,kh,heads", [(1, 4, 4), (64, 4, 8), (203, 4, 8), (778, 16, 32), (2048, 16, 32), (130, 4, 16)])
def test_gdn_conv_prep_equals_the_reference_chain(seq_len, kh, heads, mode):
    """clef_gdn_conv_prep (one launch) against the reference kernels causal_conv_silu_kernel -> gdn_prep_kernel on the
    same GPU, the convolved rows in f32 in between: all six outputs byte for byte, from f32 and from bf16 rows."""
    kd, k = 128, 4
    conv_dim = 2 * kh * kd + heads * kd
    rng = np.random.default_rng(seq_len * 7 + kh)
    xb = normal_bf16(rng, (seq_len, conv_dim))
    w = (rng.standard_normal((conv_dim, k)) * 0.5).astype(np.float32)
    n_seq = min(5, seq_len)
    seq_start = slot_map = hist = None
    if mode != "plain":
        seq_start, slot_map = packed_sequences(rng, seq_len, n_seq)
    if mode == "history":
        hist = normal_bf16(rng, (n_seq, k - 1, conv_dim))
    dw = torch.from_numpy(w).cuda()
    d_ss = None if seq_start is None else i32(seq_start)
    d_sm = None if hist is None else i32(slot_map)
    conv = ref_gpu.causal_conv_silu(dev_f32_from_bits(xb), dw, seq_len, conv_dim, k, d_ss,
                                    None if hist is None else dev_f32_from_bits(hist), d_sm)
    ref = ref_gpu.gdn_prep(conv.contiguous().view(-1), seq_len, kh, kd, heads, conv_dim)
    dev = clef.Device(0)
    # under the shape-general kernel choice the entry point declines (the caller runs the two calls) ...
    lib = clef.load()
    dx, dh = dev_bf16(xb), (None if hist is None else dev_bf16(hist))
    bufs = [torch.empty(heads * ((seq_len + 63) // 64) * 2 * 64 * 128, dtype=torch.uint8, device="cuda") for _ in range(4)]
    kn_, v_ = torch.empty(seq_len, heads, kd, device="cuda"), torch.empty(seq_len, heads * kd, device="cuda")
    clef.set_kernel_choice(1)
    assert lib.clef_gdn_conv_prep(stream(), ptr(dx), ptr(dw), ptr(v_), ptr(bufs[0]), ptr(bufs[1]), ptr(bufs[2]), ptr(bufs[3]), ptr(kn_),
                                  seq_len, conv_dim, k, ptr(d_ss), ptr(dh), ptr(d_sm), heads, kh, kd,
                                  float(np.float32(1.0) / np.sqrt(np.float32(kd))), 0) == 1
    # ... and by default it is one launch (1, 2 or 4 value heads per key head; other ratios decline)
    clef.set_kernel_choice(0)
    assert lib.clef_gdn_conv_prep(stream(), ptr(dx), ptr(dw), ptr(v_), ptr(bufs[0]), ptr(bufs[1]), ptr(bufs[2]), ptr(bufs[3]), ptr(kn_),
                                  seq_len, 2 * kh * kd + 3 * kh * kd, k, ptr(d_ss), ptr(dh), ptr(d_sm), 3 * kh, kh, kd, 0.1, 0) == 1
    for x_in, h_in in ((dev_f32_from_bits(xb), None if hist is None else dev_f32_from_bits(hist)),
                       (dev_bf16(xb), None if hist is None else dev_bf16(hist))):
        got = dev.gdn_conv_prep_dev(x_in, dw, seq_len, kh, kd, heads, conv_dim, k, d_ss, h_in, d_sm)
        torch.cuda.synchronize()
        for name in ("q_hi", "q_lo", "k_hi", "k_lo"):
            assert torch.equal(got[name], ref[name]), name
        assert torch.equal(got["kn"].view(-1).view(torch.int32), ref["kn"].view(torch.int32))
        assert torch.equal(got["v"].view(-1).view(torch.int32), ref["v"].view(torch.int32))
    # and the two-call composition of this library with an f32 intermediate gives the same bytes
    mid = dev.causal_conv_silu_dev(dev_f32_from_bits(xb), dw, seq_len, conv_dim, k, d_ss,
                                   None if hist is None else dev_f32_from_bits(hist), d_sm)
    two = dev.gdn_prep_dev(mid, seq_len, kh, kd, heads, conv_dim)
    for name in ("q_hi", "q_lo", "k_hi", "k_lo"):
        assert torch.equal(two[name], got[name]), name


@pytest.mark.parametrize("tokens", [1, 778, 4099])
def test_splitting_copies(tokens):
    rng = np.random.default_rng(tokens)
    dev = clef.Device(0)
    heads, hd = 16, 128
    qg = normal_bf16(rng, (tokens, heads, 2 * hd))
    q, gate = dev.split_q_gate_dev(dev_bf16(qg), tokens, heads, hd)
    rq, rg = ref_gpu.split_q_gate(dev_f32_from_bits(qg), tokens, heads, hd)
    assert np.array_equal(bits(q), qg[:, :, :hd]) and np.array_equal(bits(gate), qg[:, :, hd:])          # elementwise.cu:386-394
    assert torch.equal(q.float(), rq) and torch.equal(gate.float(), rg)
    qf, gf = dev.split_q_gate_dev(dev_f32_from_bits(qg), tokens, heads, hd)
    assert torch.equal(qf, rq) and torch.equal(gf, rg)
    kh, kd, vh, vd = 16, 128, 32, 128
    mixed = normal_bf16(rng, (tokens, 2 * kh * kd + vh * vd))
    q, k, v = dev.split_qkv_dev(dev_bf16(mixed), tokens, kh, kd, vh, vd)
    rq, rk, rv = ref_gpu.split_qkv(dev_f32_from_bits(mixed), tokens, kh, kd, vh, vd)
    assert np.array_equal(bits(q), mixed[:, : kh * kd]) and np.array_equal(bits(k), mixed[:, kh * kd: 2 * kh * kd])
    assert np.array_equal(bits(v), mixed[:, 2 * kh * kd:])                                                      # elementwise.cu:417-425
    assert torch.equal(q.float(), rq) and torch.equal(k.float(), rk) and torch.equal(v.float(), rv)
    src = normal_bf16(rng, (tokens, kh, kd))
    out = dev.repeat_interleave_dev(dev_bf16(src), tokens, kh, 2, kd)
    ro = ref_gpu.repeat_interleave(dev_f32_from_bits(src), tokens, kh, 2, kd)
    assert np.array_equal(bits(out), np.repeat(src, 2, axis=1))                                                 # elementwise.cu:437-444
    assert torch.equal(out.float(), ro)
    outf = dev.repeat_interleave_dev(dev_f32_from_bits(src), tokens, kh, 2, kd)
    assert torch.equal(outf, ro)


def test_gdn_prep_argument_errors():
    lib = clef.load()
    from gpu_util import ptr, stream
    x = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(64, 4, device="cuda")
    assert lib.clef_causal_conv_silu(stream(), ptr(x), ptr(x), ptr(w), 64, 64, 4, None, None, None, 0) == -1     # out aliases x
    assert lib.clef_causal_conv_silu(stream(), None, ptr(x), ptr(w), 64, 64, 4, None, None, None, 0) == -1
    assert lib.clef_split_q_gate(stream(), ptr(x), ptr(x), ptr(x), 4, 2, 12, 0) == -1                              # 12 values < 16 bytes
    assert lib.clef_repeat_interleave(stream(), ptr(x), ptr(x), 4, 2, 2, 12, 0) == -1
    assert lib.clef_gdn_gates(stream(), ptr(x), ptr(x), ptr(w), ptr(w), None, ptr(w), 4, 2, 0) == -1
    assert lib.clef_conv_hist_save(stream(), ptr(x), ptr(x), None, 0, 64, 4, 64, 0) == 0                          # nothing to save
