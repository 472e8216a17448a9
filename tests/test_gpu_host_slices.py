"""The host-slice launchers (include/clef_host.h): host buffers in, host buffers out, row tiles
streamed through two CUDA streams. Results must equal the CPU oracle's (exact kernels) or the
device-resident C-ABI path's (kernels with approximate intrinsics), byte for byte."""
import numpy as np
import pytest
import torch

import aiis_clef_b200 as clef
from oracle import binding as orc
from gpu_util import dev_bf16
from util import assert_bytes_equal, normal_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def host_dev():
    d = clef.HostDevice(0)
    yield d
    d.close()


def pinned(a: np.ndarray) -> torch.Tensor:
    t = torch.from_numpy(a)
    return t.pin_memory()


@pytest.mark.parametrize("rows", [1, 778, 8192, 20000])
def test_host_rms_norm_quantise(host_dev, rows):
    cols = 2048
    rng = np.random.default_rng(rows)
    x = normal_bf16(rng, (rows, cols), outlier_channels=8)
    w = (rng.standard_normal(cols) * 0.1).astype(np.float32)
    rp, pb, sb = clef.nvfp4_sizes(rows, cols, 128)
    packed, scales = pinned(np.full(pb, 0xA5, np.uint8)), pinned(np.full(sb, 0xA5, np.uint8))
    xin = orc.bits_to_torch_bf16(x).pin_memory()
    host_dev.rms_norm_quantise_nvfp4(xin, w, packed, scales, rows, cols, 1e-6, 64.0)
    want_p, want_s = orc.rms_norm_quantise_nvfp4(x, w, rows, cols, 1e-6, 64.0)
    assert_bytes_equal(packed.numpy(), want_p, "host rms_norm+quant packed")
    assert_bytes_equal(scales.numpy(), want_s, "host rms_norm+quant scales")


@pytest.mark.parametrize("rows", [7, 8192])
def test_host_swiglu_quantise_and_quantise(host_dev, rows):
    cols = 6144
    rng = np.random.default_rng(rows + 1)
    gate, up = normal_bf16(rng, (rows, cols)), normal_bf16(rng, (rows, cols))
    rp, pb, sb = clef.nvfp4_sizes(rows, cols, 128)
    packed, scales = np.full(pb, 0xA5, np.uint8), np.full(sb, 0xA5, np.uint8)   # pageable host memory also works
    host_dev.swiglu_quantise_nvfp4(gate, up, packed, scales, rows, cols, 64.0)
    ref_p, ref_s = clef.Device(0).swiglu_quantise_nvfp4_dev(dev_bf16(gate), dev_bf16(up), rows, cols, 64.0, 128)
    torch.cuda.synchronize()
    assert_bytes_equal(packed, ref_p.cpu().numpy().reshape(-1), "host swiglu+quant packed")
    assert_bytes_equal(scales, ref_s.cpu().numpy(), "host swiglu+quant scales")
    p2, s2 = np.full(pb, 0xA5, np.uint8), np.full(sb, 0xA5, np.uint8)
    host_dev.quantise_nvfp4(gate, p2, s2, rows, cols, 64.0)
    want_p, want_s = orc.quantise_nvfp4(gate, rows, cols, 64.0)
    assert_bytes_equal(p2, want_p, "host quantise packed")
    assert_bytes_equal(s2, want_s, "host quantise scales")


@pytest.mark.parametrize("tokens", [5, 1300])
def test_host_gated(host_dev, tokens):
    vh, cols = 16, 128
    rows = tokens * vh
    rng = np.random.default_rng(tokens)
    x, g = normal_bf16(rng, (rows, cols)), normal_bf16(rng, (rows, cols))
    w = (1 + rng.standard_normal(cols) * 0.1).astype(np.float32)
    tp, pb, sb = clef.nvfp4_sizes(tokens, vh * cols, 128)
    packed, scales = np.full(pb, 0xA5, np.uint8), np.full(sb, 0xA5, np.uint8)
    host_dev.rms_norm_gated_quantise_nvfp4(x, g, w, packed, scales, rows, cols, vh, 1e-6, 64.0)
    ref_p, ref_s = clef.Device(0).rms_norm_gated_quantise_nvfp4_dev(dev_bf16(x), dev_bf16(g), torch.from_numpy(w).cuda(),
                                                                     rows, cols, vh, 1e-6, 64.0, 128)
    torch.cuda.synchronize()
    assert_bytes_equal(packed, ref_p.cpu().numpy().reshape(-1), "host gated packed")
    assert_bytes_equal(scales, ref_s.cpu().numpy(), "host gated scales")


def test_host_rope_and_embed(host_dev):
    rows, heads, hd, rot = 3000, 16, 128, 64
    rng = np.random.default_rng(9)
    x = normal_bf16(rng, (rows, heads, hd))
    table_rows = 4096
    cos, sin = orc.rope_tables(np.arange(table_rows, dtype=np.int32), rot, 1e7)
    pos = rng.integers(0, table_rows, rows).astype(np.int32)
    out = np.zeros_like(x)
    host_dev.rope(out, x, cos, sin, table_rows, rows, heads, hd, rot, pos)
    d = clef.Device(0)
    want = d.rope_apply_dev(dev_bf16(x), torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda(), rows, heads, hd, rot,
                            pos_map=torch.from_numpy(pos).cuda())
    torch.cuda.synchronize()
    assert_bytes_equal(out, orc.bf16_bits(want.cpu()), "host rope")
    out2 = np.zeros_like(x)
    host_dev.rope(out2, x, cos, sin, table_rows, rows, heads, hd, rot, None)          # position = row index
    _, want2 = orc.rope(x, cos, sin, rows, heads, hd, rot)
    from util import bf16_ulp_distance
    assert bf16_ulp_distance(out2.reshape(-1), want2.reshape(-1)).max() <= 2
    with pytest.raises(clef.ClefError, match="outside"):
        host_dev.rope(out, x, cos, sin, table_rows, rows, heads, hd, rot, pos + 5000)
    vocab, hidden, tokens = 5000, 2048, 9000
    table = normal_bf16(rng, (vocab, hidden), scale=0.02)
    ids = rng.integers(0, vocab, tokens).astype(np.int32)
    got = np.zeros((tokens, hidden), np.uint16)
    host_dev.embed_gather(dev_bf16(table), ids, got, tokens, hidden)
    assert_bytes_equal(got, table[ids], "host embed gather")


def test_pipelined_mode_gives_the_same_bytes(host_dev):
    """clef_device_set_pipelined: calls return once enqueued and overlap; after clef_device_synchronize every output
    equals the synchronous mode's, also when the same call sequence runs several times over the same buffers."""
    rows, hidden, inter = 3000, 2048, 1024
    rng = np.random.default_rng(31)
    x, g, u = (orc.bits_to_torch_bf16(normal_bf16(rng, shape)).pin_memory() for shape in ((rows, hidden), (rows, inter), (rows, inter)))
    w1 = (rng.standard_normal(hidden) * 0.1).astype(np.float32)
    w2 = (rng.standard_normal(hidden) * 0.3).astype(np.float32)
    rp = (rows + 127) // 128 * 128

    def outputs():
        return [torch.empty(rp * hidden // 2, dtype=torch.uint8).pin_memory(), torch.empty(rp * hidden // 16, dtype=torch.uint8).pin_memory(),
                torch.empty(rp * hidden // 2, dtype=torch.uint8).pin_memory(), torch.empty(rp * hidden // 16, dtype=torch.uint8).pin_memory(),
                torch.empty(rp * inter // 2, dtype=torch.uint8).pin_memory(), torch.empty(rp * inter // 16, dtype=torch.uint8).pin_memory()]

    def sequence(o):
        host_dev.rms_norm_quantise_nvfp4(x, w1, o[0], o[1], rows, hidden, 1e-6, 64.0)
        host_dev.rms_norm_quantise_nvfp4(x, w2, o[2], o[3], rows, hidden, 1e-6, 64.0)     # different weights, same arena
        host_dev.swiglu_quantise_nvfp4(g, u, o[4], o[5], rows, inter, 48.0)

    want = outputs()
    sequence(want)
    host_dev.set_pipelined(True)
    try:
        got = outputs()
        for _ in range(3):
            sequence(got)
        host_dev.synchronize()
        for a, b in zip(got, want):
            assert torch.equal(a, b)
    finally:
        host_dev.set_pipelined(False)
    assert not torch.equal(want[0], want[2])


@pytest.mark.parametrize("rows", [1, 778, 20000])
def test_host_quantise_fp8(host_dev, rows):
    """Device::quantise_fp8 (src/cuda/mod.rs:1065-1092) through the host-slice launcher, against the CPU oracle."""
    cols = 2048
    rng = np.random.default_rng(rows + 8)
    x = normal_bf16(rng, (rows, cols), outlier_channels=4)
    out, scales = pinned(np.full(rows * cols, 0xA5, np.uint8)), pinned(np.zeros(rows, np.uint16))
    host_dev.quantise_fp8(orc.bits_to_torch_bf16(x).pin_memory(), out, scales, rows, cols)
    want_q, want_s = orc.quantise_fp8(x, rows, cols)
    assert_bytes_equal(out.numpy(), want_q.reshape(-1), "host fp8 codes")
    assert_bytes_equal(scales.numpy(), want_s, "host fp8 scales")


def test_table_uploaded_through_the_handle_then_gathered_over_several_tiles(host_dev):
    """clef_device_alloc, clef_device_upload from pinned memory (asynchronous, stream 0), then at once
    clef_host_embed_gather over more than three row tiles (odd tiles run on the handle's second stream), then
    download and free: the gather must see the whole uploaded table, the download the same bytes."""
    vocab, hidden, tokens = 60000, 2048, 20000            # a 245 MB upload; 20,000 rows = 4 tiles of about 6,000
    rng = np.random.default_rng(47)
    table = orc.bits_to_torch_bf16(normal_bf16(rng, (vocab, hidden), scale=0.02)).pin_memory()
    ids = rng.integers(0, vocab, tokens).astype(np.int32)
    ids[-5:] = vocab - 1                                  # the end of the table: the last bytes the upload writes
    nbytes = vocab * hidden * 2
    for mode in (False, True):
        host_dev.set_pipelined(mode)
        try:
            address = host_dev.alloc(nbytes)
            host_dev.upload(address, table, nbytes)
            got = pinned(np.zeros((tokens, hidden), np.uint16))
            host_dev.embed_gather_from(address, ids, got, tokens, hidden)
            back = pinned(np.zeros(vocab * hidden, np.uint16))
            host_dev.download(back, address, nbytes)      # waits for its copy (and, behind the fence, for the gather)
            host_dev.free(address)
            host_dev.synchronize()
            want = orc.bf16_bits(table)
            assert_bytes_equal(got.numpy(), want[ids], f"gather from an uploaded table (pipelined={mode})")
            assert_bytes_equal(back.numpy(), want.reshape(-1), "download of the uploaded table")
        finally:
            host_dev.set_pipelined(False)


@pytest.mark.parametrize("f32", [True, False], ids=["f32", "bf16"])
def test_plain_host_wrappers_equal_the_device_entry_points(host_dev, f32):
    """Device::{rms_norm, rms_norm_gated, swiglu, causal_conv_silu, rope_tables} as host-slice calls
    (src/cuda/mod.rs:853-973): host arrays in, host arrays out, byte for byte what the device-resident entry points
    give on the same values (those are compared with the reference kernels in test_gpu_parity_elem.py and
    test_gpu_gdn_prep.py); several row tiles on both streams, optional operands absent."""
    dev = clef.Device(0)
    rng = np.random.default_rng(5 + int(f32))
    as_host = (lambda bits: orc.bits_to_torch_bf16(bits).float().numpy()) if f32 else (lambda bits: bits)
    as_dev = (lambda bits: dev_bf16(bits).float()) if f32 else dev_bf16
    out_like = lambda a: np.empty_like(a)
    same = lambda got, want, what: assert_bytes_equal(got.view(np.uint8).reshape(-1), want.contiguous().cpu().view(torch.uint8).numpy().reshape(-1), what)
    # rms_norm: 20,000 x 2048 is several tiles
    rows, cols = 20000, 2048
    xb = normal_bf16(rng, (rows, cols), outlier_channels=4)
    w = (rng.standard_normal(cols) * 0.1).astype(np.float32)
    x, out = as_host(xb), out_like(as_host(xb))
    host_dev.rms_norm(x, w, out, rows, cols, 1e-6)
    same(out, dev.rms_norm_dev(as_dev(xb), torch.from_numpy(w).cuda(), rows, cols, 1e-6), "host rms_norm")
    host_dev.rms_norm(x, None, out, rows, cols, 1e-6)
    same(out, dev.rms_norm_dev(as_dev(xb), None, rows, cols, 1e-6), "host rms_norm without weight")
    # rms_norm_gated over head rows
    rows, cols = 1300 * 16, 128
    xb, gb = normal_bf16(rng, (rows, cols)), normal_bf16(rng, (rows, cols))
    wg = (1.0 + rng.standard_normal(cols) * 0.1).astype(np.float32)
    x, g, out = as_host(xb), as_host(gb), out_like(as_host(xb))
    host_dev.rms_norm_gated(x, g, wg, out, rows, cols, 1e-6)
    same(out, dev.rms_norm_gated_dev(as_dev(xb), as_dev(gb), torch.from_numpy(wg).cuda(), rows, cols, 1e-6), "host rms_norm_gated")
    host_dev.rms_norm_gated(x, None, wg, out, rows, cols, 1e-6)
    same(out, dev.rms_norm_gated_dev(as_dev(xb), None, torch.from_numpy(wg).cuda(), rows, cols, 1e-6), "host rms_norm_gated without gate")
    # swiglu on flat arrays whose length is not a multiple of a large power of two
    total = 4 * 1234567
    gb, ub = normal_bf16(rng, (total,)), normal_bf16(rng, (total,))
    g, u, out = as_host(gb), as_host(ub), out_like(as_host(gb))
    host_dev.swiglu(g, u, out, total)
    same(out, dev.swiglu_dev(as_dev(gb), as_dev(ub), total), "host swiglu")
    # causal convolution + silu of one sequence
    rows, channels, k = 777, 1024, 4
    xb = normal_bf16(rng, (rows, channels))
    wc = (rng.standard_normal((channels, k)) * 0.5).astype(np.float32)
    x, out = as_host(xb), out_like(as_host(xb))
    host_dev.causal_conv_silu(x, wc, out, rows, channels, k)
    same(out, dev.causal_conv_silu_dev(as_dev(xb), torch.from_numpy(wc).cuda(), rows, channels, k), "host causal_conv_silu")
    # rope tables
    if f32:
        count, rot = 70000, 64
        pos = rng.integers(0, 1 << 20, count).astype(np.int32)
        cos, sin = np.empty((count, rot), np.float32), np.empty((count, rot), np.float32)
        host_dev.rope_tables(pos, cos, sin, count, rot, 1e7)
        want_c, want_s = dev.rope_tables_dev(torch.from_numpy(pos).cuda(), count, rot, 1e7)
        same(cos, want_c, "host rope_tables cos")
        same(sin, want_s, "host rope_tables sin")
