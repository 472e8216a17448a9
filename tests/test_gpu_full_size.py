"""Full-size cases of BASELINE.json: 70,000 rows (above the reference launch layer's 65,535 grid.y fold,
src/cuda/mod.rs:7701-7758) and the 130,712-row pass, compared ON THE DEVICE with the reference's own
kernels (bit-exact NVFP4, bf16 within the ulp bounds), plus size-independent properties: the row-range
shards of a pass concatenate to the single-GPU bytes, pad rows are zero, a graph replay equals the eager call."""
import numpy as np
import pytest
import torch

import aiis_clef_b200 as clef
from oracle import ref_gpu

pytestmark = pytest.mark.gpu

HIDDEN, INTER, VH = 2048, 6144, 16


def randn_bf16(gen, *shape):
    return torch.randn(*shape, device="cuda", generator=gen, dtype=torch.float32).to(torch.bfloat16)


@pytest.fixture(autouse=True)
def _cleanup():
    clef.set_kernel_choice(0)
    yield
    torch.cuda.empty_cache()


def ulp_key(t: torch.Tensor) -> torch.Tensor:
    b = t.view(torch.int16).to(torch.int32) & 0xFFFF
    return torch.where((b & 0x8000) != 0, 0x8000 - b, b)


def max_bf16_ulp(a: torch.Tensor, b: torch.Tensor) -> int:
    return int((ulp_key(a) - ulp_key(b)).abs().max())


@pytest.mark.parametrize("rows", [70000, 130712])
def test_rms_norm_quantise_full_size(rows):
    dev = clef.Device(0)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(rows)
    x = randn_bf16(gen, rows, HIDDEN)
    x[:, torch.randperm(HIDDEN, device="cuda", generator=gen)[:8]] *= 20.0
    w = torch.randn(HIDDEN, device="cuda", generator=gen) * 0.1
    gs = 448.0 * 6.0 / 30.0
    packed, scales = dev.rms_norm_quantise_nvfp4_dev(x, w, rows, HIDDEN, 1e-6, gs, 128)
    normed = ref_gpu.rms_norm(x.float(), w, rows, HIDDEN, 1e-6)
    ref_p, ref_s = ref_gpu.quantise_nvfp4(normed, rows, HIDDEN, gs)
    assert torch.equal(packed.view(-1), ref_p) and torch.equal(scales, ref_s)
    rows_padded = packed.shape[0]
    assert rows_padded % 128 == 0 and not packed[rows:].any()           # pad rows are zero codes
    assert packed[rows - 1].any()                                         # the last live row was written
    # bf16 norm output: the reference f32 result rounded to nearest even (the tuned kernel keeps the same tree)
    out = dev.rms_norm_dev(x, w, rows, HIDDEN, 1e-6)
    assert max_bf16_ulp(out, normed.to(torch.bfloat16)) <= 1
    # plain quantiser on the same activations
    p2, s2 = dev.quantise_nvfp4_dev(x, rows, HIDDEN, 3.0, 128)
    r2p, r2s = ref_gpu.quantise_nvfp4(x.float(), rows, HIDDEN, 3.0)
    assert torch.equal(p2.view(-1), r2p) and torch.equal(s2, r2s)


@pytest.mark.parametrize("rows", [70000, 130712])
def test_swiglu_quantise_full_size(rows):
    dev = clef.Device(0)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(rows + 1)
    gate, up = randn_bf16(gen, rows, INTER), randn_bf16(gen, rows, INTER)
    packed, scales = dev.swiglu_quantise_nvfp4_dev(gate, up, rows, INTER, 48.0, 128)
    ref_p, ref_s = ref_gpu.swiglu_quantise_nvfp4(gate.float(), up.float(), rows, INTER, 48.0)
    assert torch.equal(packed.view(-1), ref_p) and torch.equal(scales, ref_s)
    del ref_p, ref_s
    act = dev.swiglu_dev(gate, up, rows * INTER)
    ref_act = ref_gpu.swiglu(gate.float(), up.float(), rows * INTER)
    assert max_bf16_ulp(act, ref_act.to(torch.bfloat16)) <= 1


def test_gated_norm_quantise_full_size():
    tokens = 130712
    dev = clef.Device(0)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(3)
    o, z = randn_bf16(gen, tokens * VH, 128), randn_bf16(gen, tokens * VH, 128)
    w = 1.0 + torch.randn(128, device="cuda", generator=gen) * 0.1
    packed, scales = dev.rms_norm_gated_quantise_nvfp4_dev(o, z, w, tokens * VH, 128, VH, 1e-6, 96.0, 128)
    ref_p, ref_s = ref_gpu.rms_norm_gated_quantise_nvfp4(o.float(), z.float(), w, tokens * VH, 128, VH, 1e-6, 96.0)
    assert torch.equal(packed.view(-1), ref_p) and torch.equal(scales, ref_s)
    out = dev.rms_norm_gated_dev(o, z, w, tokens * VH, 128, 1e-6)
    ref = ref_gpu.rms_norm_gated(o.float(), z.float(), w, tokens * VH, 128, 1e-6)
    assert max_bf16_ulp(out, ref.to(torch.bfloat16)) <= 1


def test_rope_and_embed_full_size():
    rows = 130712
    dev = clef.Device(0)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4)
    positions = torch.arange(rows, dtype=torch.int32, device="cuda")       # one request of 130,712 tokens at slot 0
    cos, sin = dev.rope_tables_dev(positions, rows, 64, 1e7)
    rc, rs = ref_gpu.rope_tables(positions, rows, 64, 1e7)
    assert torch.equal(cos, rc) and torch.equal(sin, rs)
    for heads in (16, 2):
        x = randn_bf16(gen, rows, heads, 128)
        out = dev.rope_apply_dev(x, cos, sin, rows, heads, 128, 64, pos_map=positions)
        ref = ref_gpu.rope(x.float(), cos, sin, rows, heads, 128, 64, None, None, positions)
        assert max_bf16_ulp(out, ref.to(torch.bfloat16)) <= 2
        assert torch.equal(out[:, :, 64:], x[:, :, 64:])
        # the same positions through seq_start / pos_base (row - seq_start[row] + *pos_base)
        seq_start = torch.zeros(rows, dtype=torch.int32, device="cuda")
        out2 = dev.rope_apply_dev(x, cos, sin, rows, heads, 128, 64, seq_start=seq_start,
                                  pos_base=torch.zeros(1, dtype=torch.int32, device="cuda"))
        assert torch.equal(out, out2)
    # q and k in one launch: long launches take the streaming kernel, short ones the kernel with hoisted loads; both
    # must give the bytes of the separate calls (sizes either side of the switch, and the ragged full size)
    for n in (130712, 40000, 8192, 20000):
        q, k = randn_bf16(gen, n, 16, 128), randn_bf16(gen, n, 2, 128)
        want_q = dev.rope_apply_dev(q, cos, sin, n, 16, 128, 64, pos_map=positions)
        want_k = dev.rope_apply_dev(k, cos, sin, n, 2, 128, 64, pos_map=positions)
        got_q, got_k = dev.rope_qk_dev(q, k, cos, sin, n, 16, 2, 128, 64, pos_map=positions)
        assert torch.equal(got_q, want_q) and torch.equal(got_k, want_k)
        ref = ref_gpu.rope(q.float(), cos, sin, n, 16, 128, 64, None, None, positions)
        assert max_bf16_ulp(got_q, ref.to(torch.bfloat16)) <= 2
        del q, k, want_q, want_k, got_q, got_k, ref
    vocab = 32768
    table = randn_bf16(gen, vocab, HIDDEN)
    ids = torch.randint(0, vocab, (rows,), device="cuda", generator=gen, dtype=torch.int32)
    h = dev.embed_gather_dev(table, ids, rows, HIDDEN)
    assert torch.equal(h, table[ids.long()])


def test_row_range_shards_concatenate_to_the_single_gpu_bytes():
    """The multi-GPU path without a second GPU: every shard of clef_shard_rows is run as its own call on its
    own slice of the inputs; the concatenation must equal the one-call result byte for byte."""
    rows = 130712
    dev = clef.Device(0)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    x = randn_bf16(gen, rows, HIDDEN)
    w = torch.randn(HIDDEN, device="cuda", generator=gen) * 0.1
    gate, up = randn_bf16(gen, rows, 1024), randn_bf16(gen, rows, 1024)
    full_p, full_s = dev.rms_norm_quantise_nvfp4_dev(x, w, rows, HIDDEN, 1e-6, 64.0, 128)
    full_gp, full_gs = dev.swiglu_quantise_nvfp4_dev(gate, up, rows, 1024, 48.0, 128)
    for n in (2, 4, 8):
        parts_p, parts_s, parts_gp, parts_gs = [], [], [], []
        for g in range(n):
            first, count = clef.shard_rows(rows, 128, n, g)
            p, s = dev.rms_norm_quantise_nvfp4_dev(x[first:first + count], w, count, HIDDEN, 1e-6, 64.0, 128)
            gp, gs = dev.swiglu_quantise_nvfp4_dev(gate[first:first + count], up[first:first + count], count, 1024, 48.0, 128)
            parts_p.append(p)
            parts_s.append(s)
            parts_gp.append(gp)
            parts_gs.append(gs)
        assert torch.equal(torch.cat(parts_p), full_p) and torch.equal(torch.cat(parts_s), full_s)
        assert torch.equal(torch.cat(parts_gp), full_gp) and torch.equal(torch.cat(parts_gs), full_gs)


def test_graph_replay_equals_the_eager_call():
    """src/gpu.rs:6158 a_graphed_chunk_matches_the_eager_one, for the fused step: captured once, replayed with new
    buffer CONTENTS at the same addresses."""
    rows = 8192
    dev = clef.Device(0)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(6)
    x, w = randn_bf16(gen, rows, HIDDEN), torch.randn(HIDDEN, device="cuda", generator=gen) * 0.1
    q = randn_bf16(gen, rows, 16, 128)
    pos = torch.arange(rows, dtype=torch.int32, device="cuda")
    cos, sin = dev.rope_tables_dev(pos, rows, 64, 1e7)
    dev.rms_norm_quantise_nvfp4_dev(x, w, rows, HIDDEN, 1e-6, 64.0, 128)     # warm-up outside the capture
    dev.rope_apply_dev(q, cos, sin, rows, 16, 128, 64, pos_map=pos)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        gp, gs = dev.rms_norm_quantise_nvfp4_dev(x, w, rows, HIDDEN, 1e-6, 64.0, 128)
        gq = dev.rope_apply_dev(q, cos, sin, rows, 16, 128, 64, pos_map=pos)
    for trial in range(3):
        x.copy_(randn_bf16(gen, rows, HIDDEN))
        q.copy_(randn_bf16(gen, rows, 16, 128))
        pos.copy_(torch.randint(0, rows, (rows,), device="cuda", generator=gen, dtype=torch.int32))
        graph.replay()
        ep, es = dev.rms_norm_quantise_nvfp4_dev(x, w, rows, HIDDEN, 1e-6, 64.0, 128)
        eq = dev.rope_apply_dev(q, cos, sin, rows, 16, 128, 64, pos_map=pos)
        assert torch.equal(gp, ep) and torch.equal(gs, es) and torch.equal(gq, eq)
