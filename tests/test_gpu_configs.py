"""The workload configurations of the benchmark definition, end to end through the public entry points:

  0. the single-layer chain on 778 rows (embedding gather -> RMSNorm -> NVFP4 -> dequantised check),
  2. the GDN gated RMSNorm chain, 32,768 rows as four 8,192-row chunks,
  4. the rung sweep 64 .. 8,192 rows with four coalesced requests per pass and per-token maps built from seeded
     request lengths (cpos / cbase / seq_end / rope_pos), outlier channels x20.

(Configuration 1 is the benchmark step, covered by the parity tests at its shapes; configuration 3, the
130,712-row pass, by test_gpu_full_size.py.) Arbiters: the CPU oracle, the reference kernels on the same GPU, and
the dequantiser semantics of src/dequant.rs restated by the oracle."""
import numpy as np
import pytest
import torch

import aiis_clef_b200 as clef
from oracle import binding as orc
from oracle import ref_gpu
from gpu_util import dev_bf16, unswizzle
from util import to_bf16_bits

pytestmark = pytest.mark.gpu
HIDDEN, VOCAB = 2048, 32768


@pytest.fixture(autouse=True)
def _cleanup():
    clef.set_kernel_choice(0)
    yield
    clef.set_kernel_choice(0)
    torch.cuda.empty_cache()


def bits(t):
    return orc.bf16_bits(t.cpu())


def test_config_0_single_layer_chain_on_778_rows():
    rows = 778
    rng = np.random.default_rng(778)
    table = to_bf16_bits((rng.standard_normal((VOCAB, HIDDEN)) * 0.02).astype(np.float32))
    outliers = rng.choice(HIDDEN, 8, replace=False)
    tf = orc.bf16_to_f32(table)
    tf[:, outliers] *= 20.0                                   # activations with 8 outlier channels x20
    table = to_bf16_bits(tf)
    ids = rng.integers(0, VOCAB, rows).astype(np.int32)
    w = (rng.standard_normal(HIDDEN) * 0.1).astype(np.float32)     # effective weight 1 + N(0, 0.1): the kernels add the 1
    dev = clef.Device(0)
    dt, di, dw = dev_bf16(table), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
    h = dev.embed_gather_dev(dt, di, rows, HIDDEN)
    assert np.array_equal(bits(h), table[ids])
    normed_f32, _ = orc.rms_norm(table[ids], w, rows, HIDDEN, 1e-6)
    gs = float(np.float32(448.0 * 6.0) / np.abs(normed_f32).max())
    packed, scales = dev.rms_norm_quantise_nvfp4_dev(h, dw, rows, HIDDEN, 1e-6, gs, 128)
    torch.cuda.synchronize()
    want_p, want_s = orc.rms_norm_quantise_nvfp4(table[ids], w, rows, HIDDEN, 1e-6, gs)
    got_p, got_s = packed.cpu().numpy().reshape(-1), scales.cpu().numpy()
    assert np.array_equal(got_s, want_s) and np.array_equal(got_p, want_p)
    # dequantised check (src/dequant.rs semantics; bounds of src/cuda/mod.rs:7624-7635): every value within half a
    # code step of its block scale, zero rows give zero codes
    rows_padded = packed.shape[0]
    blocks = HIDDEN // 16
    row_major = unswizzle(got_s, rows_padded, blocks, 128)[:rows]
    scale_f32 = orc.e4m3_table()[row_major]
    deq = orc.dequantise(got_p[: rows * HIDDEN // 2], scale_f32, gs, HIDDEN, rows)
    step = np.repeat(scale_f32 / np.float32(gs), 16, axis=1)            # one E2M1 unit in real units, per element
    err = np.abs(deq.reshape(rows, HIDDEN) - normed_f32)
    assert (err <= step * 1.0 + 1e-12).all()                             # E2M1 steps are at most 2 units wide
    assert not got_p[rows * HIDDEN // 2:].any()                          # pad rows are zero codes
    rel = np.linalg.norm(deq.reshape(rows, HIDDEN) - normed_f32) / np.linalg.norm(normed_f32)
    assert rel < 0.2


def test_config_2_gated_chain_in_four_chunks():
    chunk, chunks, vh = 8192, 4, 16
    gen = torch.Generator(device="cuda")
    gen.manual_seed(32768)
    dev = clef.Device(0)
    o = torch.randn(chunks * chunk * vh, 128, device="cuda", generator=gen).to(torch.bfloat16)
    z = torch.randn(chunks * chunk * vh, 128, device="cuda", generator=gen).to(torch.bfloat16)
    w = 1.0 + torch.randn(128, device="cuda", generator=gen) * 0.1
    parts_p, parts_s = [], []
    for c in range(chunks):
        sl = slice(c * chunk * vh, (c + 1) * chunk * vh)
        p, s = dev.rms_norm_gated_quantise_nvfp4_dev(o[sl], z[sl], w, chunk * vh, 128, vh, 1e-6, 96.0, 128)
        parts_p.append(p)
        parts_s.append(s)
    whole_p, whole_s = dev.rms_norm_gated_quantise_nvfp4_dev(o, z, w, chunks * chunk * vh, 128, vh, 1e-6, 96.0, 128)
    assert torch.equal(torch.cat(parts_p), whole_p) and torch.equal(torch.cat(parts_s), whole_s)
    ref_p, ref_s = ref_gpu.rms_norm_gated_quantise_nvfp4(o.float(), z.float(), w, chunks * chunk * vh, 128, vh, 1e-6, 96.0)
    assert torch.equal(whole_p.view(-1), ref_p) and torch.equal(whole_s, ref_s)


@pytest.mark.parametrize("rung", [64, 128, 256, 512, 1024, 2048, 4096, 8192])
def test_config_4_rung_with_four_coalesced_requests(rung):
    """Four requests share one pass of `rung` rows (64-row granules): ids, RoPE positions (rope_pos) and cache
    positions (cpos) come from the pass maps; each request's rows must come out exactly as if the request had been
    run alone with its own positions."""
    rng = np.random.default_rng(rung)
    capacity = 16384
    gran = rung // 64
    cuts = np.sort(rng.choice(np.arange(1, gran), 3, replace=False)) if gran >= 4 else np.arange(1, gran)
    sizes = np.diff(np.concatenate([[0], cuts, [gran]])) * 64
    chunks = []
    for slot, rows in enumerate(sizes):
        start = int(rng.integers(0, 4000))                      # tokens already in this request's cache
        live = int(rows - rng.integers(0, 40)) if rows > 64 else int(rows)   # ragged: the tail granule is padded
        req = rng.integers(0, VOCAB, start + live).astype(np.uint32)
        chunks.append((req, start, slot, int(rows)))
    m = clef.pass_maps(chunks, capacity)
    assert m["total"] == rung
    dev = clef.Device(0)
    table = to_bf16_bits((rng.standard_normal((VOCAB, HIDDEN)) * 0.02).astype(np.float32))
    tf = orc.bf16_to_f32(table)
    tf[:, rng.choice(HIDDEN, 8, replace=False)] *= 20.0
    table = to_bf16_bits(tf)
    w = (rng.standard_normal(HIDDEN) * 0.1).astype(np.float32)
    dt, dw = dev_bf16(table), torch.from_numpy(w).cuda()
    ids = torch.from_numpy(m["ids"].astype(np.int32)).cuda()
    h = dev.embed_gather_dev(dt, ids, rung, HIDDEN)
    packed, scales = dev.rms_norm_quantise_nvfp4_dev(h, dw, rung, HIDDEN, 1e-6, 64.0, 128)
    want_p, want_s = orc.rms_norm_quantise_nvfp4(table[m["ids"].astype(np.int64)], w, rung, HIDDEN, 1e-6, 64.0)
    assert np.array_equal(packed.cpu().numpy().reshape(-1), want_p) and np.array_equal(scales.cpu().numpy(), want_s)
    # RoPE over the whole pass with the pass's position map, against each request run alone
    table_rows = int(m["rope_pos"].max()) + 1
    cos, sin = dev.rope_tables_dev(torch.arange(table_rows, dtype=torch.int32, device="cuda"), table_rows, 64, 1e7)
    q = torch.randn(rung, 16, 128, device="cuda").to(torch.bfloat16)
    k = torch.randn(rung, 2, 128, device="cuda").to(torch.bfloat16)
    v = torch.randn(rung, 2, 128, device="cuda").to(torch.bfloat16)
    rope_pos = torch.from_numpy(m["rope_pos"]).cuda()
    q_all = dev.rope_apply_dev(q, cos, sin, rung, 16, 128, 64, pos_map=rope_pos)
    cache_rows = capacity * len(chunks)
    cache_k = torch.zeros(cache_rows, 2, 128, dtype=torch.bfloat16, device="cuda")
    cache_v = torch.zeros(cache_rows, 2, 128, dtype=torch.bfloat16, device="cuda")
    cpos = torch.from_numpy(m["cpos"]).cuda()
    dev.rope_kv_write_dev(cache_k, cache_v, k, v, cos, sin, rung, 2, 128, 64, pos_map=rope_pos, cache_map=cpos)
    for i, (req, start, slot, rows) in enumerate(chunks):
        off = int(m["offs"][i])
        sl = slice(off, off + rows)
        assert (m["cbase"][sl] == slot * capacity).all() and (m["seq_end"][sl] == off + int(m["rows_real"][i])).all()
        # alone: positions start .. start + rows through seq_start / pos_base instead of a map
        alone = dev.rope_apply_dev(q[sl].contiguous(), cos, sin, rows, 16, 128, 64,
                                   pos_base=torch.tensor([start], dtype=torch.int32, device="cuda"))
        assert torch.equal(q_all[sl], alone)
        k_alone = dev.rope_apply_dev(k[sl].contiguous(), cos, sin, rows, 2, 128, 64,
                                     pos_base=torch.tensor([start], dtype=torch.int32, device="cuda"))
        seg = slice(slot * capacity + start, slot * capacity + start + rows)
        assert torch.equal(cache_k[seg], k_alone) and torch.equal(cache_v[seg], v[sl])
    written = torch.zeros(cache_rows, dtype=torch.bool, device="cuda")
    written[cpos.long()] = True
    assert not cache_k[~written].any() and not cache_v[~written].any()
