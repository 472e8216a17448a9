"""CPU tests of the host-side companions: per-token maps, the rung ladder, the multi-GPU row split.
The expectations restate the reference's own unit tests (paths inside the aiis-clef tree)."""
import re
from pathlib import Path

import numpy as np
import pytest

import aiis_clef_b200 as clef
from aiis_clef_b200 import lib as clef_lib_mod

ROOT = Path(__file__).resolve().parent.parent


def test_host_header_and_binding_agree(clef_lib):
    text = (ROOT / "include" / "clef_host.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = sorted(set(re.findall(r"\b(clef_[a-z0-9_]+)\s*\(", text)))
    assert set(names) == set(clef_lib_mod.HOST_SYMBOLS)
    lib = clef.load_host()
    for name in names:
        assert hasattr(lib, name), f"{name} is declared but not exported"


def test_pass_maps_describe_the_whole_request():
    """src/gpu.rs:4118-4186 pass_maps_must_describe_the_whole_request."""
    capacity = 4096
    ids = (100 + (np.arange(4096) % 900)).astype(np.uint32)
    cases = [
        [(ids, 0, 0, 4096)], [(ids, 0, 0, 2048)], [(ids, 2048, 0, 2048)], [(ids, 0, 0, 1024)],
        [(ids, 1024, 0, 1024)], [(ids, 3072, 0, 1024)], [(ids[:700], 384, 0, 384)],
        [(ids, 0, 0, 1024), (ids, 1024, 1, 1024)],
    ]
    for chunks in cases:
        m = clef.pass_maps(chunks, capacity)
        total = sum(c[3] for c in chunks)
        assert m["total"] == total
        for key in ("cpos", "cbase", "seq_end", "ids", "seq_start", "slot_map", "rope_pos"):
            assert m[key].size == total
        assert m["chunk_start"].size == total // 64 and m["state_slot"].size == total // 64
        for i, (req, pos, slot, rows) in enumerate(chunks):
            off, real = int(m["offs"][i]), int(m["rows_real"][i])
            assert real == min(rows, req.size - pos)
            seg = slot * capacity
            t = np.arange(rows)
            sl = slice(off, off + rows)
            assert (m["cbase"][sl] == seg).all()
            assert (m["cpos"][sl] == seg + pos + t).all()
            assert (m["rope_pos"][sl] == pos + t).all()
            assert (m["seq_end"][sl] == off + real).all()
            assert (m["seq_start"][sl] == off).all()
            assert (m["slot_map"][sl] == slot).all()
            assert (m["ids"][off:off + real] == req[pos:pos + real]).all()
            assert (m["ids"][off + real:off + rows] == req[-1]).all()          # pad rows repeat the last id
            assert tuple(m["hist_save"][i]) == (off + real - 1, slot)
            g0 = off // 64
            assert m["chunk_start"][g0] == (1 if i > 0 else 0)
            assert (m["chunk_start"][g0 + 1:g0 + rows // 64] == 0).all()
            assert (m["state_slot"][g0:g0 + rows // 64] == slot).all()
        assert m["cache_len"] == min(slot * capacity + pos for _, pos, slot, _ in chunks)
    assert clef.pass_maps([], capacity)["cache_len"] == 0


def test_pass_maps_refusals():
    ids = np.arange(100, dtype=np.uint32)
    with pytest.raises(clef.ClefError, match="granule"):
        clef.pass_maps([(ids, 0, 0, 100)], 4096)
    with pytest.raises(clef.ClefError, match="share slot"):
        clef.pass_maps([(ids, 0, 3, 64), (ids, 0, 3, 64)], 4096)
    with pytest.raises(clef.ClefError, match="at least one token"):
        clef.pass_maps([(np.zeros(0, np.uint32), 0, 0, 64)], 4096)
    with pytest.raises(clef.ClefError, match="graphed geometry"):
        clef.pass_maps([(ids, 0, 0, 192)], 4096, check_geometry=True)
    assert clef.pass_maps([(ids, 0, 0, 128)], 4096, check_geometry=True)["total"] == 128


def test_rung_ladder():
    """src/gpu.rs:4204-4287 the_two_ladders_agree_on_their_primitives."""
    assert clef.pass_geometries(1, 8192) == [64, 128, 256, 512, 1024, 2048, 4096, 8192]
    assert clef.rungs_decompose(16717) == [(0, 8192), (8192, 8192), (16384, 256), (16640, 64), (16704, 64)]
    assert [r for _, r in clef.rungs_decompose(6144, slots=1)] == [4096, 2048]
    assert [r for _, r in clef.rungs_decompose(6144, slots=3)] == [6144]
    # a chunk limit that is not a multiple of the 64-row granule is kept as it is (Rungs::body_at clamps to
    # max(top, 64) only, src/gpu.rs:715): the ladder ends in the limit itself
    assert clef.pass_geometries(1, 1000) == [64, 128, 256, 512, 1000]
    assert clef.pass_geometries(1, 10) == [64]
    assert [r for _, r in clef.rungs_decompose(2100, slots=1, max_chunk=1000)] == [1000, 1000, 64, 64]
    cut = clef.rungs_decompose(130712)
    assert sum(r for _, r in cut) >= 130712 and sum(r for _, r in cut) - 130712 < 64
    assert all(a[0] + a[1] == b[0] for a, b in zip(cut, cut[1:]))
    g4 = clef.pass_geometries(4, 8192)
    assert 16384 in g4 and 32768 in g4 and 24576 in g4 and g4 == sorted(set(g4))
    assert all(g % 64 == 0 for g in g4)


def test_shard_rows_cover_the_pass():
    for rows in (0, 1, 127, 128, 129, 8192, 70000, 130712):
        for n in (1, 2, 4, 8):
            spans = [clef.shard_rows(rows, 128, n, g) for g in range(n)]
            assert spans[0][0] == 0
            for (a0, an), (b0, _) in zip(spans, spans[1:]):
                assert a0 + an == b0
            assert sum(s[1] for s in spans) == rows
            for first, count in spans:
                assert count == 0 or first % 128 == 0
            for first, count in spans:
                if count and first + count != rows:
                    assert count % 128 == 0
    # 130,712 rows: 130,816 / 65,408 / 32,768 / 16,384 padded rows per GPU at 1 / 2 / 4 / 8 GPUs
    for n, padded in ((1, 130816), (2, 65408), (4, 32768), (8, 16384)):
        first, count = clef.shard_rows(130712, 128, n, 0)
        assert -(-count // 128) * 128 == padded
    with pytest.raises(clef.ClefError):
        clef.shard_rows(10, 128, 2, 2)
