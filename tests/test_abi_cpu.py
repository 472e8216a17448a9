"""CPU-only checks of the C-ABI library: it builds for sm_100a, loads, exports every symbol the header
declares, and refuses bad arguments before touching CUDA. No kernel is launched here."""
import ctypes
import re
from pathlib import Path

import pytest

import aiis_clef_b200 as clef
from aiis_clef_b200 import lib as clef_lib_mod

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "clef_fused.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(clef_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(clef_lib):
    names = declared_symbols()
    assert len(names) >= 16
    assert set(names) == set(clef_lib_mod.SYMBOLS), "include/clef_fused.h and the ctypes table list different symbols"
    for name in names:
        assert hasattr(clef_lib, name), f"{name} is declared but not exported"


def test_version_and_layout_helpers(clef_lib):
    assert clef_lib.clef_version() >= 100
    # src/swizzle.rs:372-380 (the_96_row_atom_matches_the_reference_strides)
    assert clef.sf_atom_for_tile_m(192) == (96, 384)
    assert clef.sf_atom_for_tile_m(128) == (128, 512)
    assert clef.sf_atom_for_tile_m(64) == (128, 512)
    assert clef.sf_atom_for_tile_m(256) == (128, 512)
    assert clef.sf_atom_for_tile_m(160) == (32, 128)
    with pytest.raises(clef.ClefError):
        clef.sf_atom_for_tile_m(0)
    # src/cuda/mod.rs:7594-7596, 8168-8172: output sizes
    assert clef.nvfp4_sizes(7, 12288, 128) == (128, 128 * 6144, 128 * 768)
    assert clef.nvfp4_sizes(769, 12288, 128) == (896, 896 * 6144, 896 * 768)
    assert clef.nvfp4_sizes(130712, 2048, 128) == (130816, 130816 * 1024, 130816 * 128)
    assert clef.nvfp4_sizes(0, 64, 128) == (0, 0, 0)
    assert clef.nvfp4_m_tile_for(778) == 128


def test_bad_arguments_are_refused_before_cuda(clef_lib):
    p = ctypes.c_void_p(0x1000)   # never dereferenced: every call below is refused on its arguments
    lib = clef_lib
    assert lib.clef_quantise_nvfp4(None, p, p, p, 4, 100, 1.0, 128, 512, 0) == -1
    assert b"multiple of 64" in lib.clef_last_error()
    assert lib.clef_quantise_nvfp4(None, None, p, p, 4, 128, 1.0, 128, 512, 0) == -1
    assert lib.clef_quantise_nvfp4(None, p, p, p, 4, 128, 1.0, 128, 512, 3) == -1
    assert lib.clef_quantise_nvfp4(None, p, p, p, -1, 128, 1.0, 128, 512, 0) == -1
    assert lib.clef_quantise_nvfp4(None, p, p, p, 4, 128, 1.0, 128, 256, 0) == -1
    assert lib.clef_quantise_nvfp4(None, ctypes.c_void_p(0x1004), p, p, 4, 128, 1.0, 128, 512, 0) == -1
    assert lib.clef_rms_norm(None, p, p, p, 4, 30, 1e-6, 0) == -1
    assert lib.clef_rms_norm_gated(None, p, p, p, None, 4, 128, 1e-6, 0) == -1
    assert lib.clef_rope(None, p, p, p, p, 4, 2, 128, 64, None, None, None, 0) == -1          # out aliases x
    assert lib.clef_rope(None, p, ctypes.c_void_p(0x2000), p, p, 4, 2, 128, 130, None, None, None, 0) == -1
    assert lib.clef_qk_norm_rope(None, p, p, p, p, p, None, 4, 2, 4096, 64, 1e-6, None, None, None, 0) == -3
    assert lib.clef_rms_norm_gated_quantise_nvfp4(None, p, p, p, p, p, 100, 128, 1e-6, 1.0, 128, 512, 16, 64, 0) == -1
    assert lib.clef_rms_norm_gated_quantise_nvfp4(None, p, p, p, p, p, 160, 128, 1e-6, 1.0, 128, 512, 16, 64, 0) == -1
    assert b"blk_mn" in lib.clef_last_error()
    assert lib.clef_embed_gather(None, p, p, p, 4, 7, 0) == -1
    assert lib.clef_to_bf16_scatter(None, p, p, 64, p, 12, 1) == -1                               # stride % 8
    assert lib.clef_to_bf16_scatter(None, p, p, 64, None, 32, 1) == -1                            # no position map
    assert lib.clef_rope_kv_write(None, p, p, p, p, p, p, 4, 2, 100, 64, None, None, None, None, None, 0) == -1   # head_dim % 8
    assert lib.clef_rope_kv_write(None, p, None, p, p, p, p, 4, 2, 128, 64, None, None, None, None, None, 0) == -1
    assert lib.clef_qk_norm_rope_kv_write(None, p, p, p, p, p, p, p, 4, 2, 4096, 64, 1e-6, None, None, None, None, None, 0) == -3
    assert lib.clef_sigmoid_mul_quantise_nvfp4(None, p, p, p, p, 4, 100, 1.0, 128, 512, 0) == -1
    assert lib.clef_add_rms_norm_quantise_nvfp4(None, None, p, p, p, p, p, 4, 2048, 1e-6, 1.0, 128, 512, 0) == -1
    assert lib.clef_add(None, p, p, ctypes.c_void_p(0x1004), 64, 0) == -1
    # the interleaved scale-tile order interleaves 32-row groups: an atom that is not a multiple of 32 is refused
    assert lib.clef_quantise_nvfp4_ex(None, p, p, p, 4, 128, 1.0, 48, 192, 0, 1) == -1
    assert b"blk_mn % 32" in lib.clef_last_error()
    assert lib.clef_quantise_nvfp4_ex(None, p, p, p, 4, 128, 1.0, 16, 64, 0, 1) == -1
    assert lib.clef_quantise_nvfp4_ex(None, p, p, p, 4, 128, 1.0, 128, 512, 0, 7) == -1          # no such order
    assert lib.clef_quantise_nvfp4_ex(None, p, p, p, 0, 128, 1.0, 96, 384, 0, 1) == 0            # 96 = 3 x 32 is fine
    assert lib.clef_set_scale_layout(1) == 0
    try:
        assert lib.clef_quantise_nvfp4(None, p, p, p, 4, 128, 1.0, 48, 192, 0) == -1             # the process default applies
        assert lib.clef_quantise_nvfp4_ex(None, p, p, p, 0, 128, 1.0, 48, 192, 0, 0) == 0        # a per-call order overrides it
    finally:
        assert lib.clef_set_scale_layout(0) == 0
    # zero-sized work is accepted without a device
    assert lib.clef_sigmoid_mul(None, p, p, p, 0, 0) == 0
    assert lib.clef_add(None, p, p, p, 0, 1) == 0
    assert lib.clef_to_bf16(None, p, p, 0, None, 0, 1) == 0
    assert lib.clef_rope_kv_write(None, p, p, p, p, p, p, 0, 2, 128, 64, None, None, None, None, None, 0) == 0
    assert lib.clef_quantise_nvfp4(None, p, p, p, 0, 128, 1.0, 128, 512, 0) == 0
    assert lib.clef_swiglu(None, p, p, p, 0, 0) == 0
    assert lib.clef_embed_gather(None, p, p, p, 0, 2048, 0) == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(clef_lib_mod, "_lib", None)
    monkeypatch.setattr(clef_lib_mod, "LIB_PATH", tmp_path / "libclef_fused.so")
    with pytest.raises(clef.ClefError, match="no CPU or PyTorch fallback"):
        clef_lib_mod.load()
