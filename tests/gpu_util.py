"""Helpers of the GPU parity tests: raw C-ABI calls into guarded buffers, uploads, comparisons."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

import aiis_clef_b200 as clef
from aiis_clef_b200 import lib as _lib
from oracle import binding as orc

GUARD = 256          # guard bytes before and after every output (keeps 256-byte alignment)
POISON = 0xA5


def dev_bf16(bits: np.ndarray) -> torch.Tensor:
    """uint16 bf16 bit patterns -> CUDA bfloat16 tensor of the same shape."""
    return orc.bits_to_torch_bf16(bits).cuda()


def dev_f32_from_bits(bits: np.ndarray) -> torch.Tensor:
    """bf16 bit patterns widened exactly to a CUDA float32 tensor (input of the reference kernels)."""
    return torch.from_numpy(orc.bf16_to_f32(bits)).cuda()


def host_bits(t: torch.Tensor) -> np.ndarray:
    return orc.bf16_bits(t.detach().cpu())


def f32_to_bf16_bits_gpu(t: torch.Tensor) -> np.ndarray:
    """Round a CUDA f32 tensor to bf16 (nearest even) and return the bit patterns."""
    return host_bits(t.to(torch.bfloat16))


class Guarded:
    """A device byte buffer with poisoned guard bands; `.ptr` addresses the payload."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        self.buf = torch.full((self.nbytes + 2 * GUARD,), POISON, dtype=torch.uint8, device="cuda")

    @property
    def ptr(self):
        return ctypes.c_void_p(self.buf.data_ptr() + GUARD)

    def payload(self) -> torch.Tensor:
        return self.buf[GUARD:GUARD + self.nbytes]

    def check_guards(self, what: str):
        head = self.buf[:GUARD].cpu().numpy()
        tail = self.buf[GUARD + self.nbytes:].cpu().numpy()
        assert (head == POISON).all(), f"{what}: bytes before the buffer were written"
        assert (tail == POISON).all(), f"{what}: bytes after the buffer were written"

    def bytes(self) -> np.ndarray:
        return self.payload().cpu().numpy()

    def as_bf16_bits(self) -> np.ndarray:
        return self.bytes().view(np.uint16)

    def as_f32(self) -> np.ndarray:
        return self.bytes().view(np.float32)


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def call(name: str, *args) -> int:
    """Call a C-ABI entry point; negative statuses raise with the library's message."""
    st = getattr(clef.load(), name)(*args)
    if st < 0:
        raise _lib.ClefError(f"{name} -> {st}: {_lib.last_error()}")
    return st


def quant_sizes(rows, cols, blk_mn=128):
    rows_padded = (rows + blk_mn - 1) // blk_mn * blk_mn
    return rows_padded, rows_padded * (cols // 2), rows_padded * (cols // 16)


# ---- comparisons ----------------------------------------------------------------------------------------
E2M1_THRESHOLDS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float64)


def unswizzle(scales: np.ndarray, rows_padded: int, blocks: int, blk_mn=128) -> np.ndarray:
    """Tiled activation-side scale bytes -> [rows_padded, blocks] (numpy, any atom)."""
    chunk = blk_mn * 4
    r = np.arange(rows_padded)[:, None]
    b = np.arange(blocks)[None, :]
    idx = ((r // blk_mn) * (blocks // 4) + b // 4) * chunk + (r % blk_mn) * 4 + b % 4
    return scales[idx]


def explain_mismatches(pre: np.ndarray, global_scale: float, got_packed, got_scales, want_packed, want_scales,
                       rows: int, cols: int, blk_mn=128, rel=4e-6):
    """Compare a GPU result with the CPU oracle for a kernel whose GPU arithmetic uses approximate
    intrinsics. `pre` holds the oracle's f32 values before quantisation ([rows, cols]).
    A differing scale byte is accepted when the oracle's scale argument is within `rel` of an E4M3
    rounding edge (both bytes are reachable); a differing code in a block with equal scale bytes is
    accepted when the oracle's scaled value is within `rel` (relative, or 1e-30 absolute) of an E2M1
    threshold or of zero. Returns (scale_mismatches, code_mismatches, unexplained)."""
    blocks = cols // 16
    rows_padded = (rows + blk_mn - 1) // blk_mn * blk_mn
    gs = unswizzle(np.asarray(got_scales), rows_padded, blocks, blk_mn)[:rows]
    ws = unswizzle(np.asarray(want_scales), rows_padded, blocks, blk_mn)[:rows]
    gp = np.asarray(got_packed).reshape(rows_padded, cols // 2)[:rows]
    wp = np.asarray(want_packed).reshape(rows_padded, cols // 2)[:rows]
    unexplained = 0
    scale_diff = gs != ws
    n_scale = int(scale_diff.sum())
    if n_scale:
        amax = np.abs(pre.reshape(rows, blocks, 16)).max(axis=2)
        sv = (amax / np.float32(6.0)).astype(np.float32) * np.float32(global_scale)
        lo = orc.to_e4m3_many((sv.astype(np.float64) * (1 - rel)).astype(np.float32))
        hi = orc.to_e4m3_many((sv.astype(np.float64) * (1 + rel)).astype(np.float32))
        ok = (np.minimum(lo, hi) <= gs) & (gs <= np.maximum(lo, hi)) & (lo != hi)
        unexplained += int((scale_diff & ~ok).sum())
    code_diff_bytes = (gp != wp) & ~np.repeat(scale_diff, 8, axis=1)
    n_code = 0
    if code_diff_bytes.any():
        table = orc.e4m3_table()
        stored_f = table[ws]
        inv = np.where(stored_f > 0, np.float32(global_scale) / np.where(stored_f > 0, stored_f, 1), 0).astype(np.float32)
        p = np.abs(pre.reshape(rows, blocks, 16) * inv[:, :, None]).astype(np.float64).reshape(rows, cols)
        near = (np.abs(p[:, :, None] - E2M1_THRESHOLDS[None, None, :]) <= rel * np.maximum(p[:, :, None], 1e-3)).any(axis=2)
        near |= p <= 1e-30
        g_lo, g_hi = gp & 0xF, gp >> 4
        w_lo, w_hi = wp & 0xF, wp >> 4
        diff_el = np.empty((rows, cols), bool)
        diff_el[:, 0::2] = g_lo != w_lo
        diff_el[:, 1::2] = g_hi != w_hi
        diff_el &= ~np.repeat(scale_diff, 16, axis=1)
        n_code = int(diff_el.sum())
        unexplained += int((diff_el & ~near).sum())
    return n_scale, n_code, unexplained
