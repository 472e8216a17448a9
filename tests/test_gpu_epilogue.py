"""The GEMM-epilogue NVFP4 quantiser (aiis_clef_b200/csrc/nvfp4_epilogue.cuh, exported as
include/clef_nvfp4_epilogue.cuh): SwiGLU on gate/up accumulators and the block quantiser as reusable device
functions, the second half of what the reference's gated GEMM does in its epilogue (kernels/gemm.cu:882-967).

A test-side kernel (oracle/ref_probe.cu, probe_epilogue) feeds f32 "accumulators" to the device functions in the
two fragment layouts they serve, and to the reference's own header functions in the reference's fragment
layout. All three must give the bytes of clef_swiglu_quantise_nvfp4 on the same matrices, scale tile orders included."""
import numpy as np
import pytest
import torch

import aiis_clef_b200 as clef
from oracle import ref_gpu
from gpu_util import Guarded, call, ptr, stream
from util import assert_bytes_equal

pytestmark = pytest.mark.gpu
F32 = 1


def accumulators(rng, rows, cols, special=False):
    g = (rng.standard_normal((rows, cols)) * 2.5).astype(np.float32)
    u = rng.standard_normal((rows, cols)).astype(np.float32)
    u[:, rng.choice(cols, 6, replace=False)] *= 20.0
    if special:
        g[1, :16] = 0.0                       # a zero block
        g[2, 16:32] = 60.0                    # beyond the short quotient's range
        g[3, 32:48] = -90.0                   # __expf(-g) overflows: the quotient is -0
        u[4, 48:64] = 1e-30                   # subnormal scale codes
        u[5, :16] = 3e20                      # clamped scale code
        u[6, 16] = np.inf
        g[7, 33] = np.nan
        u[8, :64] = 0.0
    return torch.from_numpy(g).cuda(), torch.from_numpy(u).cuda()


@pytest.mark.parametrize("interleaved", [False, True], ids=["activation-order", "interleaved-order"])
@pytest.mark.parametrize("rows,cols,special", [(128, 64, True), (300, 1024, True), (778, 6144, False), (1, 128, False)])
def test_epilogue_device_functions_equal_the_standalone_kernel_and_the_reference_header(rows, cols, special, interleaved):
    rng = np.random.default_rng(rows + cols)
    rows_padded = (rows + 127) // 128 * 128
    accg, accu = accumulators(rng, rows_padded, cols, special)
    gscale_g, gscale_u, out_global = 0.37, 1.9, 448.0 * 6.0 / 200.0
    # the standalone entry point on the scaled matrices (f32 activations: the literal arithmetic of the reference)
    gg, gu = (accg * np.float32(gscale_g)).contiguous(), (accu * np.float32(gscale_u)).contiguous()
    packed, scales = Guarded(rows_padded * cols // 2), Guarded(rows_padded * cols // 16)
    assert call("clef_swiglu_quantise_nvfp4_ex", stream(), ptr(gg), ptr(gu), packed.ptr, scales.ptr, rows, cols, out_global, 128, 512,
                F32, 1 if interleaved else 0) == 0
    torch.cuda.synchronize()
    want_p, want_s = packed.bytes(), scales.bytes()
    names = {0: "a thread holds the block", 1: "mma.sync fragment layout", 2: "reference header, fragment layout"}
    for mode in (2, 1, 0):
        got_p, got_s = ref_gpu.probe_epilogue(accg, accu, rows, rows_padded, cols, gscale_g, gscale_u, out_global, mode,
                                              interleaved=interleaved)
        torch.cuda.synchronize()
        assert_bytes_equal(got_s.cpu().numpy(), want_s, f"scales, {names[mode]}")
        assert_bytes_equal(got_p.cpu().numpy(), want_p, f"packed, {names[mode]}")


def test_epilogue_bytes_equal_the_tuned_kernel_on_bf16_accumulators():
    """With accumulators that are bf16 values (and unit scales) the epilogue functions must give the bytes of the tuned
    bf16 SwiGLU + NVFP4 kernel, which takes the short quotient through a different instruction sequence."""
    rows, cols = 384, 6144
    rng = np.random.default_rng(5)
    g = torch.from_numpy((rng.standard_normal((rows, cols)) * 2.0).astype(np.float32)).cuda().to(torch.bfloat16)
    u = torch.from_numpy(rng.standard_normal((rows, cols)).astype(np.float32)).cuda().to(torch.bfloat16)
    dev = clef.Device(0)
    want_p, want_s = dev.swiglu_quantise_nvfp4_dev(g, u, rows, cols, 48.0, 128)
    for mode in (0, 1):
        got_p, got_s = ref_gpu.probe_epilogue(g.float().contiguous(), u.float().contiguous(), rows, rows, cols, 1.0, 1.0, 48.0, mode)
        torch.cuda.synchronize()
        assert torch.equal(got_s, want_s) and torch.equal(got_p, want_p.view(-1))
