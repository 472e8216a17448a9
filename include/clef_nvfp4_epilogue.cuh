/* Device-side companion of clef_fused.h for CUDA translation units that hold a GEMM: the NVFP4 activation
 * quantiser of a gated-GEMM epilogue as reusable __device__ functions, so that a GEMM (a tcgen05 kernel on
 * B200) can write the NVFP4 operand of the next projection straight from its accumulators instead of
 * running clef_swiglu_quantise_nvfp4 on a stored gate/up matrix.
 *
 * Replaces: the epilogue of aiis-clef's gated NVFP4 GEMM, kernels/gemm.cu:882-967 (SwiGLU on the accumulator
 * fragment at :895-921, the block maximum across the fragment's four lanes at :932-933, to_e4m3 / to_e2m1 at
 * :938-958, the tiled scale address at :945-951).
 *
 *   clef::swiglu_epilogue_value(accg, accu, gscale_g, gscale_u)            one value
 *   clef::nvfp4_swiglu_epilogue_block16(accg[16], accu[16], ...)           a thread holds the block (tcgen05.ld 32x32b)
 *   clef::nvfp4_swiglu_epilogue_quad4(accg[4], accu[4], ..., row_live)      four lanes hold the block (mma.sync m16n8)
 *   clef::nvfp4_quantise_block16 / nvfp4_quantise_quad4                     the quantiser alone, any activation
 *   clef::nvfp4_scale_offset(row, block, blocks_per_row, blk_mn, order)    scale address, both tile orders
 *
 * The bytes equal clef_swiglu_quantise_nvfp4 on accg * gscale_g and accu * gscale_u. Header-only; compile with
 * nvcc for sm_100a. This file forwards to the implementation kept beside the kernels. */
#pragma once

#include "../aiis_clef_b200/csrc/nvfp4_epilogue.cuh"
