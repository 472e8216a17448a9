// Launcher of the unit-structured f32 quantisers, shared by the translation units that dispatch to them.
#pragma once

#include "abi_support.cuh"
#include "kernels_hot.cuh"

namespace clef {
namespace abi {

// The unit-structured f32 quantisers (MODE 0 plain, 1 SwiGLU first, 2 x * sigmoid(gate) first); one unit per warp per step.
template <int MODE>
inline void launch_unit_quant_f32(cudaStream_t s, const DeviceInfo& dev, const float* gate, const float* up, uint8_t* packed,
                                  uint8_t* scales, int rows, int rows_total, int cols, float global_scale, int blk_mn,
                                  int chunk) {
    constexpr int kMinCtas = MODE == 0 ? 4 : 3;
    static std::atomic<int> occ{0};
    const int per_sm = ctas_per_sm(unit_quant_f32_hot_kernel<MODE, kMinCtas>, 0, occ);
    const uint32_t segs = (uint32_t)(cols / 512);
    const uint32_t live_units = (uint32_t)rows * segs, total_units = (uint32_t)rows_total * segs;
    const size_t ctas = ((size_t)total_units + 7) / 8;
    launch_hot(unit_quant_f32_hot_kernel<MODE, kMinCtas>, clamp_grid(ctas, (size_t)dev.sms * per_sm), 0, s, gate, up, packed,
               scales, live_units, total_units, cols, global_scale, blk_mn, chunk, make_fast_div(segs),
               make_fast_div((uint32_t)blk_mn));
}

}  // namespace abi
}  // namespace clef
