// Shared between the translation units of libclef_fused.so (not installed).
#pragma once

namespace clef {

// Records a message for clef_last_error() on the calling thread and returns `code`.
int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

// 0: tuned kernels where the shape allows (default); 1: shape-general kernels only (clef_set_kernel_choice).
int kernel_choice();

// CLEF_SF_ACTIVATION (default) or CLEF_SF_INTERLEAVED (clef_set_scale_layout).
int scale_layout();

}  // namespace clef
