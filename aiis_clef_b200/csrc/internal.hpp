// Shared between the translation units of libclef_fused.so (not installed).
#pragma once

namespace clef {

// Records a message for clef_last_error() on the calling thread and returns `code`.
int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

}  // namespace clef
