// Empty stand-in: the reference only uses ABSL_UNREACHABLE and has its own
// fallback when that macro is undefined.
#pragma once
