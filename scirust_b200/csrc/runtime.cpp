// CPU runtime library (no CUDA dependency). Entry points are plain C so Python reaches them with
// ctypes. This file holds the version probe; the other translation units add the deterministic
// fp32 math, allocators, collectives and samplers.
#include <stdint.h>

extern "C" int sbrt_version() { return 1; }
