// Test infrastructure (oracle build only): the four half-precision helpers the
// reference takes from simde, expressed with the compiler's native _Float16
// (IEEE binary16, round-to-nearest-even conversions, as simde's native path).
#pragma once
#include <cstdint>
#include <cstring>

typedef _Float16 simde_float16;

static inline simde_float16 simde_uint16_as_float16(uint16_t v) { simde_float16 r; std::memcpy(&r, &v, sizeof(r)); return r; }
static inline uint16_t simde_float16_as_uint16(simde_float16 v) { uint16_t r; std::memcpy(&r, &v, sizeof(r)); return r; }
static inline float simde_float16_to_float32(simde_float16 v) { return static_cast<float>(v); }
static inline simde_float16 simde_float16_from_float32(float v) { return static_cast<simde_float16>(v); }
