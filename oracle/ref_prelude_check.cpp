// TEST INFRASTRUCTURE ONLY.  A thin C wrapper over arithmetic primitives of the reference's own CPU prelude,
// compiled from the reference sources where they lie (never copied into this repository) into
// oracle/_ref/libref_prelude.so by oracle/Makefile when the reference tree is present.  The tests use it to
// check the oracle's number formats and elementary functions against the code the reference's CPU target
// links: `half` conversions (prelude/slang-cpp-scalar-intrinsics.h:563-636, struct half :670-741) and the
// F32_* math wrappers (:142-247).  The example kernels themselves cannot be built from the reference (they
// need its compiler), so this pins the arithmetic the kernels are made of, not the kernels.
#include "slang-cpp-prelude.h"

extern "C" {
unsigned ref_f32tof16(float v) { return f32tof16(v); }
float ref_f16tof32(unsigned bits) { return f16tof32(bits); }
// Arithmetic on the prelude's `half` type, whatever it resolves to with this compiler (_Float16 with GCC 12 and
// later, :664-666; the struct with f32tof16 / f16tof32 otherwise).  Results are stored to a half before they
// are read back, as the generated code stores every NFloat value.
static half from_bits(unsigned b) { half h; uint16_t u = (uint16_t)b; memcpy(&h, &u, 2); return h; }
static unsigned to_bits(half h) { uint16_t u; memcpy(&u, &h, 2); return u; }
unsigned ref_half_add(unsigned a, unsigned b) { volatile half r = from_bits(a) + from_bits(b); return to_bits(r); }
unsigned ref_half_mul(unsigned a, unsigned b) { volatile half r = from_bits(a) * from_bits(b); return to_bits(r); }
unsigned ref_half_from_float(float v) { volatile half r = (half)v; return to_bits(r); }
int ref_half_is_builtin(void) { return sizeof(half) == 2 && (half)1.5f == (half)1.5f ? 1 : 0; }
float ref_F32_exp(float v) { return F32_exp(v); }
float ref_F32_sin(float v) { return F32_sin(v); }
float ref_F32_cos(float v) { return F32_cos(v); }
float ref_F32_tanh(float v) { return F32_tanh(v); }
float ref_F32_sqrt(float v) { return F32_sqrt(v); }
float ref_F32_max(float a, float b) { return F32_max(a, b); }
}
