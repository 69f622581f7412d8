/* Thin exports of the reference's OWN scalar primitives, compiled from the headers
 * where they lie in the reference checkout (never copied into this repository).
 * TEST INFRASTRUCTURE ONLY: used to check that the oracle's scalar rules (wrapping
 * add, NaN-dropping max, exact f16 widening) are the reference's.
 *
 * Built by oracle/build.py into oracle/_ref/libref_scalar.so when the reference
 * checkout is present; its rts/c directory is given with -I on the compiler command
 * line, so the three includes below resolve to the reference's files.
 */
#include <math.h>
#include <stdbool.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#define SCALAR_FUN_ATTR static inline
#include "scalar.h"
#include "half.h"
#include "scalar_f16.h"

uint32_t ref_add32(uint32_t a, uint32_t b) { return add32(a, b); }
float ref_fadd32(float a, float b) { return fadd32(a, b); }
float ref_fmul32(float a, float b) { return fmul32(a, b); }
float ref_fmax32(float a, float b) { return fmax32(a, b); }
float ref_halfbits2float(uint16_t h) { return halfbits2float(h); }
uint16_t ref_float2halfbits(float f) { return float2halfbits(f); }
bool ref_ult32(uint32_t a, uint32_t b) { return ult32(a, b); }
uint32_t ref_and32(uint32_t a, uint32_t b) { return a & b; }
int64_t ref_sext_i32_i64(int32_t x) { return sext_i32_i64(x); }
