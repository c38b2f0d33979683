// Builds the reference's own host-side functions for this path into a shared library (oracle/_ref/libref_shim.so) so
// the tests can pin the CPU oracle against them.  Nothing of the reference is copied: its headers are included from
// where the reference tree lies at build time (-I <reference>/altar1-4xgx10-switchless/engine).  TEST INFRASTRUCTURE.
//   route_ref            engine/experts/tests/testdata.h:339-355   (168 experts, top-8, x2.5)
//   route_sigmoid        engine/experts/formats.cuh:142-163
//   i4_value_bits        engine/experts/formats.cuh:117-119
//   pack_fp8/read_fp8    engine/experts/layout.h:108-119, 162-165
//   pack_int4/read_i4    engine/experts/layout.h:78-95, 133-149
//   pack_bf16            engine/experts/layout.h:96-107
#include "experts/tests/testdata.h"

extern "C" {
int ref_kE() { return gx::kE; }
int ref_kTopK() { return gx::kTopK; }
void ref_route(const float* l, const float* bias, int M, int* idx, float* w) { gx::route_ref(l, bias, M, idx, w); }
float ref_route_sigmoid(float l) { return gx::route_sigmoid(l); }
uint16_t ref_i4_value_bits(int u, int uz, uint16_t s) { return gx::i4_value_bits(u, uz, s); }
float ref_e4m3_to_f(uint8_t b) { return gx::e4m3_to_f(b); }
uint16_t ref_f_to_bf16_bits(float f) { return gx::f_to_bf16_bits(f); }
void ref_pack_fp8(const uint8_t* w, int N, int K, uint8_t* out) { gx::pack_fp8(w, N, K, out); }
float ref_read_fp8(const uint8_t* m, int K, int n, int k) { return gx::read_fp8(m, K, n, k); }
void ref_pack_int4(const uint8_t* wp, const uint16_t* s, const uint32_t* zp, int N, int K, uint8_t* out) {
  gx::pack_int4(wp, s, zp, N, K, out);
}
uint16_t ref_read_i4(const uint8_t* m, int K, int n, int k) { return gx::read_i4(m, K, n, k); }
void ref_pack_bf16(const uint16_t* w, int N, int K, uint8_t* out) { gx::pack_bf16(w, N, K, out); }
// the reference's FP8 weight value, e4m3 * s[n/128][k/128] (testdata.h:120-125)
float ref_fp8_value(const uint8_t* w, const float* s, int K, int n, int k) {
  return gx::e4m3_to_f(w[(size_t)n * K + k]) * s[(n / 128) * (K / 128) + k / 128];
}
}
