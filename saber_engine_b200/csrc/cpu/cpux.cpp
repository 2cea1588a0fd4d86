// Host twin of the W4A8 integer linear and of the routed-expert chain
// (gate_up GEMM -> SiLU(gate) * up -> per-token int8 quant -> down GEMM), byte-equal to the device:
// the accumulation is exact int32 and every float step is a single rounding in a fixed order, so
// the AVX2 path must match the scalar law bit for bit (the tests keep a control that must FAIL).
//
// Parity: crates/saber-cpux/src/lib.rs:1-27 (AVX-512 expert chain, byte-equal to the card),
// :252 gemm, :414 expert_chain.
#include <immintrin.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

namespace {

inline int8_t nib(const uint8_t* w, size_t k) {     // plain layout: low nibble = even element
  const uint8_t b = w[k >> 1];
  const int v = (k & 1) ? (b >> 4) : (b & 15);
  return static_cast<int8_t>(v >= 8 ? v - 16 : v);
}

int32_t dot_scalar(const int8_t* a, const uint8_t* w, int K) {
  int32_t acc = 0;
  for (int k = 0; k < K; ++k) acc += int32_t(a[k]) * int32_t(nib(w, k));
  return acc;
}

#if defined(__AVX2__)
int32_t dot_avx2(const int8_t* a, const uint8_t* w, int K) {
  __m256i acc = _mm256_setzero_si256();
  const __m128i m4 = _mm_set1_epi8(0x0F);
  int k = 0;
  for (; k + 32 <= K; k += 32) {
    const __m128i p = _mm_loadu_si128(reinterpret_cast<const __m128i*>(w + (k >> 1)));   // 32 nibbles
    const __m128i lo = _mm_and_si128(p, m4);                       // even elements
    const __m128i hi = _mm_and_si128(_mm_srli_epi16(p, 4), m4);    // odd elements
    // interleave back to element order, then sign-extend the 4-bit values: (x ^ 8) - 8
    const __m128i e0 = _mm_unpacklo_epi8(lo, hi), e1 = _mm_unpackhi_epi8(lo, hi);
    __m256i wv = _mm256_set_m128i(e1, e0);
    const __m256i eight = _mm256_set1_epi8(8);
    wv = _mm256_sub_epi8(_mm256_xor_si256(wv, eight), eight);
    const __m256i av = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(a + k));
    // widen to 16 bit and multiply-add pairs into 32 bit: exact
    const __m256i a_lo = _mm256_cvtepi8_epi16(_mm256_castsi256_si128(av));
    const __m256i a_hi = _mm256_cvtepi8_epi16(_mm256_extracti128_si256(av, 1));
    const __m256i w_lo = _mm256_cvtepi8_epi16(_mm256_castsi256_si128(wv));
    const __m256i w_hi = _mm256_cvtepi8_epi16(_mm256_extracti128_si256(wv, 1));
    acc = _mm256_add_epi32(acc, _mm256_madd_epi16(a_lo, w_lo));
    acc = _mm256_add_epi32(acc, _mm256_madd_epi16(a_hi, w_hi));
  }
  __m128i s = _mm_add_epi32(_mm256_castsi256_si128(acc), _mm256_extracti128_si256(acc, 1));
  s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x4E));
  s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0xB1));
  int32_t r = _mm_cvtsi128_si32(s);
  for (; k < K; ++k) r += int32_t(a[k]) * int32_t(nib(w, k));
  return r;
}
#endif

inline float bf16_round(float x) {                    // round to nearest even, as the device does
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7F800000u) == 0x7F800000u) return x;
  u += 0x7FFFu + ((u >> 16) & 1u);
  u &= 0xFFFF0000u;
  memcpy(&x, &u, 4);
  return x;
}

}  // namespace

extern "C" {

int saber_cpux_has_avx2() {
#if defined(__AVX2__)
  return __builtin_cpu_supports("avx2") ? 1 : 0;
#else
  return 0;
#endif
}

// out[m, n] = bf16(acc * (a_scale[m] * w_scale[n])) as float. w: [N, K/2] nibbles, row-major.
void saber_cpux_gemm_w4a8(const int8_t* a, const float* a_scale, const uint8_t* w, const float* w_scale,
                          float* out, int M, int N, int K, int use_simd) {
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      int32_t acc;
#if defined(__AVX2__)
      acc = (use_simd && saber_cpux_has_avx2()) ? dot_avx2(a + size_t(m) * K, w + size_t(n) * (K / 2), K)
                                                 : dot_scalar(a + size_t(m) * K, w + size_t(n) * (K / 2), K);
#else
      acc = dot_scalar(a + size_t(m) * K, w + size_t(n) * (K / 2), K);
#endif
      out[size_t(m) * N + n] = bf16_round(float(acc) * (a_scale[m] * w_scale[n]));
    }
}

// Per-token symmetric int8: scale = amax / 127, q = clamp(rint(x * (127 / amax))).
void saber_cpux_quant_rows(const float* x, int8_t* q, float* scale, int M, int K) {
  for (int m = 0; m < M; ++m) {
    float amax = 0.f;
    for (int k = 0; k < K; ++k) amax = fmaxf(amax, fabsf(x[size_t(m) * K + k]));
    const float inv = amax > 0.f ? 127.f / amax : 0.f;
    scale[m] = amax / 127.f;
    for (int k = 0; k < K; ++k) {
      int v = int(nearbyintf(x[size_t(m) * K + k] * inv));
      q[size_t(m) * K + k] = int8_t(v > 127 ? 127 : (v < -127 ? -127 : v));
    }
  }
}

// One routed expert: x [M, H] (bf16-rounded floats) -> out [M, H].
void saber_cpux_expert_chain(const float* x, const uint8_t* w_gate_up, const float* s_gate_up,
                             const uint8_t* w_down, const float* s_down, float* out, int M, int H, int I,
                             int use_simd) {
  std::vector<int8_t> q(size_t(M) * (H > I ? H : I));
  std::vector<float> sc(M), gu(size_t(M) * 2 * I), hmid(size_t(M) * I);
  saber_cpux_quant_rows(x, q.data(), sc.data(), M, H);
  saber_cpux_gemm_w4a8(q.data(), sc.data(), w_gate_up, s_gate_up, gu.data(), M, 2 * I, H, use_simd);
  for (int m = 0; m < M; ++m)
    for (int i = 0; i < I; ++i) {
      const float g = gu[size_t(m) * 2 * I + i], u = gu[size_t(m) * 2 * I + I + i];
      hmid[size_t(m) * I + i] = bf16_round(g / (1.f + expf(-g)) * u);
    }
  saber_cpux_quant_rows(hmid.data(), q.data(), sc.data(), M, I);
  saber_cpux_gemm_w4a8(q.data(), sc.data(), w_down, s_down, out, M, H, I, use_simd);
}

}  // extern "C"
