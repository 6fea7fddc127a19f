/* TEST INFRASTRUCTURE ONLY - plain-C restatement of the integer part of the
 * reference's weight+activation grouped GEMM (w8a8 / w4a4):
 *
 *   acc[m][n] = sum_k qa[m][k] * qb[n][k]            exact int32
 *       (mma.m16n8k32.s8 / m16n8k64.s4 with s32 accumulators,
 *        mxmoe/kernels/src/include/cuda_utils.cuh:350-449, main loop
 *        mxmoe/kernels/src/include/cta_gemm.cuh:423-608)
 *   C[m][n]   = fp16_rn( float(acc) * float( fp16_rn(sa[m] * sb[n]) ) )
 *       (mxmoe/kernels/src/include/mm_tile.cuh:468-496 scale_frag with T=float,
 *        :642-646 __float22half2_rn store)
 *
 * Built by oracle/Makefile (`make port`) into oracle/liboracle_c.so.
 */
#include <stdint.h>
#include <stddef.h>

/* codes are int8 (4-bit codes are passed already sign-extended) */
void oracle_int_gemm(const int8_t* qa, const int8_t* qb, int M, int N, int K, int32_t* acc) {
  for (int m = 0; m < M; ++m) {
    const int8_t* a = qa + (size_t)m * K;
    for (int n = 0; n < N; ++n) {
      const int8_t* b = qb + (size_t)n * K;
      int32_t s = 0;
      for (int k = 0; k < K; ++k) s += (int32_t)a[k] * (int32_t)b[k];
      acc[(size_t)m * N + n] = s;
    }
  }
}

static inline float h2f(uint16_t h) {
  _Float16 x;
  __builtin_memcpy(&x, &h, 2);
  return (float)x;
}
static inline uint16_t f2h(float f) {
  _Float16 x = (_Float16)f; /* round to nearest even */
  uint16_t h;
  __builtin_memcpy(&h, &x, 2);
  return h;
}

/* sa, sb, out: IEEE binary16 bit patterns */
void oracle_wxax_epilogue(const int32_t* acc, const uint16_t* sa, const uint16_t* sb, int M, int N, uint16_t* out) {
  for (int m = 0; m < M; ++m) {
    float fa = h2f(sa[m]);
    for (int n = 0; n < N; ++n) {
      /* product of two binary16 values is exact in binary32, so one rounding to binary16 */
      float s  = h2f(f2h(fa * h2f(sb[n])));
      float v  = (float)acc[(size_t)m * N + n] * s;
      out[(size_t)m * N + n] = f2h(v);
    }
  }
}
