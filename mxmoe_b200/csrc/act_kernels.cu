// Activation prologue kernels of the mixed-precision grouped GEMM:
//
//   quant_act        gather rows by expert, optional sign flip + fast Walsh-Hadamard
//                    transform, per-token symmetric quantisation, pack along K
//                    (the role of the reference's `quant_act_kernel`, launched at
//                    mxmoe/kernels/src/ref_bind.cu:531-544; its source is not part
//                    of the reference, so the contract is taken from the call site
//                    and the quantiser from mxmoe/quant/quant.py:40-84)
//   quant_tokens     the same rotation + quantisation done ONCE PER TOKEN into
//   + gather_rows    token-major stores (one per activation format in use), then a
//                    pure copy of each routed row into its expert's slot: with
//                    top-k routing this does the arithmetic T times instead of
//                    T*topk times
//   quant_tokens_scatter  both in one pass (top-k <= 8): the token's packed words are
//                    formed once in registers and stored to each of its routed slots
//   silu_mul_quant   h = silu(gate) * up on the gate_up output, then quantise + pack
//                    for the down projection
//                    (`silu_mul_then_quant_kernel`, ref_bind.cu:701-716)
//
// A row is owned by 1, 2, 4 or 8 warps (<= 64 values per thread, kept in
// registers); reductions and the transform run on warp shuffles, with a
// shared-memory exchange only across the warps of one row.
//
// Packed formats (mxmoe/kernels/src/include/quantize.cuh:424-475): uint16 words,
// first k in the most significant field, two's-complement fields.
#include <cuda_fp16.h>
#include <cstdint>

#include "act_kernels.h"

namespace mxb {
namespace {

constexpr int kBlock = 256;  // 8 warps
constexpr int kJ     = 8;    // 16-byte chunks per lane (8 values each)

struct RowInfo {
  int tag;          // 0 copy fp16, 1 int8 per token, 2 int4 per token, 3 int4 per token expanded to bytes
  int k;            // logical row length
  __half* q_dst;    // where the packed row goes
  __half* s_dst;    // where the scale goes (may be null for tag 0)
};

__device__ __forceinline__ RowInfo locate_row(const ActArgs& a, int row) {
  const int e = row < a.rows_routed ? a.row_expert[row] : a.num_experts;
  RowInfo r;
  r.tag = a.exp_qtag[e];
  r.k   = (e == a.num_experts) ? a.k_shared : a.k;
  if (a.rec_stride > 0) {
    // record layout: one fixed-size record per row, whatever its format
    r.q_dst = a.q_store + (int64_t)row * a.rec_stride;
    r.s_dst = a.rec_scale_off >= 0 ? r.q_dst + a.rec_scale_off : (a.s_store ? a.s_store + row : nullptr);
    return r;
  }
  const int local = row - a.exp_row_start[e];
  const int pack  = r.tag == 0 ? 1 : (r.tag == 2 ? 4 : 2);
  // without explicit offset tables every row owns one fp16-sized slot of `k` halfs: expert e's
  // packed rows start at slot exp_row_start[e] and are stored back to back at their own pitch
  const int64_t q0 = a.exp_q_off ? (int64_t)a.exp_q_off[e] : (int64_t)a.exp_row_start[e] * a.k;
  const int64_t s0 = a.exp_s_off ? (int64_t)a.exp_s_off[e] : (int64_t)a.exp_row_start[e];
  r.q_dst = a.q_store + q0 + (int64_t)local * (r.k / pack);
  r.s_dst = a.s_store ? a.s_store + s0 + local : nullptr;
  return r;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// chunk index of register row j of this thread: element index = chunk * 8 + e, bits e | lane | j | w
template <int kWarps>
__device__ __forceinline__ int chunk_of(int w, int j, int lane) { return (w * kJ + j) * 32 + lane; }

__device__ __forceinline__ void unpack8(const uint4& g, float (&x)[8]) {
  const __half2* gh = reinterpret_cast<const __half2*>(&g);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __half22float2(gh[e]);
    x[2 * e] = f.x;
    x[2 * e + 1] = f.y;
  }
}

// y = (x .* signs) H_k / sqrt(k), natural (Sylvester) order: the transform of
// mxmoe/quant/hadamard_utils.py:62-94, result rounded to fp16 values.
template <int kWarps>
__device__ __forceinline__ void rotate_row(float (&x)[kJ][8], const int8_t* signs, int nchunk, int k, int w, int lane,
                                           bool row_ok, float* xch) {
  // chunks per lane that hold data (a power of two; equals kJ whenever a row spans several warps)
  const int jeff = max(1, min(kJ, nchunk / (32 * kWarps)));
  if (signs) {
#pragma unroll
    for (int j = 0; j < kJ; ++j) {
      const int ci = chunk_of<kWarps>(w, j, lane);
      if (row_ok && ci < nchunk) {
        const int2 sg = __ldg(reinterpret_cast<const int2*>(signs) + ci);
        const signed char* sc = reinterpret_cast<const signed char*>(&sg);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[j][e] *= (float)sc[e];
      }
    }
  }
  // bits 0..2: inside a chunk
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
#pragma unroll
    for (int s = 1; s < 8; s <<= 1) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if ((e & s) == 0) {
          const float p = x[j][e], q = x[j][e | s];
          x[j][e] = p + q;
          x[j][e | s] = p - q;
        }
      }
    }
  }
  // bits 3..7: across lanes; upper lane gets (other - mine), lower lane (mine + other): one FMA each
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float sgn = (lane & o) ? -1.f : 1.f;
#pragma unroll
    for (int j = 0; j < kJ; ++j) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float other = __shfl_xor_sync(0xffffffffu, x[j][e], o);
        x[j][e] = fmaf(sgn, x[j][e], other);
      }
    }
  }
  // next bits: across the chunks of one lane
#pragma unroll
  for (int s = 1; s < kJ; s <<= 1) {
    if (s < jeff) {
#pragma unroll
      for (int j = 0; j < kJ; ++j) {
        if ((j & s) == 0) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float p = x[j][e], q = x[j | s][e];
            x[j][e] = p + q;
            x[j | s][e] = p - q;
          }
        }
      }
    }
  }
  // top bits: across the warps of the row, through shared memory
  if (kWarps > 1) {
#pragma unroll
    for (int s = 1; s < kWarps; s <<= 1) {
      const float sgn = (w & s) ? -1.f : 1.f;
#pragma unroll
      for (int j = 0; j < kJ; ++j) {
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 8; ++e) xch[threadIdx.x * 8 + e] = x[j][e];
        __syncthreads();
        const int partner = (threadIdx.x ^ (s * 32)) * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) x[j][e] = fmaf(sgn, x[j][e], xch[partner + e]);
      }
    }
  }
  const float norm = 1.0f / sqrtf((float)k);
#pragma unroll
  for (int j = 0; j < kJ; ++j)
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
      // round to fp16 values two at a time (packed conversion)
      const float2 r = __half22float2(__floats2half2_rn(x[j][e] * norm, x[j][e + 1] * norm));
      x[j][e]     = r.x;
      x[j][e + 1] = r.y;
    }
}

template <int kWarps>
__device__ __forceinline__ float row_amax(const float (&x)[kJ][8], int warp, int row_in_blk, int lane, float* red) {
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < kJ; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(x[j][e]));
  amax = warp_max(amax);
  if (kWarps > 1) {
    __syncthreads();
    if (lane == 0) red[warp] = amax;
    __syncthreads();
    amax = 0.f;
#pragma unroll
    for (int i = 0; i < kWarps; ++i) amax = fmaxf(amax, red[row_in_blk * kWarps + i]);
  }
  return amax;
}

// Quantiser of one row held in registers.  scale = fp16(amax / qmax); code = rint(clamp(fp16(x / scale)))
// (quant.py:77-82 evaluated in fp16, as the reference does for fp16 activations).  The fp32 quotient is
// formed by Markstein's sequence (q0 = x*r, residual by FMA, one correction with the correctly rounded
// reciprocal r), which yields the correctly rounded fp32 quotient; rounding that once to fp16 is the
// correctly rounded fp16 quotient.  An all-zero row gets scale 0 and codes 0.
struct RowQuant {
  float qmax, sc, rcp;
  __half sc_h;
  __device__ __forceinline__ RowQuant(float amax, int tag) {
    qmax = tag == 1 ? 127.f : 7.f;   // tags 2 and 3 are both 4-bit
    sc_h = __float2half_rn(__fdiv_rn(amax, qmax));
    sc   = __half2float(sc_h);
    rcp  = sc != 0.f ? __frcp_rn(sc) : 0.f;
  }
  // correctly rounded fp32 quotient v / sc (Markstein: one FMA residual, one FMA correction)
  __device__ __forceinline__ float quotient(float v) const {
    const float q = v * rcp;
    return fmaf(fmaf(-q, sc, v), rcp, q);
  }
  // Codes of two values: quotient rounded once to fp16 (the reference divides in fp16), clamped, rounded to the
  // nearest-even integer.  Clamp and rounding run on packed halves, and the integer is read off the mantissa of
  // 1536 + q (fp16 has unit spacing in [1024, 2048), so the addition IS the round-to-nearest-even): no
  // float<->half or float->int conversion instruction is issued per value - those share the 16-lane
  // special-function pipe with exp and reciprocal and were what bound the kernels.
  // bit pattern of (1536 + code0, 1536 + code1) as packed halves: the two's-complement code sits in the low
  // mantissa bits (512 is a multiple of 16 and of 256, so `bits & 0xf` / `bits & 0xff` IS the 4- / 8-bit code)
  __device__ __forceinline__ uint32_t bits2(float v0, float v1) const {
    __half2 h = __floats2half2_rn(quotient(v0), quotient(v1));
    const __half2 lim = __float2half2_rn(qmax);
    h = __hmin2(__hmax2(h, __hneg2(lim)), lim);
    h = __hadd2(h, __float2half2_rn(1536.f));
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  __device__ __forceinline__ void code2(float v0, float v1, int& c0, int& c1) const {
    const uint32_t b = bits2(v0, v1);
    c0 = (int)(b & 0x3ffu) - 512;
    c1 = (int)((b >> 16) & 0x3ffu) - 512;
  }
};

// Expanded int4 (tag 3) straight from the packed-half bit patterns of 8 consecutive codes (b01 = codes 0, 1; ...):
// the same bytes store_codes produces for tag 3 - every code as the byte 16*q, high nibbles of the packed row's
// bytes first - with shifts, masks and byte permutes only.
__device__ __forceinline__ void expanded4_words(uint32_t b01, uint32_t b23, uint32_t b45, uint32_t b67, uint32_t& d0,
                                                uint32_t& d4) {
  const uint32_t x01 = (b01 << 4) & 0x00F000F0u, x23 = (b23 << 4) & 0x00F000F0u;   // byte 0: even code, byte 2: odd code
  const uint32_t x45 = (b45 << 4) & 0x00F000F0u, x67 = (b67 << 4) & 0x00F000F0u;
  const uint32_t ylo = __byte_perm(x23, x01, 0x6240);   // c2, c0, c3, c1
  const uint32_t yhi = __byte_perm(x67, x45, 0x6240);   // c6, c4, c7, c5
  d0 = __byte_perm(ylo, yhi, 0x5410);                   // c2, c0, c6, c4
  d4 = __byte_perm(ylo, yhi, 0x7632);                   // c3, c1, c7, c5
}
__device__ __forceinline__ void store_expanded4_words(__half* q_dst, int ci, uint32_t d0, uint32_t d4) {
  uint32_t* d = reinterpret_cast<uint32_t*>(q_dst) + 8 * (ci >> 2) + (ci & 3);
  d[0] = d0;
  d[4] = d4;
}
__device__ __forceinline__ void store_expanded4(__half* q_dst, int ci, uint32_t b01, uint32_t b23, uint32_t b45,
                                                uint32_t b67) {
  uint32_t d0, d4;
  expanded4_words(b01, b23, b45, b67, d0, d4);
  store_expanded4_words(q_dst, ci, d0, d4);
}

// pack 8 consecutive codes of a row and store them as chunk `ci` of the packed row
__device__ __forceinline__ void store_codes(__half* q_dst, int ci, int tag, const int (&code)[8]) {
  if (tag == 1) {
    // uint16 word = code[2i] << 8 | code[2i+1]
    uint2 o;
    o.x = ((uint32_t)(code[1] & 0xff)) | ((uint32_t)(code[0] & 0xff) << 8) | ((uint32_t)(code[3] & 0xff) << 16) |
          ((uint32_t)(code[2] & 0xff) << 24);
    o.y = ((uint32_t)(code[5] & 0xff)) | ((uint32_t)(code[4] & 0xff) << 8) | ((uint32_t)(code[7] & 0xff) << 16) |
          ((uint32_t)(code[6] & 0xff) << 24);
    reinterpret_cast<uint2*>(q_dst)[ci] = o;
  } else {
    // uint16 word = c0 << 12 | c1 << 8 | c2 << 4 | c3
    const uint32_t w0 = ((uint32_t)(code[0] & 0xf) << 12) | ((uint32_t)(code[1] & 0xf) << 8) |
                        ((uint32_t)(code[2] & 0xf) << 4) | (uint32_t)(code[3] & 0xf);
    const uint32_t w1 = ((uint32_t)(code[4] & 0xf) << 12) | ((uint32_t)(code[5] & 0xf) << 8) |
                        ((uint32_t)(code[6] & 0xf) << 4) | (uint32_t)(code[7] & 0xf);
    const uint32_t w  = w0 | (w1 << 16);
    if (tag == 2) {
      reinterpret_cast<uint32_t*>(q_dst)[ci] = w;
    } else {
      // tag 3: the bytes the GEMM's own int4 -> int8 unpacking would produce from the packed row: every
      // 16 packed bytes become 16 bytes of high nibbles then 16 bytes of low nibbles, each nibble moved
      // to the top of its byte (the byte 16*q).  These 4 packed bytes are bytes 4*(ci%4).. of chunk ci/4.
      uint32_t* d = reinterpret_cast<uint32_t*>(q_dst) + 8 * (ci >> 2) + (ci & 3);
      d[0] = w & 0xF0F0F0F0u;
      d[4] = (w << 4) & 0xF0F0F0F0u;
    }
  }
}

// write one row in format `tag` (0 fp16 copy, 1 int8, 2 int4 packed, 3 int4 expanded) to q_dst / s_dst
template <int kWarps>
__device__ __forceinline__ void emit_row(const float (&x)[kJ][8], float amax, int tag, __half* q_dst, __half* s_dst,
                                         int nchunk, int w, int lane) {
  if (tag == 0) {
#pragma unroll
    for (int j = 0; j < kJ; ++j) {
      const int ci = chunk_of<kWarps>(w, j, lane);
      if (ci < nchunk) {
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) oh[e] = __floats2half2_rn(x[j][2 * e], x[j][2 * e + 1]);
        reinterpret_cast<uint4*>(q_dst)[ci] = o;
      }
    }
    return;
  }
  const RowQuant rq(amax, tag);
  if (w == 0 && lane == 0) *s_dst = rq.sc_h;
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
    const int ci = chunk_of<kWarps>(w, j, lane);
    if (ci >= nchunk) continue;
    if (tag == 3) {
      store_expanded4(q_dst, ci, rq.bits2(x[j][0], x[j][1]), rq.bits2(x[j][2], x[j][3]), rq.bits2(x[j][4], x[j][5]),
                      rq.bits2(x[j][6], x[j][7]));
      continue;
    }
    int code[8];
#pragma unroll
    for (int e = 0; e < 8; e += 2) rq.code2(x[j][e], x[j][e + 1], code[e], code[e + 1]);
    store_codes(q_dst, ci, tag, code);
  }
}

// The same row written to several destinations: the packed words of each chunk are formed once and stored to
// every destination d whose bit is set in `dst_mask`.  Lane d of the warp holds destination d: its packed row at
// q_base + my_q and its scale at s_base + my_s (offsets in halfs; no scale if negative); the offsets are fetched
// by shuffle where they are used, so that they cost no registers next to the row.  `dst_mask` is the same in
// every lane.  Bits are those emit_row writes.
constexpr int kMaxDst = 8;
template <int kWarps>
__device__ __forceinline__ void emit_row_multi(const float (&x)[kJ][8], float amax, int tag, __half* q_base, int my_q,
                                               __half* s_base, int my_s, unsigned dst_mask, int nchunk, int w,
                                               int lane) {
  const RowQuant rq(amax, tag == 0 ? 1 : tag);
  if (tag != 0) {
    for (unsigned m = dst_mask; m; m &= m - 1) {
      const int sd = __shfl_sync(0xffffffffu, my_s, __ffs(m) - 1);
      if (w == 0 && lane == 0 && sd >= 0) s_base[sd] = rq.sc_h;
    }
  }
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
    const int ci  = chunk_of<kWarps>(w, j, lane);
    const bool on = ci < nchunk;
    if (chunk_of<kWarps>(w, j, 0) >= nchunk) break;   // no lane of the warp has this chunk
    if (tag == 0) {
      uint4 o;
      __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) oh[e] = __floats2half2_rn(x[j][2 * e], x[j][2 * e + 1]);
      for (unsigned m = dst_mask; m; m &= m - 1) {
        const int qd = __shfl_sync(0xffffffffu, my_q, __ffs(m) - 1);
        if (on) reinterpret_cast<uint4*>(q_base + qd)[ci] = o;
      }
    } else if (tag == 3) {
      uint32_t d0, d4;
      expanded4_words(rq.bits2(x[j][0], x[j][1]), rq.bits2(x[j][2], x[j][3]), rq.bits2(x[j][4], x[j][5]),
                      rq.bits2(x[j][6], x[j][7]), d0, d4);
      for (unsigned m = dst_mask; m; m &= m - 1) {
        const int qd = __shfl_sync(0xffffffffu, my_q, __ffs(m) - 1);
        if (on) store_expanded4_words(q_base + qd, ci, d0, d4);
      }
    } else {
      int code[8];
#pragma unroll
      for (int e = 0; e < 8; e += 2) rq.code2(x[j][e], x[j][e + 1], code[e], code[e + 1]);
      for (unsigned m = dst_mask; m; m &= m - 1) {
        const int qd = __shfl_sync(0xffffffffu, my_q, __ffs(m) - 1);
        if (on) store_codes(q_base + qd, ci, tag, code);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// fused gather + (rotate) + quantise, one pass per routed row (operator-API path, any top-k)
template <int kWarps>
__global__ void __launch_bounds__(kBlock) quant_act_kernel(ActArgs a) {
  __shared__ float xch[kWarps > 1 ? kBlock * 8 : 1];
  __shared__ float red[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_in_blk = warp / kWarps, w = warp % kWarps;
  const int row     = blockIdx.x * (8 / kWarps) + row_in_blk;
  const int live    = a.rows_dev ? min(a.rows_total, __ldg(a.rows_dev)) : a.rows_total;
  if (blockIdx.x * (8 / kWarps) >= live) return;   // the whole block lies beyond the live rows
  const bool row_ok = row < live;

  RowInfo ri{0, 0, nullptr, nullptr};
  if (row_ok) ri = locate_row(a, row);
  const int nchunk = ri.k >> 3;
  const __half* src = nullptr;
  if (row_ok) {
    const int64_t tok = row < a.rows_routed ? a.row_token[row] : (int64_t)(row - a.rows_routed);
    src = a.in + tok * a.k;
  }
  float x[kJ][8];
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
    const int ci = chunk_of<kWarps>(w, j, lane);
    if (row_ok && ci < nchunk) {
      unpack8(__ldg(reinterpret_cast<const uint4*>(src) + ci), x[j]);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) x[j][e] = 0.f;
    }
  }
  if (a.rotate) rotate_row<kWarps>(x, a.signs, nchunk, ri.k, w, lane, row_ok, xch);
  const float amax = row_amax<kWarps>(x, warp, row_in_blk, lane, red);
  if (!row_ok) return;
  emit_row<kWarps>(x, amax, ri.tag, ri.q_dst, ri.s_dst, nchunk, w, lane);
}

// ---------------------------------------------------------------------------------------------
// (rotate) + quantise once per token into token-major stores, one per activation format in use
template <int kWarps>
__global__ void __launch_bounds__(kBlock, 3) quant_tokens_kernel(TokenQuantArgs a) {
  __shared__ float xch[kWarps > 1 ? kBlock * 8 : 1];
  __shared__ float red[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_in_blk = warp / kWarps, w = warp % kWarps;
  const int tok     = blockIdx.x * (8 / kWarps) + row_in_blk;
  const bool row_ok = tok < a.num_tokens;
  const int nchunk  = a.k >> 3;
  float x[kJ][8];
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
    const int ci = chunk_of<kWarps>(w, j, lane);
    if (row_ok && ci < nchunk) {
      unpack8(__ldg(reinterpret_cast<const uint4*>(a.in + (int64_t)tok * a.k) + ci), x[j]);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) x[j][e] = 0.f;
    }
  }
  if (a.rotate) rotate_row<kWarps>(x, a.signs, nchunk, a.k, w, lane, row_ok, xch);
  const float amax = row_amax<kWarps>(x, warp, row_in_blk, lane, red);
  if (!row_ok) return;
  if (a.f16) emit_row<kWarps>(x, amax, 0, a.f16 + (int64_t)tok * a.k, nullptr, nchunk, w, lane);
  if (a.q8) emit_row<kWarps>(x, amax, 1, a.q8 + (int64_t)tok * (a.k / 2), a.s8 + tok, nchunk, w, lane);
  if (a.q4) emit_row<kWarps>(x, amax, 2, a.q4 + (int64_t)tok * (a.k / 4), a.s4 + tok, nchunk, w, lane);
  if (a.q4x) emit_row<kWarps>(x, amax, 3, a.q4x + (int64_t)tok * (a.k / 2), a.s4 + tok, nchunk, w, lane);
}

// quant_tokens with the routed copies written by the same pass: the token's row goes to the expert-sorted slot
// of each of its `topk` routing slots (slot_row[tok * topk + s], tables of `r` as for gather_rows) in that
// expert's format, and to the token-major stores of `a` that are not null.  Same bits as quant_tokens followed
// by gather_rows, without the second pass over the rows.
template <int kWarps>
__global__ void __launch_bounds__(kBlock, 2) quant_tokens_scatter_kernel(TokenQuantArgs a, ActArgs r, const int* slot_row,
                                                                         int topk) {
  __shared__ float xch[kWarps > 1 ? kBlock * 8 : 1];
  __shared__ float red[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_in_blk = warp / kWarps, w = warp % kWarps;
  const int tok     = blockIdx.x * (8 / kWarps) + row_in_blk;
  const bool row_ok = tok < a.num_tokens;
  const int nchunk  = a.k >> 3;
  // destinations first: their loads are in flight during the transform
  // (as 32-bit offsets from the stores: the launcher checks that they fit)
  const bool s_in_record = r.rec_stride > 0 && r.rec_scale_off >= 0;
  __half* s_base         = s_in_record ? r.q_store : r.s_store;
  int my_tag = -1, my_q = 0, my_s = -1;
  if (row_ok && lane < topk) {
    const int row = __ldg(slot_row + (int64_t)tok * topk + lane);
    if (row >= 0 && row < r.rows_routed) {
      const RowInfo ri = locate_row(r, row);
      my_tag = ri.tag;
      my_q   = (int)(ri.q_dst - r.q_store);
      my_s   = ri.s_dst ? (int)(ri.s_dst - s_base) : -1;
    }
  }
  float x[kJ][8];
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
    const int ci = chunk_of<kWarps>(w, j, lane);
    if (row_ok && ci < nchunk) {
      unpack8(__ldg(reinterpret_cast<const uint4*>(a.in + (int64_t)tok * a.k) + ci), x[j]);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) x[j][e] = 0.f;
    }
  }
  if (a.rotate) rotate_row<kWarps>(x, a.signs, nchunk, a.k, w, lane, row_ok, xch);
  const float amax = row_amax<kWarps>(x, warp, row_in_blk, lane, red);
  if (!row_ok) return;   // a warp serves one row: it leaves as a whole
  if (a.f16) emit_row<kWarps>(x, amax, 0, a.f16 + (int64_t)tok * a.k, nullptr, nchunk, w, lane);
  if (a.q8) emit_row<kWarps>(x, amax, 1, a.q8 + (int64_t)tok * (a.k / 2), a.s8 + tok, nchunk, w, lane);
  if (a.q4) emit_row<kWarps>(x, amax, 2, a.q4 + (int64_t)tok * (a.k / 4), a.s4 + tok, nchunk, w, lane);
  if (a.q4x) emit_row<kWarps>(x, amax, 3, a.q4x + (int64_t)tok * (a.k / 2), a.s4 + tok, nchunk, w, lane);
  unsigned by_tag[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) by_tag[t] = __ballot_sync(0xffffffffu, my_tag == t);
#pragma unroll
  for (int t = 0; t < 4; ++t)
    if (by_tag[t]) emit_row_multi<kWarps>(x, amax, t, r.q_store, my_q, s_base, my_s, by_tag[t], nchunk, w, lane);
}

// copy every routed (and shared-expert) row from the token-major store of its expert's format into
// the expert-sorted activation store; one warp per row, 16-byte chunks
__global__ void __launch_bounds__(kBlock) gather_rows_kernel(ActArgs a, TokenQuantArgs t) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  if (row >= a.rows_total) return;
  const RowInfo ri  = locate_row(a, row);
  const int64_t tok = row < a.rows_routed ? a.row_token[row] : (int64_t)(row - a.rows_routed);
  const int pack    = ri.tag == 0 ? 1 : (ri.tag == 2 ? 4 : 2);
  const __half* src = ri.tag == 0 ? (t.f16 ? t.f16 : t.in) : (ri.tag == 1 ? t.q8 : (ri.tag == 2 ? t.q4 : t.q4x));
  const uint4* s = reinterpret_cast<const uint4*>(src + tok * (a.k / pack));
  uint4* d       = reinterpret_cast<uint4*>(ri.q_dst);
  const int n16  = (a.k / pack) >> 3;
  for (int c = lane; c < n16; c += 32) d[c] = __ldg(s + c);
  if (ri.tag != 0 && lane == 0) *ri.s_dst = (ri.tag == 1 ? t.s8 : t.s4)[tok];
}

// ---------------------------------------------------------------------------------------------
// h = silu(gate) * up, then quantise; one pass per routed row.  Values are fp16 after the product,
// so they are kept as half2 (32 registers per thread for 64 values).
// kSilu = false: the rows are h already ([rows, k] fp16, e.g. left by a GEMM epilogue that applied silu * up):
// only the quantiser runs, on the same registers.
template <int kWarps, bool kSilu>
__device__ __forceinline__ void rows_quant_body(const ActArgs& a) {
  __shared__ float red[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_in_blk = warp / kWarps, w = warp % kWarps;
  const int row     = blockIdx.x * (8 / kWarps) + row_in_blk;
  const int live    = a.rows_dev ? min(a.rows_total, __ldg(a.rows_dev)) : a.rows_total;
  if (blockIdx.x * (8 / kWarps) >= live) return;   // the whole block lies beyond the live rows
  const bool row_ok = row < live;
  RowInfo ri{0, 0, nullptr, nullptr};
  if (row_ok) ri = locate_row(a, row);
  const int nchunk = ri.k >> 3;
  const __half* src = nullptr;
  if (row_ok) {
    // gate_up rows: [gate (k) | up (k)]; routed rows first, shared-expert rows in their own buffer
    constexpr int kIn = kSilu ? 2 : 1;
    if (row < a.rows_routed) src = a.in + (int64_t)row * kIn * a.k;
    else                     src = a.in_shared + (int64_t)(row - a.rows_routed) * kIn * a.k_shared;
  }
  __half2 h[kJ][4];
  __half2 m2 = __float2half2_rn(0.f);
  // every load of the row is issued before the first value is used: the kernel waits on memory, not on issue
  // slots, and 24 warps per SM with all their loads in flight beat 40 warps that load chunk by chunk
  uint4 gq[kJ], uq[kJ];
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
    const int ci = chunk_of<kWarps>(w, j, lane);
    if (row_ok && ci < nchunk) {
      gq[j] = __ldg(reinterpret_cast<const uint4*>(src) + ci);
      if (kSilu) uq[j] = __ldg(reinterpret_cast<const uint4*>(src + ri.k) + ci);
    }
  }
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
    const int ci = chunk_of<kWarps>(w, j, lane);
    if (row_ok && ci < nchunk) {
      const uint4 g = gq[j];
      const uint4 u = uq[j];
      const __half2* gh = reinterpret_cast<const __half2*>(&g);
      const __half2* uh = reinterpret_cast<const __half2*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (kSilu) {
          const float2 gf = __half22float2(gh[e]);
          // silu in fp32, rounded to fp16; product rounded to fp16 (fp16 module semantics)
          const float s0 = __fdividef(gf.x, 1.f + __expf(-gf.x));
          const float s1 = __fdividef(gf.y, 1.f + __expf(-gf.y));
          h[j][e] = __hmul2(__floats2half2_rn(s0, s1), uh[e]);
        } else {
          h[j][e] = gh[e];
        }
        m2 = __hmax2(m2, __habs2(h[j][e]));
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) h[j][e] = __float2half2_rn(0.f);
    }
  }
  float amax = warp_max(fmaxf(__low2float(m2), __high2float(m2)));
  if (kWarps > 1) {
    __syncthreads();
    if (lane == 0) red[warp] = amax;
    __syncthreads();
    amax = 0.f;
#pragma unroll
    for (int i = 0; i < kWarps; ++i) amax = fmaxf(amax, red[row_in_blk * kWarps + i]);
  }
  if (!row_ok) return;
  __half* q_dst = ri.q_dst;
  if (ri.tag == 0) {
#pragma unroll
    for (int j = 0; j < kJ; ++j) {
      const int ci = chunk_of<kWarps>(w, j, lane);
      if (ci < nchunk) reinterpret_cast<uint4*>(q_dst)[ci] = *reinterpret_cast<const uint4*>(h[j]);
    }
    return;
  }
  const RowQuant rq(amax, ri.tag);
  if (w == 0 && lane == 0) *ri.s_dst = rq.sc_h;
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
    const int ci = chunk_of<kWarps>(w, j, lane);
    if (ci >= nchunk) continue;
    if (ri.tag == 3) {
      uint32_t b[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h[j][e]);
        b[e] = rq.bits2(f.x, f.y);
      }
      store_expanded4(q_dst, ci, b[0], b[1], b[2], b[3]);
      continue;
    }
    int code[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __half22float2(h[j][e]);
      rq.code2(f.x, f.y, code[2 * e], code[2 * e + 1]);
    }
    store_codes(q_dst, ci, ri.tag, code);
  }
}

template <int kWarps>
__global__ void __launch_bounds__(kBlock, 3) silu_mul_quant_kernel(ActArgs a) { rows_quant_body<kWarps, true>(a); }
template <int kWarps>
__global__ void __launch_bounds__(kBlock, 3) rows_quant_kernel(ActArgs a) { rows_quant_body<kWarps, false>(a); }

#define MXB_DISPATCH_WARPS(kmax, rows, KERNEL, ...)                                                   \
  do {                                                                                                \
    if ((kmax) <= 2048)      KERNEL<1><<<((rows) + 7) / 8, kBlock, 0, stream>>>(__VA_ARGS__);          \
    else if ((kmax) <= 4096) KERNEL<2><<<((rows) + 3) / 4, kBlock, 0, stream>>>(__VA_ARGS__);          \
    else if ((kmax) <= 8192) KERNEL<4><<<((rows) + 1) / 2, kBlock, 0, stream>>>(__VA_ARGS__);          \
    else                     KERNEL<8><<<(rows), kBlock, 0, stream>>>(__VA_ARGS__);                    \
  } while (0)

}  // namespace

cudaError_t launch_quant_act(const ActArgs& a, cudaStream_t stream) {
  if (a.rows_total <= 0) return cudaSuccess;
  const int kmax = a.k > a.k_shared ? a.k : a.k_shared;
  if (!a.rotate && !a.row_token) {
    // rows in place, no rotation: the quantiser alone (the second half of silu_mul_quant)
    MXB_DISPATCH_WARPS(kmax, a.rows_total, rows_quant_kernel, a);
  } else {
    MXB_DISPATCH_WARPS(kmax, a.rows_total, quant_act_kernel, a);
  }
  return cudaGetLastError();
}

cudaError_t launch_silu_mul_quant(const ActArgs& a, cudaStream_t stream) {
  if (a.rows_total <= 0) return cudaSuccess;
  const int kmax = a.k > a.k_shared ? a.k : a.k_shared;
  MXB_DISPATCH_WARPS(kmax, a.rows_total, silu_mul_quant_kernel, a);
  return cudaGetLastError();
}

cudaError_t launch_quant_tokens(const TokenQuantArgs& t, cudaStream_t stream) {
  if (t.num_tokens <= 0) return cudaSuccess;
  MXB_DISPATCH_WARPS(t.k, t.num_tokens, quant_tokens_kernel, t);
  return cudaGetLastError();
}

cudaError_t launch_quant_tokens_scatter(const TokenQuantArgs& t, const ActArgs& r, const int* slot_row, int topk,
                                        cudaStream_t stream) {
  if (t.num_tokens <= 0) return cudaSuccess;
  if (topk < 1 || topk > kMaxDst) return cudaErrorInvalidValue;
  MXB_DISPATCH_WARPS(t.k, t.num_tokens, quant_tokens_scatter_kernel, t, r, slot_row, topk);
  return cudaGetLastError();
}

cudaError_t launch_gather_rows(const ActArgs& a, const TokenQuantArgs& t, cudaStream_t stream) {
  if (a.rows_total <= 0) return cudaSuccess;
  gather_rows_kernel<<<(a.rows_total + 7) / 8, kBlock, 0, stream>>>(a, t);
  return cudaGetLastError();
}

}  // namespace mxb
