// Activation prologue kernels of the mixed-precision grouped GEMM:
//
//   quant_act        gather rows by expert, optional sign flip + fast Walsh-Hadamard
//                    transform, per-token symmetric quantisation, pack along K
//                    (the role of the reference's `quant_act_kernel`, launched at
//                    mxmoe/kernels/src/ref_bind.cu:531-544; its source is not part
//                    of the reference, so the contract is taken from the call site
//                    and the quantiser from mxmoe/quant/quant.py:40-84)
//   silu_mul_quant   h = silu(gate) * up on the gate_up output, then the same
//                    quantise + pack for the down projection
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
  int tag;          // 0 copy fp16, 1 int8 per token, 2 int4 per token
  int k;            // logical row length
  int64_t q_off;    // write offset of the packed row, in halfs
  int64_t s_off;    // write offset of the scale, in halfs
};

__device__ __forceinline__ RowInfo locate_row(const ActArgs& a, int row) {
  const int e     = row < a.rows_routed ? a.row_expert[row] : a.num_experts;
  const int local = row - a.exp_row_start[e];
  RowInfo r;
  r.tag  = a.exp_qtag[e];
  r.k    = (e == a.num_experts) ? a.k_shared : a.k;
  const int pack = r.tag == 0 ? 1 : (r.tag == 1 ? 2 : 4);
  // without explicit offset tables every row owns one fp16-sized slot of `k` halfs: expert e's
  // packed rows start at slot exp_row_start[e] and are stored back to back at their own pitch
  const int64_t q0 = a.exp_q_off ? (int64_t)a.exp_q_off[e] : (int64_t)a.exp_row_start[e] * a.k;
  const int64_t s0 = a.exp_s_off ? (int64_t)a.exp_s_off[e] : (int64_t)a.exp_row_start[e];
  r.q_off = q0 + (int64_t)local * (r.k / pack);
  r.s_off = s0 + local;
  return r;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// kWarps warps per row, rows_per_block = 8 / kWarps.  kSilu selects the loader.
template <int kWarps, bool kSilu>
__global__ void __launch_bounds__(kBlock) act_quant_kernel(ActArgs a) {
  __shared__ float xch[kWarps > 1 ? kBlock * 8 : 1];   // cross-warp exchange, one chunk at a time
  __shared__ float red[8];

  const int warp       = threadIdx.x >> 5;
  const int lane       = threadIdx.x & 31;
  const int row_in_blk = warp / kWarps;
  const int w          = warp % kWarps;  // warp index within the row
  const int row        = blockIdx.x * (8 / kWarps) + row_in_blk;
  const bool row_ok    = row < a.rows_total;

  RowInfo ri{0, 0, 0, 0};
  if (row_ok) ri = locate_row(a, row);
  const int nchunk = ri.k >> 3;  // 16-byte chunks in the row

  // ------------------------------------------------------------------ load
  float x[kJ][8];
  const __half* src = nullptr;
  const __half* src_up = nullptr;
  if (row_ok) {
    if (kSilu) {
      // gate_up rows: [gate (k) | up (k)]; routed rows first, shared-expert rows after them
      if (row < a.rows_routed) src = a.in + (int64_t)row * 2 * a.k;
      else                     src = a.in_shared + (int64_t)(row - a.rows_routed) * 2 * a.k_shared;
      src_up = src + ri.k;
    } else {
      const int64_t tok = row < a.rows_routed ? a.row_token[row] : (int64_t)(row - a.rows_routed);
      src = a.in + tok * a.k;
    }
  }
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
    const int ci = (w * kJ + j) * 32 + lane;
    if (row_ok && ci < nchunk) {
      const uint4 g = __ldg(reinterpret_cast<const uint4*>(src) + ci);
      const __half2* gh = reinterpret_cast<const __half2*>(&g);
      if (kSilu) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(src_up) + ci);
        const __half2* uh = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 gf = __half22float2(gh[e]);
          // silu evaluated in fp32 and rounded to fp16, product rounded to fp16 (fp16 module semantics)
          const __half s0 = __float2half_rn(gf.x / (1.f + expf(-gf.x)));
          const __half s1 = __float2half_rn(gf.y / (1.f + expf(-gf.y)));
          const __half2 h = __hmul2(__halves2half2(s0, s1), uh[e]);
          const float2 hf = __half22float2(h);
          x[j][2 * e] = hf.x;
          x[j][2 * e + 1] = hf.y;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __half22float2(gh[e]);
          x[j][2 * e] = f.x;
          x[j][2 * e + 1] = f.y;
        }
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) x[j][e] = 0.f;
    }
  }

  // ------------------------------------------------- optional Hadamard rotation
  // y = (x .* signs) H_k / sqrt(k), natural (Sylvester) order: the transform of
  // mxmoe/quant/hadamard_utils.py:62-94.  Element index = chunk * 8 + e with
  // chunk = (w * 8 + j) * 32 + lane, so the index bits are e | lane | j | w.
  if (!kSilu && a.rotate) {
    // chunks per lane that hold data (a power of two; equals kJ whenever a row spans several warps)
    const int jeff = max(1, min(kJ, nchunk / (32 * kWarps)));
    if (a.signs) {
#pragma unroll
      for (int j = 0; j < kJ; ++j) {
        const int ci = (w * kJ + j) * 32 + lane;
        if (row_ok && ci < nchunk) {
          const int2 sg = __ldg(reinterpret_cast<const int2*>(a.signs) + ci);
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
    // bits 3..7: across lanes
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const bool upper = (lane & o) != 0;
#pragma unroll
      for (int j = 0; j < kJ; ++j) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float other = __shfl_xor_sync(0xffffffffu, x[j][e], o);
          x[j][e] = upper ? other - x[j][e] : x[j][e] + other;
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
        const bool upper = (w & s) != 0;
#pragma unroll
        for (int j = 0; j < kJ; ++j) {
          __syncthreads();
#pragma unroll
          for (int e = 0; e < 8; ++e) xch[threadIdx.x * 8 + e] = x[j][e];
          __syncthreads();
          const int partner = (threadIdx.x ^ (s * 32)) * 8;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float other = xch[partner + e];
            x[j][e] = upper ? other - x[j][e] : x[j][e] + other;
          }
        }
      }
    }
    const float norm = 1.0f / sqrtf((float)ri.k);
#pragma unroll
    for (int j = 0; j < kJ; ++j)
#pragma unroll
      for (int e = 0; e < 8; ++e) x[j][e] = __half2float(__float2half_rn(x[j][e] * norm));
  }

  // --------------------------------------------------------- per-token abs max
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
  if (!row_ok) return;

  __half* q_dst = a.q_store + ri.q_off;
  if (ri.tag == 0) {
#pragma unroll
    for (int j = 0; j < kJ; ++j) {
      const int ci = (w * kJ + j) * 32 + lane;
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

  // scale = fp16(amax / qmax); code = rint(clamp(fp16(x / scale), -qmax, qmax))   (quant.py:77-82,
  // evaluated in fp16 like the reference does for fp16 activations; IEEE fp32 division followed
  // by one rounding to fp16 is the correctly rounded fp16 quotient)
  const float qmax   = ri.tag == 1 ? 127.f : 7.f;
  const __half sc_h  = __float2half_rn(__fdiv_rn(amax, qmax));
  const float sc     = __half2float(sc_h);
  if (w == 0 && lane == 0) a.s_store[ri.s_off] = sc_h;

#pragma unroll
  for (int j = 0; j < kJ; ++j) {
    const int ci = (w * kJ + j) * 32 + lane;
    if (ci >= nchunk) continue;
    int code[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float v = 0.f;
      if (sc != 0.f) {
        v = __half2float(__float2half_rn(__fdiv_rn(x[j][e], sc)));
        v = fminf(fmaxf(v, -qmax), qmax);
      }
      code[e] = __float2int_rn(v);
    }
    if (ri.tag == 1) {
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
      reinterpret_cast<uint32_t*>(q_dst)[ci] = w0 | (w1 << 16);
    }
  }
}

template <bool kSilu>
cudaError_t launch(const ActArgs& a, cudaStream_t stream) {
  const int kmax = a.k > a.k_shared ? a.k : a.k_shared;
  if (a.rows_total <= 0) return cudaSuccess;
  if (kmax <= 2048) {
    act_quant_kernel<1, kSilu><<<(a.rows_total + 7) / 8, kBlock, 0, stream>>>(a);
  } else if (kmax <= 4096) {
    act_quant_kernel<2, kSilu><<<(a.rows_total + 3) / 4, kBlock, 0, stream>>>(a);
  } else if (kmax <= 8192) {
    act_quant_kernel<4, kSilu><<<(a.rows_total + 1) / 2, kBlock, 0, stream>>>(a);
  } else {
    act_quant_kernel<8, kSilu><<<a.rows_total, kBlock, 0, stream>>>(a);
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_quant_act(const ActArgs& a, cudaStream_t stream) { return launch<false>(a, stream); }
cudaError_t launch_silu_mul_quant(const ActArgs& a, cudaStream_t stream) { return launch<true>(a, stream); }

}  // namespace mxb
