// Online Hadamard rotation of rows whose length is not a power of two: n = K * m with a K x K Hadamard
// factor and m a power of two (1408 = 176 x 8 for the Qwen1.5-MoE expert intermediate, 14336 = 28 x 512 for
// Mixtral).  This is what the reference applies to the down-projection input when its online rotation is on
// (matmul_hadU_cuda, mxmoe/quant/hadamard_utils.py:96-105, hooked in at mxmoe/quant/rotation.py:403-421):
//
//     y[r, a*m + t] = scale * sum_a' hadK[a, a'] * z[r, a'*m + t]
//
// where z is the row after the natural-order Walsh-Hadamard transform over each group of m contiguous
// elements.  For m == 8 that transform runs in registers while the tile is loaded (kFwht8); for larger m the
// caller runs the power-of-two transform over [rows * K, m] first and this kernel only mixes the K groups.
//
// The mixing is a small dense contraction with a +-1 matrix: per block of 16 rows x 8 values of t it is a
// [128, K] x [K, K] product on mma.sync.m16n8k16 (fp16 in, fp32 accumulate).  It is not one of the grouped-GEMM
// hot loops: at 8192 tokens x top-4 it is 16 GFLOP beside the layer's 567 GFLOP, and it is bounded by reading and
// writing the rows once (2 x 92 MB).
#include "had_kernels.h"

#include <cstdint>

namespace mxb {

namespace {

constexpr int kThreads = 256;   // 8 warps: warp w owns the m16 tile of rows 2w, 2w+1 of the block's 16 rows
constexpr int kRowsPerBlock = 16;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// KP: K rounded up to a multiple of 16 (rows and columns beyond K are zero)
template <int KP, bool kFwht8>
__global__ void __launch_bounds__(kThreads) had_kron_kernel(const __half* __restrict__ in, __half* __restrict__ out,
                                                            const __half* __restrict__ hadK, int rows, int K, int m,
                                                            float scale) {
  constexpr int LD = KP + 8;                         // row pitch of both shared tiles (halfs): keeps ldmatrix conflict-free
  extern __shared__ __align__(16) uint8_t smem[];
  __half* sH = reinterpret_cast<__half*>(smem);      // [KP][LD]   hadK[a][a']
  __half* sZ = sH + KP * LD;                         // [128][LD]  z[(r, t)][a'], later the output staging [16][K * 8]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = K * m;
  const int tblocks = m >> 3;                        // groups of 8 values of t

  for (int i = tid; i < KP * LD; i += kThreads) {
    const int a = i / LD, ap = i - a * LD;
    sH[i] = (a < K && ap < K) ? hadK[a * K + ap] : __float2half(0.f);
  }
  // zero the padding columns of the row tile once (columns K .. KP-1 feed the MMA)
  for (int i = tid; i < 128 * (KP - K); i += kThreads) {
    const int r = i / (KP - K), c = K + i % (KP - K);
    sZ[r * LD + c] = __float2half(0.f);
  }
  __syncthreads();

  const int row_tiles = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
  for (int tile = blockIdx.x; tile < row_tiles * tblocks; tile += gridDim.x) {
    const int row0 = (tile / tblocks) * kRowsPerBlock;
    const int t0   = (tile % tblocks) * 8;
    // ---- load 16 rows x K groups x 8 values; transform over the 8 values if the whole m is here
    for (int i = tid; i < kRowsPerBlock * K; i += kThreads) {
      const int r = i / K, ap = i - r * K;
      float v[8];
      if (row0 + r < rows) {
        const uint4 raw = *reinterpret_cast<const uint4*>(in + (int64_t)(row0 + r) * n + (int64_t)ap * m + t0);
        const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(h2[j]);
          v[2 * j] = f.x; v[2 * j + 1] = f.y;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.f;
      }
      if (kFwht8) {
#pragma unroll
        for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if ((j & h) == 0) {
              const float x = v[j], y = v[j + h];
              v[j] = x + y; v[j + h] = x - y;
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) sZ[(r * 8 + j) * LD + ap] = __float2half(v[j] * scale);
    }
    __syncthreads();
    // ---- C[(r, t), a] = sum_a' Z[(r, t), a'] * hadK[a, a']: warp w computes rows 16w .. 16w+15, all KP columns
    float acc[KP / 8][4];
#pragma unroll
    for (int j = 0; j < KP / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const uint32_t zbase = (uint32_t)__cvta_generic_to_shared(sZ + (16 * warp + (lane & 15)) * LD + (lane >> 4) * 8);
    // B fragments of two n-tiles per ldmatrix.x4: lanes 0-7 rows n0..n0+7 at k0, 8-15 the same rows at k0+8,
    // 16-23 rows n0+8.. at k0, 24-31 at k0+8
    const uint32_t hbase = (uint32_t)__cvta_generic_to_shared(sH + ((lane & 7) + ((lane >> 4) << 3)) * LD + ((lane >> 3) & 1) * 8);
#pragma unroll
    for (int ks = 0; ks < KP / 16; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(a, zbase + ks * 32);
#pragma unroll
      for (int jp = 0; jp < KP / 16; ++jp) {
        uint32_t b[4];
        ldmatrix_x4(b, hbase + (jp * 16 * LD + ks * 16) * 2);
        mma_16816(acc[2 * jp], a, b[0], b[1]);
        mma_16816(acc[2 * jp + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();                                 // every warp has read its rows of sZ: reuse it as output staging
    // ---- stage the results as [r][a * 8 + t] so that the rows leave in 16-byte pieces
    __half* sO = sZ;
    const int g = lane >> 2, tq = lane & 3;          // accumulator rows g and g + 8 of the m16 tile: t = g, r = 2w / 2w + 1
#pragma unroll
    for (int j = 0; j < KP / 8; ++j) {
      const int a0 = 8 * j + 2 * tq;
      if (a0 < K) {
        sO[(2 * warp) * (K * 8) + a0 * 8 + g]     = __float2half(acc[j][0]);
        sO[(2 * warp + 1) * (K * 8) + a0 * 8 + g] = __float2half(acc[j][2]);
      }
      if (a0 + 1 < K) {
        sO[(2 * warp) * (K * 8) + (a0 + 1) * 8 + g]     = __float2half(acc[j][1]);
        sO[(2 * warp + 1) * (K * 8) + (a0 + 1) * 8 + g] = __float2half(acc[j][3]);
      }
    }
    __syncthreads();
    for (int i = tid; i < kRowsPerBlock * K; i += kThreads) {
      const int r = i / K, a = i - r * K;
      if (row0 + r < rows)
        *reinterpret_cast<uint4*>(out + (int64_t)(row0 + r) * n + (int64_t)a * m + t0) =
            *reinterpret_cast<const uint4*>(sO + r * (K * 8) + a * 8);
    }
    __syncthreads();                                 // the staging area becomes the next tile's input
    // the padding columns were overwritten only if K * 8 * 16 reaches them: restore the zeros
    if (KP != K) {
      for (int i = tid; i < 128 * (KP - K); i += kThreads) {
        const int r = i / (KP - K), c = K + i % (KP - K);
        sZ[r * LD + c] = __float2half(0.f);
      }
      __syncthreads();
    }
  }
}

template <int KP>
size_t smem_bytes() { return (size_t)(KP * (KP + 8) + 128 * (KP + 8)) * sizeof(__half); }

template <int KP>
cudaError_t launch(const __half* in, __half* out, const __half* hadK, int rows, int K, int m, float scale, bool fwht8,
                   cudaStream_t stream) {
  static_assert(128 * (KP + 8) >= 16 * KP * 8, "output staging must fit into the row tile");
  const size_t smem = smem_bytes<KP>();
  cudaError_t e;
  auto k1 = had_kron_kernel<KP, true>;
  auto k0 = had_kron_kernel<KP, false>;
  if ((e = cudaFuncSetAttribute(fwht8 ? k1 : k0, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
  int dev = 0, sms = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  const long long tiles = (long long)((rows + kRowsPerBlock - 1) / kRowsPerBlock) * (m >> 3);
  const int per_sm = smem > 100 * 1024 ? 2 : 4;
  const int grid = (int)(tiles < (long long)sms * per_sm ? tiles : (long long)sms * per_sm);
  if (fwht8) k1<<<grid, kThreads, smem, stream>>>(in, out, hadK, rows, K, m, scale);
  else       k0<<<grid, kThreads, smem, stream>>>(in, out, hadK, rows, K, m, scale);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_had_kron(const __half* in, __half* out, const __half* hadK, int rows, int K, int m, float scale,
                            bool fwht8, cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  if (K <= 32)  return launch<32>(in, out, hadK, rows, K, m, scale, fwht8, stream);
  if (K <= 64)  return launch<64>(in, out, hadK, rows, K, m, scale, fwht8, stream);
  if (K <= 176) return launch<176>(in, out, hadK, rows, K, m, scale, fwht8, stream);
  return cudaErrorInvalidValue;
}

}  // namespace mxb
