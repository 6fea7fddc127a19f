// Device code shared by the single-CTA and the CTA-pair grouped GEMM kernels: bounded waits,
// tile lookup, the fused epilogue and the 4-bit converters.
#pragma once
#include "gg_types.h"
#include "ptx.cuh"

namespace mxb {
namespace ggc {

using namespace ptx;

constexpr uint64_t kTimeoutNs = 1000000000ull;

// `timeout_ns`: how long the wait may last (the launch's limit, GGStatus::timeout_ms, default 1 s)
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_flag, int backoff_ns = 0,
                                         uint64_t timeout_ns = kTimeoutNs) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it       = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (backoff_ns) __nanosleep(backoff_ns);
    if ((++it & 63u) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > timeout_ns) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// The same for a whole warp: lane 0 polls (every polling thread is one more access to the mbarrier in shared
// memory), the outcome is broadcast.  __shfl_sync orders the lanes' later shared-memory reads after lane 0's
// observation of the barrier.
__device__ __forceinline__ bool warp_wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_flag, int lane,
                                              uint64_t timeout_ns = kTimeoutNs) {
  int ok = 1;
  if (lane == 0) ok = wait_bar(bar, parity, abort_flag, 0, timeout_ns) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// per-problem scheduling tables kept in shared memory
struct Sched {
  int total_tiles;
  int pad[3];
  int tile_end[kMaxProblems];   // inclusive prefix sum of tiles
  int m_eff[kMaxProblems];      // rows of each problem
  int row0[kMaxProblems];       // row shift of each problem
  int meta[kMaxProblems];       // n_tiles << 16 | nkb << 4 | scheme   (nkb < 4096)
  int c_shift[kMaxProblems];    // first row of C minus first row of A (0 unless the problem redirects C)
};

struct Tile {
  int p, m_tile, n_tile, scheme, nkb;
  int odd;   // stages of two K blocks: the last stage of the tile holds one
};

// Fill the tables (all threads of the CTA; contains two __syncthreads).  `rows_per_tile` x `cols_per_tile`
// is the tile of C: 128 x 256 for the single-CTA kernel, 256 x 256 for the CTA pair, 176 x 128 for the
// kernel with swapped operands.
// problems of the kernels that cannot redirect C have no c_row0_dev
__device__ __forceinline__ int c_shift_of(const GGProblemDev&, int) { return 0; }
__device__ __forceinline__ int c_shift_of(const GGSwapProblemDev& pr, int r0) {
  return pr.c_row0_dev ? *pr.c_row0_dev - r0 : 0;
}

// `packed_rows_per_tile` (> 0) replaces rows_per_tile for problems with packed 4-bit activations
// `two_kblocks`: a pipeline stage holds TWO K blocks of a problem whose weights are 4-bit (the 32-token geometry
// of the kernel with swapped operands); nkb then counts stages and bit 31 of meta says that the last one holds one
template <typename Problem>
__device__ __forceinline__ void build_sched(Sched* sc, const Problem* problems, int count, int rows_per_tile,
                                            int cols_per_tile = kBN, int packed_rows_per_tile = 0, bool two_kblocks = false) {
  const int tid = threadIdx.x, lane = tid & 31;
  for (int p = tid; p < count; p += blockDim.x) {
    const Problem& pr = problems[p];
    int m = pr.M;
    if (pr.m_dev) m = min(max(*pr.m_dev, 0), pr.M);
    const int r0     = pr.row0_dev ? *pr.row0_dev : pr.row0;
    const int nt     = (pr.N + cols_per_tile - 1) / cols_per_tile;
    const int kelems = (pr.scheme == SCH_FP16 || pr.scheme == SCH_W4A16G128) ? 64 : 128;
    int nkb          = (pr.K + kelems - 1) / kelems;
    unsigned odd     = 0;
    if (two_kblocks && (pr.scheme == SCH_W4A4_XA || pr.scheme == SCH_W4A16G128)) {
      odd = (unsigned)(nkb & 1);
      nkb = (nkb + 1) >> 1;
    }
    const int rpt   = (packed_rows_per_tile > 0 && pr.scheme == SCH_W4A4) ? packed_rows_per_tile : rows_per_tile;
    sc->tile_end[p] = ((m + rpt - 1) / rpt) * nt;
    sc->m_eff[p]    = m;
    sc->row0[p]     = r0;
    sc->meta[p]     = (int)((odd << 31) | ((unsigned)nt << 16) | ((unsigned)nkb << 4) | (unsigned)pr.scheme);
    sc->c_shift[p]  = c_shift_of(pr, r0);
  }
  __syncthreads();
  if (tid < 32) {
    int carry = 0;
    for (int base = 0; base < count; base += 32) {
      const int p = base + lane;
      int v       = (p < count) ? sc->tile_end[p] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
      }
      v += carry;
      if (p < count) sc->tile_end[p] = v;
      carry = __shfl_sync(0xffffffffu, v, 31);
    }
    if (lane == 0) sc->total_tiles = carry;
  }
  __syncthreads();
}

__device__ __forceinline__ Tile find_tile(const Sched* c, int count, int t) {
  int lo = 0, hi = count - 1;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (t < c->tile_end[mid]) hi = mid; else lo = mid + 1;
  }
  const int start = lo ? c->tile_end[lo - 1] : 0;
  const int meta  = c->meta[lo];
  const int nt    = (meta >> 16) & 0x7FFF;
  const int idx   = t - start;
  Tile r;
  r.p      = lo;
  r.m_tile = idx / nt;
  r.n_tile = idx - r.m_tile * nt;
  r.scheme = meta & 15;
  r.nkb    = (meta >> 4) & 0xFFF;
  r.odd    = (int)((unsigned)meta >> 31);
  return r;
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// 4-bit code pair (bits [0,4) of each 16-bit half) -> half2, exact (1024 + q) - 1024,
// then one fp16 FMA with (scale, zero): the arithmetic of quantize.cuh:79-93, :189-190.
__device__ __forceinline__ uint32_t dequant_pair(uint32_t w, int nib, __half2 s2, __half2 z2) {
  uint32_t h = ((w >> (4 * nib)) & 0x000f000fu) | 0x64006400u;
  __half2 q  = __hsub2(*reinterpret_cast<__half2*>(&h), __half2half2(__ushort_as_half((unsigned short)0x6400)));
  __half2 r  = __hfma2(q, s2, z2);
  return *reinterpret_cast<uint32_t*>(&r);
}

// ---------------------------------------------------------------------------------- converters
// w4a4: `rows` packed rows of 64 bytes (128 two's-complement nibbles) at `src` -> rows of 128 int8
// bytes at `dst` in the 128-byte-swizzled operand layout.  Code q becomes the byte 16*q: both
// operands carry the factor, the accumulator is 256x the true one and is shifted back in the
// epilogue.  `ct` = thread index in the converter group of kCvtThreads threads.
template <int kCvtThreads>
__device__ __forceinline__ void convert_w4a4(uint32_t src, uint32_t dst, int rows, int ct) {
  const int iters = rows * 4 / kCvtThreads;
#pragma unroll 4
  for (int i = 0; i < iters; ++i) {
    const int g   = i * kCvtThreads + ct;
    const int row = g >> 2;
    const int c   = g & 3;
    const uint4 w = lds128(src + row * 64 + c * 16);
    uint4 hi, lo;
    hi.x = w.x & 0xF0F0F0F0u; lo.x = (w.x << 4) & 0xF0F0F0F0u;
    hi.y = w.y & 0xF0F0F0F0u; lo.y = (w.y << 4) & 0xF0F0F0F0u;
    hi.z = w.z & 0xF0F0F0F0u; lo.z = (w.z << 4) & 0xF0F0F0F0u;
    hi.w = w.w & 0xF0F0F0F0u; lo.w = (w.w << 4) & 0xF0F0F0F0u;
    const uint32_t drow = dst + row * 128;
    const int sw        = row & 7;
    sts128(drow + (((2 * c) ^ sw) << 4), hi);
    sts128(drow + (((2 * c + 1) ^ sw) << 4), lo);
  }
}

// w4a16 group-128: which part of the packed weight tile a converter thread owns.  A packed row holds
// 8 interleaved n-rows x 64 k as 8 chunks of 16 bytes; chunk 2*kb16 + fh carries, for the 16-k block
// kb16, the rows n_lo = 32*(prow/8) + 16*fh + prow%8 (nibbles 0,1) and n_lo + 8 (nibbles 2,3).
template <int kPackedRows, int kCvtThreads>   // packed rows: 64 = a 256-row B tile, 32 = one CTA's 128-row half
struct W4A16Lane {
  static constexpr int kGroups = kCvtThreads / (2 * kPackedRows);   // thread groups that split the four 16-k blocks
  static constexpr int kIters  = 4 / kGroups;
  static_assert(kGroups >= 1 && kGroups <= 4 && kIters * kGroups == 4, "unsupported converter geometry");
  int prow, fh, r, n_lo, kb0;
  __device__ __forceinline__ explicit W4A16Lane(int ct) {
    const int c2 = ct % (2 * kPackedRows);
    prow = c2 >> 1;
    fh   = c2 & 1;
    kb0  = (ct / (2 * kPackedRows)) * kIters;
    r    = prow & 7;
    n_lo = 32 * (prow >> 3) + 16 * fh + r;
  }
  // 16-k block handled in iteration i (rotated per row so that neighbouring threads hit different banks)
  __device__ __forceinline__ int kb16(int i) const { return kb0 + ((prow + i) % kIters); }
};

template <int kPackedRows, int kCvtThreads>
__device__ __forceinline__ void convert_w4a16(const W4A16Lane<kPackedRows, kCvtThreads>& ln, uint32_t raw_b,
                                              uint32_t op_b, __half2 sz_lo, __half2 sz_hi) {
  const uint32_t src = raw_b + ln.prow * 128;
  const uint32_t dlo = op_b + ln.n_lo * 128;
  const uint32_t dhi = dlo + 8 * 128;
  const __half2 s_lo = __half2half2(__low2half(sz_lo)), z_lo = __half2half2(__high2half(sz_lo));
  const __half2 s_hi = __half2half2(__low2half(sz_hi)), z_hi = __half2half2(__high2half(sz_hi));
#pragma unroll
  for (int i = 0; i < W4A16Lane<kPackedRows, kCvtThreads>::kIters; ++i) {
    const int kb16 = ln.kb16(i);
    const uint4 w  = lds128(src + (2 * kb16 + ln.fh) * 16);
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      const int c = cc ^ ln.fh;   // odd threads write the other k-half first (bank spread)
      const uint32_t phys = (uint32_t)(((2 * kb16 + c) ^ ln.r) << 4);
      uint4 o;
      // nibble 2*fl + c of every word: fl = 0 -> row n_lo, fl = 1 -> row n_hi
      o.x = dequant_pair(w.x, c, s_lo, z_lo); o.y = dequant_pair(w.y, c, s_lo, z_lo);
      o.z = dequant_pair(w.z, c, s_lo, z_lo); o.w = dequant_pair(w.w, c, s_lo, z_lo);
      sts128(dlo + phys, o);
      o.x = dequant_pair(w.x, 2 + c, s_hi, z_hi); o.y = dequant_pair(w.y, 2 + c, s_hi, z_hi);
      o.z = dequant_pair(w.z, 2 + c, s_hi, z_hi); o.w = dequant_pair(w.w, 2 + c, s_hi, z_hi);
      sts128(dhi + phys, o);
    }
  }
}

// ---------------------------------------------------------------------------------- epilogue
// One warp handles 32 rows (TMEM lanes) x 256 columns of a tile.
struct EpiCtx {
  int N, ldc, out_mode, acc_shift, n_col0;
  bool valid, is_int;
  int64_t grow;   // row inside the buffers (C, scale_a)
  __half sa;
};

// Everything that does not depend on the accumulator: fetched before waiting for it.  `row` is the
// row inside the problem this thread owns; `sbw` is this warp's 256-entry staging area for the
// per-channel scales of the tile.
__device__ __forceinline__ EpiCtx epi_prefetch(const GGProblemDev* pr, const Sched* sc, const Tile& ti, int row,
                                               int lane, __half* sbw) {
  EpiCtx c;
  c.N         = pr->N;
  c.ldc       = pr->ldc;
  c.out_mode  = pr->out_mode;
  c.n_col0    = ti.n_tile * kBN;
  c.valid     = row < sc->m_eff[ti.p];
  c.grow      = (int64_t)sc->row0[ti.p] + row;
  c.is_int    = (ti.scheme != SCH_FP16 && ti.scheme != SCH_W4A16G128);
  c.acc_shift = (ti.scheme == SCH_W4A4 || ti.scheme == SCH_W4A4_XA) ? 8 : 0;   // 4-bit codes ride in the high nibble of each byte
  c.sa        = __float2half(0.f);
  if (c.is_int && c.out_mode == OUT_FP16) {
    const int n = c.n_col0 + lane * 8;
    uint4 sv    = make_uint4(0, 0, 0, 0);
    if (n < c.N) sv = __ldg(reinterpret_cast<const uint4*>(pr->scale_b + n));
    if (c.valid) c.sa = pr->scale_a[c.grow * pr->sa_stride];
    __syncwarp();
    *reinterpret_cast<uint4*>(sbw + lane * 8) = sv;
    __syncwarp();
  }
  return c;
}

// Convert and store 32 accumulator columns (one tcgen05.ld chunk) of this thread's row.
__device__ __forceinline__ void epi_store_chunk(const EpiCtx& c, const GGProblemDev* pr, const uint32_t (&v)[32], int ch,
                                                const __half* sbw) {
  const int n0 = c.n_col0 + ch * 32;
  if (!c.valid || n0 >= c.N) return;
  if (c.out_mode == OUT_ACC) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(pr->C) + c.grow * c.ldc + n0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (n0 + j * 4 < c.N) {
        uint4 o;
        if (c.is_int) {
          o.x = (uint32_t)((int)v[4 * j + 0] >> c.acc_shift);
          o.y = (uint32_t)((int)v[4 * j + 1] >> c.acc_shift);
          o.z = (uint32_t)((int)v[4 * j + 2] >> c.acc_shift);
          o.w = (uint32_t)((int)v[4 * j + 3] >> c.acc_shift);
        } else {
          o = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
        *reinterpret_cast<uint4*>(dst + j * 4) = o;
      }
    }
    return;
  }
  __half* dst        = reinterpret_cast<__half*>(pr->C) + c.grow * c.ldc + n0;
  const __half2 sa2  = __half2half2(c.sa);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (n0 + j * 8 < c.N) {
      uint32_t o[4];
      if (c.is_int) {
        // C = fp16_rn( float(acc) * float( fp16_rn(sa * sb) ) )   (mm_tile.cuh:490-493)
        const uint4 sbv   = *reinterpret_cast<const uint4*>(sbw + ch * 32 + j * 8);
        const __half2* s2 = reinterpret_cast<const __half2*>(&sbv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 p = __half22float2(__hmul2(sa2, s2[e]));     // two fp16-rounded scale products
          const float f0 = (float)((int)v[8 * j + 2 * e] >> c.acc_shift) * p.x;
          const float f1 = (float)((int)v[8 * j + 2 * e + 1] >> c.acc_shift) * p.y;
          __half2 h      = __floats2half2_rn(f0, f1);
          o[e]           = *reinterpret_cast<uint32_t*>(&h);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          __half2 h = __floats2half2_rn(__uint_as_float(v[8 * j + 2 * e]), __uint_as_float(v[8 * j + 2 * e + 1]));
          o[e]      = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      *reinterpret_cast<uint4*>(dst + j * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// Drain 256 accumulator columns of this warp's 32 TMEM lanes (`taddr`: lane quarter and column base
// already applied) and store the rows.  Two 32-column TMEM loads are in flight per wait.
__device__ __forceinline__ void epi_store(const EpiCtx& c, const GGProblemDev* pr, uint32_t taddr, const __half* sbw) {
#pragma unroll 1
  for (int ch = 0; ch < kBN / 32; ch += 2) {
    uint32_t v0[32], v1[32];
    tmem_ld_32x32(taddr + ch * 32, v0);
    tmem_ld_32x32(taddr + ch * 32 + 32, v1);
    tmem_ld_wait();
    epi_store_chunk(c, pr, v0, ch, sbw);
    epi_store_chunk(c, pr, v1, ch + 1, sbw);
  }
}

// fp16 conversion of 32 accumulator columns of this thread's row into 4 x 16 bytes
__device__ __forceinline__ void epi_convert_chunk(const EpiCtx& c, const uint32_t (&v)[32], int ch, const __half* sbw,
                                                  uint4 (&out)[4]) {
  const __half2 sa2 = __half2half2(c.sa);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t o[4];
    if (c.is_int) {
      const uint4 sbv   = *reinterpret_cast<const uint4*>(sbw + ch * 32 + j * 8);
      const __half2* s2 = reinterpret_cast<const __half2*>(&sbv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 p = __half22float2(__hmul2(sa2, s2[e]));
        const float f0 = (float)((int)v[8 * j + 2 * e] >> c.acc_shift) * p.x;
        const float f1 = (float)((int)v[8 * j + 2 * e + 1] >> c.acc_shift) * p.y;
        __half2 h      = __floats2half2_rn(f0, f1);
        o[e]           = *reinterpret_cast<uint32_t*>(&h);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        __half2 h = __floats2half2_rn(__uint_as_float(v[8 * j + 2 * e]), __uint_as_float(v[8 * j + 2 * e + 1]));
        o[e]      = *reinterpret_cast<uint32_t*>(&h);
      }
    }
    out[j] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// Same result as epi_store for fp16 output, but rows are transposed through a 4 KiB per-warp
// shared-memory buffer (`stg`, 32 rows x 128 bytes, 16-byte chunks XOR-swizzled by row) so that one
// store instruction writes four full 128-byte lines instead of 16 bytes of 32 different rows.
// `m_rows`: rows of the problem; `row_base`: problem row of this warp's lane 0.
__device__ __forceinline__ void epi_store_staged(const EpiCtx& c, const GGProblemDev* pr, uint32_t taddr,
                                                 const __half* sbw, uint32_t stg, int lane, int row_base, int m_rows) {
  if (c.out_mode != OUT_FP16) {          // raw accumulators keep the direct path
    epi_store(c, pr, taddr, sbw);
    return;
  }
  const int64_t grow0 = c.grow - lane;   // buffer row of lane 0
  __half* cbase = reinterpret_cast<__half*>(pr->C);
#pragma unroll 1
  for (int ch = 0; ch < kBN / 32; ch += 2) {
    uint32_t v0[32], v1[32];
    tmem_ld_32x32(taddr + ch * 32, v0);
    tmem_ld_32x32(taddr + ch * 32 + 32, v1);
    tmem_ld_wait();
    uint4 o[4];
    __syncwarp();                        // the previous round's reads of the buffer are done
    epi_convert_chunk(c, v0, ch, sbw, o);
#pragma unroll
    for (int j = 0; j < 4; ++j) sts128(stg + lane * 128 + ((j ^ (lane & 7)) << 4), o[j]);
    epi_convert_chunk(c, v1, ch + 1, sbw, o);
#pragma unroll
    for (int j = 0; j < 4; ++j) sts128(stg + lane * 128 + (((4 + j) ^ (lane & 7)) << 4), o[j]);
    __syncwarp();
    // 8 rounds: lanes 0-7 -> row 4i, lanes 8-15 -> row 4i+1, ...; lane%8 = 16-byte chunk of the 128-byte row
    const int n0 = c.n_col0 + ch * 32 + (lane & 7) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r   = i * 4 + (lane >> 3);
      const uint4 w = lds128(stg + r * 128 + (((lane & 7) ^ (r & 7)) << 4));
      if (row_base + r < m_rows && n0 < c.N)
        *reinterpret_cast<uint4*>(cbase + (grow0 + r) * c.ldc + n0) = w;
    }
  }
}

}  // namespace ggc
}  // namespace mxb
