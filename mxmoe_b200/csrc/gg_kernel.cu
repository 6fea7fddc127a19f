// Persistent mixed-precision grouped GEMM for sm_100a.
//
// One launch walks a device-side list of problems C[M,N] = A[M,K] x B[N,K]^T,
// each with its own quantisation scheme (the counterpart of the reference's
// generated `groupgemm_hz_fused_<i>_impl`, mxmoe/kernels/compose_kernel.py:150-295,
// whose per-scheme branches are cta_gemm.cuh:7-107 (fp16), :291-421 (w4a16 g128)
// and :423-608 (w8a8 / w4a4)).
//
// Structure of one CTA (320 threads, one CTA per SM, static round-robin tiles of
// 128 x 256):
//   warp 0      TMA producer: streams operand tiles (128 bytes of K per row and
//               stage) into a ring of shared-memory stages.
//   warp 1      MMA issuer: tcgen05.mma kind::i8 / kind::f16, accumulators in
//               TMEM (two 256-column buffers, so the epilogue of tile i overlaps
//               the main loop of tile i+1).
//   warps 2-5   epilogue: tcgen05.ld -> fused scales -> fp16 -> global stores.
//   warps 6-9   converter (only for 4-bit operands): unpack int4 -> int8 or
//               dequantise 4-bit weights -> fp16 into the swizzled operand tile.
//
// Every wait is bounded (1 s of %globaltimer); on expiry the CTA raises an abort
// flag, records an error in the status block, and all roles drain to a common
// exit that frees TMEM.
#include "gg_types.h"
#include "ptx.cuh"

namespace mxb {

using namespace ptx;

namespace {

constexpr int kThreads       = 320;
constexpr int kOpABytes      = kBM * kRowBytes;         // 16 KiB
constexpr int kOpBBytes      = kBN * kRowBytes;         // 32 KiB
constexpr int kRawABytes     = kBM * 64;                // packed int4 A: 64 bytes per row
constexpr int kRawBBytes     = kBN * 64;                // packed int4 B (w4a4: 256 x 64 B; w4a16: 64 x 128 B)
constexpr uint64_t kTimeoutNs = 1000000000ull;

template <bool kCvt>
struct Cfg {
  static constexpr int kStages     = kCvt ? 3 : 4;
  static constexpr int kStageBytes = kOpABytes + kOpBBytes + (kCvt ? kRawABytes + kRawBBytes : 0);
  static constexpr int kRingBytes  = kStages * kStageBytes;
};

struct Ctrl {
  uint64_t full[4];
  uint64_t cvt[4];
  uint64_t empty[4];
  uint64_t tfull[2];
  uint64_t tempty[2];
  uint32_t tmem_base;
  int abort_flag;
  int total_tiles;
  int pad;
  int tile_end[kMaxProblems];   // inclusive prefix sum of tiles
  int m_eff[kMaxProblems];      // rows of each problem
  int row0[kMaxProblems];       // row shift of each problem
  int meta[kMaxProblems];       // n_tiles << 16 | nkb << 4 | scheme   (nkb < 4096)
  __half sb_stage[4][kBN];      // per epilogue warp: per-channel scales of the current tile
};

template <bool kCvt>
constexpr int smem_bytes() {
  return 1024 + Cfg<kCvt>::kRingBytes + (int)sizeof(Ctrl);
}

__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it       = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 63u) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > kTimeoutNs) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

struct Tile {
  int p, m_tile, n_tile, scheme, nkb;
};

__device__ __forceinline__ Tile find_tile(const Ctrl* c, int count, int t) {
  int lo = 0, hi = count - 1;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (t < c->tile_end[mid]) hi = mid; else lo = mid + 1;
  }
  const int start = lo ? c->tile_end[lo - 1] : 0;
  const int meta  = c->meta[lo];
  const int nt    = meta >> 16;
  const int idx   = t - start;
  Tile r;
  r.p      = lo;
  r.m_tile = idx / nt;
  r.n_tile = idx - r.m_tile * nt;
  r.scheme = meta & 15;
  r.nkb    = (meta >> 4) & 0xFFF;
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

}  // namespace

template <bool kCvt>
__global__ void __launch_bounds__(kThreads, 1)
gg_persistent_kernel(const GGProblemDev* __restrict__ problems, int count, GGStatus* __restrict__ status) {
  using C = Cfg<kCvt>;
  extern __shared__ uint8_t smem_raw[];
  // operand tiles need 1024-byte alignment for the 128-byte swizzle
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen        = smem_raw + (smem_base - smem_u32(smem_raw));
  Ctrl* ctrl               = reinterpret_cast<Ctrl*>(smem_gen + C::kRingBytes);
  volatile int* abort_flag = &ctrl->abort_flag;

  const int tid  = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if (count > kMaxProblems) {
    if (tid == 0 && blockIdx.x == 0) atomicCAS(&status->error, 0, kDevErrTooMany);
    return;
  }

  auto opA  = [&](int s) { return smem_base + s * C::kStageBytes; };
  auto opB  = [&](int s) { return smem_base + s * C::kStageBytes + kOpABytes; };
  auto rawA = [&](int s) { return smem_base + s * C::kStageBytes + kOpABytes + kOpBBytes; };
  auto rawB = [&](int s) { return smem_base + s * C::kStageBytes + kOpABytes + kOpBBytes + kRawABytes; };

  // ------------------------------------------------------------------ setup
  if (tid == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->cvt[s]), 128);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctrl->tfull[b]), 1);
      mbar_init(smem_u32(&ctrl->tempty[b]), 128);
    }
    ctrl->abort_flag = 0;
    fence_mbar_init();
  }
  for (int p = tid; p < count; p += kThreads) {
    const GGProblemDev& pr = problems[p];
    int m = pr.M;
    if (pr.m_dev) m = min(max(*pr.m_dev, 0), pr.M);
    const int r0     = pr.row0_dev ? *pr.row0_dev : pr.row0;
    const int nt     = (pr.N + kBN - 1) / kBN;
    const int kelems = (pr.scheme == SCH_W8A8 || pr.scheme == SCH_W4A4) ? 128 : 64;
    const int nkb    = (pr.K + kelems - 1) / kelems;
    ctrl->tile_end[p] = ((m + kBM - 1) / kBM) * nt;
    ctrl->m_eff[p]    = m;
    ctrl->row0[p]     = r0;
    ctrl->meta[p]     = (nt << 16) | (nkb << 4) | pr.scheme;
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < count; base += 32) {
      const int p = base + lane;
      int v       = (p < count) ? ctrl->tile_end[p] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
      }
      v += carry;
      if (p < count) ctrl->tile_end[p] = v;
      carry = __shfl_sync(0xffffffffu, v, 31);
    }
    if (lane == 0) ctrl->total_tiles = carry;
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  const uint32_t tmem_base = ctrl->tmem_base;
  const int total_tiles    = ctrl->total_tiles;

  // ------------------------------------------------------------------ roles
  if (warp == 0) {
    // ===== TMA producer =====
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const Tile ti          = find_tile(ctrl, count, t);
        const GGProblemDev* pr = problems + ti.p;
        const int a_row        = ctrl->row0[ti.p] + ti.m_tile * kBM;
        for (int kb = 0; kb < ti.nkb; ++kb) {
          if (!wait_bar(smem_u32(&ctrl->empty[stage]), phase ^ 1u, abort_flag)) {
            atomicCAS(&status->error, 0, kDevErrTimeout);
            atomicCAS(&status->where, 0, (1 << 24) | t);
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(&ctrl->full[stage]);
          if (ti.scheme == SCH_W8A8) {
            mbar_expect_tx(bar, kOpABytes + kOpBBytes);
            tma_load_2d(opA(stage), &pr->tmA, bar, kb * 128, a_row);
            tma_load_2d(opB(stage), &pr->tmB, bar, kb * 128, ti.n_tile * kBN);
          } else if (ti.scheme == SCH_FP16) {
            mbar_expect_tx(bar, kOpABytes + kOpBBytes);
            tma_load_2d(opA(stage), &pr->tmA, bar, kb * 64, a_row);
            tma_load_2d(opB(stage), &pr->tmB, bar, kb * 64, ti.n_tile * kBN);
          } else if (kCvt && ti.scheme == SCH_W4A4) {
            // packed rows: 64 bytes (128 codes) of K per stage
            mbar_expect_tx(bar, kRawABytes + kRawBBytes);
            tma_load_2d(rawA(stage), &pr->tmA, bar, kb * 64, a_row);
            tma_load_2d(rawB(stage), &pr->tmB, bar, kb * 64, ti.n_tile * kBN);
          } else if (kCvt && ti.scheme == SCH_W4A16G128) {
            // A: fp16 straight into the operand tile; B: [N/4, K] uint16 words, 64 rows x 128 bytes
            mbar_expect_tx(bar, kOpABytes + (kBN / 4) * 128);
            tma_load_2d(opA(stage), &pr->tmA, bar, kb * 64, a_row);
            tma_load_2d(rawB(stage), &pr->tmB, bar, kb * 128, ti.n_tile * (kBN / 4));
          }
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer =====
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      // The converter arrives on cvt[s] only for tiles with a 4-bit operand, so those barriers complete
      // fewer phases than full[s] / empty[s]: their parity is tracked per stage, on use (bit s).
      uint32_t cvt_parity = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const Tile ti = find_tile(ctrl, count, t);
        if (!wait_bar(smem_u32(&ctrl->tempty[acc]), acc_phase ^ 1u, abort_flag)) {
          atomicCAS(&status->error, 0, kDevErrTimeout);
          atomicCAS(&status->where, 0, (2 << 24) | t);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        const bool is_int     = (ti.scheme == SCH_W8A8 || ti.scheme == SCH_W4A4);
        const bool has_cvt    = kCvt && (ti.scheme == SCH_W4A4 || ti.scheme == SCH_W4A16G128);
        const uint32_t idesc  = is_int ? idesc_i8(kBM, kBN) : idesc_f16(kBM, kBN);
        for (int kb = 0; kb < ti.nkb; ++kb) {
          bool w = wait_bar(smem_u32(&ctrl->full[stage]), phase, abort_flag);
          if (w && has_cvt) {
            w = wait_bar(smem_u32(&ctrl->cvt[stage]), (cvt_parity >> stage) & 1u, abort_flag);
            cvt_parity ^= 1u << stage;
          }
          if (!w) {
            atomicCAS(&status->error, 0, kDevErrTimeout);
            atomicCAS(&status->where, 0, (3 << 24) | t);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint64_t adesc = smem_desc_sw128(opA(stage));
          const uint64_t bdesc = smem_desc_sw128(opB(stage));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // one MMA consumes 32 bytes of K per row: advance the start address by 32 B (>> 4 = 2)
            const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
            if (is_int) mma_i8_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accum);
            else        mma_f16_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accum);
          }
          mma_commit(smem_u32(&ctrl->empty[stage]));
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        mma_commit(smem_u32(&ctrl->tfull[acc]));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp < 6) {
    // ===== epilogue (TMEM lane quarter = warp % 4) =====
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      const Tile ti          = find_tile(ctrl, count, t);
      const GGProblemDev* pr = problems + ti.p;
      // everything that does not depend on the accumulator is fetched before waiting for it
      const int M        = ctrl->m_eff[ti.p];
      const int N        = pr->N;
      const int row      = ti.m_tile * kBM + q * 32 + lane;   // row inside the problem
      const bool valid   = row < M;
      const int64_t grow = (int64_t)ctrl->row0[ti.p] + row;   // row inside the buffers
      const bool is_int  = (ti.scheme == SCH_W8A8 || ti.scheme == SCH_W4A4);
      const int out_mode = pr->out_mode;
      const int ldc      = pr->ldc;
      __half* sbw        = ctrl->sb_stage[warp - 2];
      __half sa          = __float2half(0.f);
      if (is_int && out_mode == OUT_FP16) {
        const int n = ti.n_tile * kBN + lane * 8;
        uint4 sv    = make_uint4(0, 0, 0, 0);
        if (n < N) sv = __ldg(reinterpret_cast<const uint4*>(pr->scale_b + n));
        if (valid) sa = pr->scale_a[grow * pr->sa_stride];
        __syncwarp();
        *reinterpret_cast<uint4*>(sbw + lane * 8) = sv;
        __syncwarp();
      }
      bool ok = wait_bar(smem_u32(&ctrl->tfull[acc]), acc_phase, abort_flag);
      ok      = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) {
          atomicCAS(&status->error, 0, kDevErrTimeout);
          atomicCAS(&status->where, 0, (4 << 24) | t);
        }
        break;
      }
      tc_fence_after_sync();
      const int acc_shift = (ti.scheme == SCH_W4A4) ? 8 : 0;  // 4-bit codes ride in the high nibble of each byte
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + acc * kBN + c * 32 + ((uint32_t)(q * 32) << 16), v);
        tmem_ld_wait();
        const int n0 = ti.n_tile * kBN + c * 32;
        if (!valid || n0 >= N) continue;
        if (out_mode == OUT_ACC) {
          uint32_t* dst = reinterpret_cast<uint32_t*>(pr->C) + grow * ldc + n0;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (n0 + j * 4 < N) {
              uint4 o;
              if (is_int) {
                o.x = (uint32_t)((int)v[4 * j + 0] >> acc_shift);
                o.y = (uint32_t)((int)v[4 * j + 1] >> acc_shift);
                o.z = (uint32_t)((int)v[4 * j + 2] >> acc_shift);
                o.w = (uint32_t)((int)v[4 * j + 3] >> acc_shift);
              } else {
                o = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              }
              *reinterpret_cast<uint4*>(dst + j * 4) = o;
            }
          }
        } else {
          __half* dst = reinterpret_cast<__half*>(pr->C) + grow * ldc + n0;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (n0 + j * 8 < N) {
              uint32_t o[4];
              if (is_int) {
                // C = fp16_rn( float(acc) * float( fp16_rn(sa * sb) ) )   (mm_tile.cuh:490-493)
                const uint4 sbv   = *reinterpret_cast<const uint4*>(sbw + c * 32 + j * 8);
                const __half2* s2 = reinterpret_cast<const __half2*>(&sbv);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float p0 = __half2float(__hmul(sa, __low2half(s2[e])));
                  const float p1 = __half2float(__hmul(sa, __high2half(s2[e])));
                  const float f0 = (float)((int)v[8 * j + 2 * e] >> acc_shift) * p0;
                  const float f1 = (float)((int)v[8 * j + 2 * e + 1] >> acc_shift) * p1;
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
      }
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&ctrl->tempty[acc]));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  } else if (kCvt) {
    // ===== converter (128 threads) =====
    const int ct = tid - 192;
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    for (int t = blockIdx.x; alive && t < total_tiles; t += gridDim.x) {
      const Tile ti = find_tile(ctrl, count, t);
      if (ti.scheme != SCH_W4A4 && ti.scheme != SCH_W4A16G128) {
        // Nothing to convert, but the ring must still be followed stage by stage: a role that ran
        // more than one ring revolution ahead of the producer would see the parity of an older
        // phase of full[s] and mistake it for the one it is waiting for.
        for (int kb = 0; kb < ti.nkb; ++kb) {
          bool ok = wait_bar(smem_u32(&ctrl->full[stage]), phase, abort_flag);
          ok      = __all_sync(0xffffffffu, ok);
          if (!ok) {
            if (lane == 0) {
              atomicCAS(&status->error, 0, kDevErrTimeout);
              atomicCAS(&status->where, 0, (6 << 24) | t);
            }
            alive = false;
            break;
          }
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
        continue;
      }
      const GGProblemDev* pr = problems + ti.p;
      // w4a16: this thread owns packed row `prow` (8 n-rows interleaved) and one half (fh) of each 16-k block
      const int prow = ct >> 1;
      const int fh   = ct & 1;
      const int r    = prow & 7;
      const int n_lo = 32 * (prow >> 3) + 16 * fh + r;  // row of the 256-row operand tile; n_hi = n_lo + 8
      const int N    = pr->N;
      const int gn   = ti.n_tile * kBN + n_lo;
      __half2 sz_lo = __float2half2_rn(0.f), sz_hi = __float2half2_rn(0.f);
      for (int kb = 0; kb < ti.nkb; ++kb) {
        if (ti.scheme == SCH_W4A16G128 && (kb & 1) == 0) {
          // (scale, zero) pairs, [K/128][N][2] fp16; one group spans two 64-k stages
          const __half2* sz = reinterpret_cast<const __half2*>(pr->scale_b) + (int64_t)(kb >> 1) * N;
          if (gn < N) sz_lo = __ldg(sz + gn);
          if (gn + 8 < N) sz_hi = __ldg(sz + gn + 8);
        }
        bool ok = wait_bar(smem_u32(&ctrl->full[stage]), phase, abort_flag);
        ok      = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) {
            atomicCAS(&status->error, 0, kDevErrTimeout);
            atomicCAS(&status->where, 0, (5 << 24) | t);
          }
          alive = false;
          break;
        }
        if (ti.scheme == SCH_W4A4) {
          // rawA (128 rows) and rawB (256 rows) are contiguous, and so are opA / opB:
          // 384 rows x 4 packed 16-byte chunks -> 384 rows x 8 int8 chunks, 128-byte swizzle.
          const uint32_t src = rawA(stage);
          const uint32_t dst = opA(stage);
#pragma unroll 4
          for (int i = 0; i < 12; ++i) {
            const int g   = i * 128 + ct;
            const int row = g >> 2;
            const int c   = g & 3;
            const uint4 w = lds128(src + row * 64 + c * 16);
            // code q (two's complement nibble) -> byte 16*q: both operands carry the factor,
            // the accumulator is 256x the true one and is shifted back in the epilogue.
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
        } else {
          const uint32_t src = rawB(stage) + prow * 128;
          const uint32_t dlo = opB(stage) + n_lo * 128;
          const uint32_t dhi = dlo + 8 * 128;
          const __half2 s_lo = __half2half2(__low2half(sz_lo)), z_lo = __half2half2(__high2half(sz_lo));
          const __half2 s_hi = __half2half2(__low2half(sz_hi)), z_hi = __half2half2(__high2half(sz_hi));
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int kb16 = (prow + i) & 3;           // rotated so that a quarter-warp hits 8 distinct bank groups
            const uint4 w  = lds128(src + (2 * kb16 + fh) * 16);
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
              const int c = cc ^ fh;                     // odd threads write the other k-half first (bank spread)
              const uint32_t phys = (uint32_t)(((2 * kb16 + c) ^ r) << 4);
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
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(&ctrl->cvt[stage]));
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncthreads();
  if (*abort_flag) {
    // give copies that are still in flight time to land before shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

cudaError_t gg_configure_kernels() {
  cudaError_t e = cudaFuncSetAttribute(gg_persistent_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       smem_bytes<false>());
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(gg_persistent_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              smem_bytes<true>());
}

void gg_launch_kernel(const GGProblemDev* problems, int count, GGStatus* status, bool needs_cvt, int num_ctas,
                      cudaStream_t stream) {
  if (needs_cvt) {
    gg_persistent_kernel<true><<<num_ctas, kThreads, smem_bytes<true>(), stream>>>(problems, count, status);
  } else {
    gg_persistent_kernel<false><<<num_ctas, kThreads, smem_bytes<false>(), stream>>>(problems, count, status);
  }
}

}  // namespace mxb
