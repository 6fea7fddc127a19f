// Persistent mixed-precision grouped GEMM for sm_100a, one CTA per SM.
//
// One launch walks a device-side list of problems C[M,N] = A[M,K] x B[N,K]^T,
// each with its own quantisation scheme (the counterpart of the reference's
// generated `groupgemm_hz_fused_<i>_impl`, mxmoe/kernels/compose_kernel.py:150-295,
// whose per-scheme branches are cta_gemm.cuh:7-107 (fp16), :291-421 (w4a16 g128)
// and :423-608 (w8a8 / w4a4)).
//
// Structure of one CTA (320 threads, static round-robin tiles of 128 x 256):
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
#include "gg_common.cuh"

namespace mxb {

using namespace ptx;
using namespace ggc;

namespace {

constexpr int kOpABytes  = kBM * kRowBytes;   // 16 KiB
constexpr int kOpBBytes  = kBN * kRowBytes;   // 32 KiB
constexpr int kRawABytes = kBM * 64;          // packed int4 A: 64 bytes per row
constexpr int kRawBBytes = kBN * 64;          // packed int4 B (w4a4: 256 x 64 B; w4a16: 64 x 128 B)

// kMode 0: no 4-bit operand; 1: only weights are converted (w4a16, w4a4 with expanded activations);
// 2: packed 4-bit activations as well.  Modes 0 and 1 leave room for the staged epilogue.
template <int kMode>
struct Cfg {
  static constexpr int kStages     = kMode ? 3 : 4;
  static constexpr int kStageBytes = kOpABytes + kOpBBytes + (kMode ? kRawBBytes : 0) + (kMode == 2 ? kRawABytes : 0);
  static constexpr int kRingBytes  = kStages * kStageBytes;
  static constexpr int kEpiBytes   = kMode < 2 ? 4 * 4096 : 0;   // 4 epilogue warps x (32 rows x 128 bytes)
  static constexpr int kCvtThreads = kMode ? 256 : 0;            // converter warps 6..13
  static constexpr int kThreads    = 192 + kCvtThreads;
};

struct Ctrl {
  uint64_t full[4];
  uint64_t cvt[4];
  uint64_t empty[4];
  uint64_t tfull[2];
  uint64_t tempty[2];
  uint32_t tmem_base;
  int abort_flag;
  int pad[2];
  Sched sched;
  __half sb_stage[4][kBN];   // per epilogue warp: per-channel scales of the current tile
};

template <int kMode>
constexpr int smem_bytes() {
  return 1024 + Cfg<kMode>::kRingBytes + Cfg<kMode>::kEpiBytes + (int)sizeof(Ctrl);
}

__device__ __forceinline__ void report(GGStatus* status, int role, int tile) {
  atomicCAS(&status->error, 0, kDevErrTimeout);
  atomicCAS(&status->where, 0, (role << 24) | tile);
}

}  // namespace

template <int kMode>
__global__ void __launch_bounds__(Cfg<kMode>::kThreads, 1)
gg_persistent_kernel(const GGProblemDev* __restrict__ problems, int count, GGStatus* __restrict__ status) {
  using C = Cfg<kMode>;
  constexpr bool kCvt = kMode != 0;
  extern __shared__ uint8_t smem_raw[];
  // operand tiles need 1024-byte alignment for the 128-byte swizzle
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen        = smem_raw + (smem_base - smem_u32(smem_raw));
  Ctrl* ctrl               = reinterpret_cast<Ctrl*>(smem_gen + C::kRingBytes + C::kEpiBytes);
  const uint32_t epi_base  = smem_base + C::kRingBytes;
  Sched* sc                = &ctrl->sched;
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
  // packed operands: [rawA |] rawB (rawA exists in mode 2 only and is directly followed by rawB)
  auto rawA = [&](int s) { return smem_base + s * C::kStageBytes + kOpABytes + kOpBBytes; };
  auto rawB = [&](int s) {
    return smem_base + s * C::kStageBytes + kOpABytes + kOpBBytes + (kMode == 2 ? kRawABytes : 0);
  };

  // ------------------------------------------------------------------ setup
  if (tid == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->cvt[s]), C::kCvtThreads ? C::kCvtThreads : 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctrl->tfull[b]), 1);
      mbar_init(smem_u32(&ctrl->tempty[b]), 128);
    }
    ctrl->abort_flag = 0;
    fence_mbar_init();
  }
  build_sched(sc, problems, count, kBM);
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  const long long prof_t0 = clock64();
  const uint32_t tmem_base = ctrl->tmem_base;
  const int total_tiles    = sc->total_tiles;

  // ------------------------------------------------------------------ roles
  if (warp == 0) {
    // ===== TMA producer =====  (B descriptors have 128-row boxes: a 256-row tile is two loads)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long w_prod = 0, n_stage = 0, n_tile = 0;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const Tile ti          = find_tile(sc, count, t);
        const GGProblemDev* pr = problems + ti.p;
        ++n_tile;
        const int a_row        = sc->row0[ti.p] + ti.m_tile * kBM;
        const int b_row        = ti.n_tile * kBN;
        for (int kb = 0; kb < ti.nkb; ++kb) {
          const long long c0 = clock64();
          const bool got = wait_bar(smem_u32(&ctrl->empty[stage]), phase ^ 1u, abort_flag);
          w_prod += clock64() - c0;
          ++n_stage;
          if (!got) {
            report(status, 1, t);
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(&ctrl->full[stage]);
          if (ti.scheme == SCH_W8A8 || ti.scheme == SCH_FP16) {
            const int x = kb * (ti.scheme == SCH_W8A8 ? 128 : 64);
            mbar_expect_tx(bar, kOpABytes + kOpBBytes);
            tma_load_2d(opA(stage), &pr->tmA, bar, x, a_row);
            tma_load_2d(opB(stage), &pr->tmB, bar, x, b_row);
            tma_load_2d(opB(stage) + kOpBBytes / 2, &pr->tmB, bar, x, b_row + kBN / 2);
          } else if (kCvt && ti.scheme == SCH_W4A4_XA) {
            // activations already one byte per code: straight into the operand tile; weights packed
            mbar_expect_tx(bar, kOpABytes + kRawBBytes);
            tma_load_2d(opA(stage), &pr->tmA, bar, kb * 128, a_row);
            tma_load_2d(rawB(stage), &pr->tmB, bar, kb * 64, b_row);
            tma_load_2d(rawB(stage) + kRawBBytes / 2, &pr->tmB, bar, kb * 64, b_row + kBN / 2);
          } else if (kMode == 2 && ti.scheme == SCH_W4A4) {
            // packed rows: 64 bytes (128 codes) of K per stage
            mbar_expect_tx(bar, kRawABytes + kRawBBytes);
            tma_load_2d(rawA(stage), &pr->tmA, bar, kb * 64, a_row);
            tma_load_2d(rawB(stage), &pr->tmB, bar, kb * 64, b_row);
            tma_load_2d(rawB(stage) + kRawBBytes / 2, &pr->tmB, bar, kb * 64, b_row + kBN / 2);
          } else if (kCvt && ti.scheme == SCH_W4A16G128) {
            // A: fp16 straight into the operand tile; B: [N/4, K] uint16 words, 2 x (32 rows x 128 bytes)
            mbar_expect_tx(bar, kOpABytes + (kBN / 4) * 128);
            tma_load_2d(opA(stage), &pr->tmA, bar, kb * 64, a_row);
            tma_load_2d(rawB(stage), &pr->tmB, bar, kb * 128, b_row / 4);
            tma_load_2d(rawB(stage) + (kBN / 8) * 128, &pr->tmB, bar, kb * 128, b_row / 4 + kBN / 8);
          }
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (blockIdx.x == 0) {
        status->prof[PROF_PROD_WAIT] = w_prod;
        status->prof[PROF_TILES]     = n_tile;
        status->prof[PROF_STAGES]    = n_stage;
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
      long long w_oper = 0, w_acc = 0, w_issue = 0;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const Tile ti = find_tile(sc, count, t);
        const long long ca = clock64();
        const bool gota = wait_bar(smem_u32(&ctrl->tempty[acc]), acc_phase ^ 1u, abort_flag);
        w_acc += clock64() - ca;
        if (!gota) {
          report(status, 2, t);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        const bool is_int     = (ti.scheme != SCH_FP16 && ti.scheme != SCH_W4A16G128);
        const bool has_cvt    = kCvt && (ti.scheme != SCH_FP16 && ti.scheme != SCH_W8A8);
        const uint32_t idesc  = is_int ? idesc_i8(kBM, kBN) : idesc_f16(kBM, kBN);
        for (int kb = 0; kb < ti.nkb; ++kb) {
          const long long c0 = clock64();
          bool w = wait_bar(smem_u32(&ctrl->full[stage]), phase, abort_flag);
          if (w && has_cvt) {
            w = wait_bar(smem_u32(&ctrl->cvt[stage]), (cvt_parity >> stage) & 1u, abort_flag);
            cvt_parity ^= 1u << stage;
          }
          if (!w) {
            report(status, 3, t);
            ok = false;
            break;
          }
          const long long c1 = clock64();
          w_oper += c1 - c0;
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
          w_issue += clock64() - c1;
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        mma_commit(smem_u32(&ctrl->tfull[acc]));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (blockIdx.x == 0) {
        status->prof[PROF_MMA_WAIT_OPER] = w_oper;
        status->prof[PROF_MMA_WAIT_ACC]  = w_acc;
        status->prof[PROF_MMA_ISSUE]     = w_issue;
      }
    }
  } else if (warp < 6) {
    // ===== epilogue (TMEM lane quarter = warp % 4) =====
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    __half* sbw = ctrl->sb_stage[warp - 2];
    long long w_epi = 0, w_store = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      const Tile ti          = find_tile(sc, count, t);
      const GGProblemDev* pr = problems + ti.p;
      const EpiCtx ec        = epi_prefetch(pr, sc, ti, ti.m_tile * kBM + q * 32 + lane, lane, sbw);
      const long long c0 = clock64();
      bool ok = wait_bar(smem_u32(&ctrl->tfull[acc]), acc_phase, abort_flag);
      ok      = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(status, 4, t);
        break;
      }
      const long long c1 = clock64();
      w_epi += c1 - c0;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * kBN + ((uint32_t)(q * 32) << 16);
      if (C::kEpiBytes) {
        epi_store_staged(ec, pr, taddr, sbw, epi_base + (warp - 2) * 4096, lane, ti.m_tile * kBM + q * 32,
                         sc->m_eff[ti.p]);
      } else {
        epi_store(ec, pr, taddr, sbw);
      }
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&ctrl->tempty[acc]));
      w_store += clock64() - c1;
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (blockIdx.x == 0 && warp == 2 && lane == 0) {
      status->prof[PROF_EPI_WAIT]  = w_epi;
      status->prof[PROF_EPI_STORE] = w_store;
    }
  } else if (kCvt) {
    // ===== converter (8 warps) =====
    const int ct = tid - 192;
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    long long w_cwait = 0, w_cwork = 0;
    constexpr int kCT = C::kCvtThreads ? C::kCvtThreads : 128;
    const W4A16Lane<64, kCT> ln(ct);
    for (int t = blockIdx.x; alive && t < total_tiles; t += gridDim.x) {
      const Tile ti          = find_tile(sc, count, t);
      const GGProblemDev* pr = problems + ti.p;
      const bool convert     = ti.scheme != SCH_FP16 && ti.scheme != SCH_W8A8;
      const int N            = pr->N;
      const int gn           = ti.n_tile * kBN + ln.n_lo;
      __half2 sz_lo = __float2half2_rn(0.f), sz_hi = __float2half2_rn(0.f);
      for (int kb = 0; kb < ti.nkb; ++kb) {
        if (ti.scheme == SCH_W4A16G128 && (kb & 1) == 0) {
          // (scale, zero) pairs, [K/128][N][2] fp16; one group spans two 64-k stages
          const __half2* sz = reinterpret_cast<const __half2*>(pr->scale_b) + (int64_t)(kb >> 1) * N;
          if (gn < N) sz_lo = __ldg(sz + gn);
          if (gn + 8 < N) sz_hi = __ldg(sz + gn + 8);
        }
        // Tiles without a 4-bit operand are followed stage by stage as well: a role that ran more than
        // one ring revolution ahead of the producer would see the parity of an older phase of full[s]
        // and mistake it for the one it is waiting for.
        const long long c0 = clock64();
        bool ok = wait_bar(smem_u32(&ctrl->full[stage]), phase, abort_flag);
        ok      = __all_sync(0xffffffffu, ok);
        const long long c1 = clock64();
        w_cwait += c1 - c0;
        if (!ok) {
          if (lane == 0) report(status, convert ? 5 : 6, t);
          alive = false;
          break;
        }
        if (convert) {
          if (ti.scheme == SCH_W4A4_XA) {
            convert_w4a4<kCT>(rawB(stage), opB(stage), kBN, ct);
          } else if (kMode == 2 && ti.scheme == SCH_W4A4) {
            // rawA (128 rows) and rawB (256 rows) are contiguous, and so are opA / opB
            convert_w4a4<kCT>(rawA(stage), opA(stage), kBM + kBN, ct);
          } else {
            convert_w4a16<64, kCT>(ln, rawB(stage), opB(stage), sz_lo, sz_hi);
          }
          fence_proxy_async_smem();
          mbar_arrive(smem_u32(&ctrl->cvt[stage]));
          w_cwork += clock64() - c1;
        }
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
    }
    if (blockIdx.x == 0 && ct == 0) {
      status->prof[PROF_CVT_WAIT] = w_cwait;
      status->prof[PROF_CVT_WORK] = w_cwork;
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncthreads();
  if (blockIdx.x == 0 && tid == 0) status->prof[PROF_TOTAL] = clock64() - prof_t0;
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

cudaError_t gg_configure_single() {
  cudaError_t e = cudaFuncSetAttribute(gg_persistent_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<0>());
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(gg_persistent_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<1>());
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(gg_persistent_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<2>());
}

void gg_launch_single(const GGProblemDev* problems, int count, GGStatus* status, int cvt_mode, int num_ctas,
                      cudaStream_t stream) {
  if (cvt_mode == 2) {
    gg_persistent_kernel<2><<<num_ctas, Cfg<2>::kThreads, smem_bytes<2>(), stream>>>(problems, count, status);
  } else if (cvt_mode == 1) {
    gg_persistent_kernel<1><<<num_ctas, Cfg<1>::kThreads, smem_bytes<1>(), stream>>>(problems, count, status);
  } else {
    gg_persistent_kernel<0><<<num_ctas, Cfg<0>::kThreads, smem_bytes<0>(), stream>>>(problems, count, status);
  }
}

}  // namespace mxb
