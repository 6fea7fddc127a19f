// Persistent mixed-precision grouped GEMM for sm_100a on CTA pairs (tcgen05 cta_group::2).
//
// Same problem list, schemes and results as gg_kernel.cu, but two CTAs of a cluster (two SMs)
// work on one 256 x 256 tile: each CTA loads (and, for 4-bit operands, converts) its own 128 rows of
// A and its own 128-row half of B, the leader CTA issues one M=256 MMA for both, and each CTA drains
// its own 128 x 256 half of the accumulator.  Per output element that is 2/3 of the operand traffic
// (L2 -> shared memory, and shared-memory conversion work) of the 128 x 256 single-CTA tile, and the
// smaller stages allow a deeper ring (6 x 32 KiB direct, 4 x 48 KiB with converter buffers).
//
// No load uses cluster multicast: every CTA fetches its own operands (the cta_group::2 form of the
// tensor load only redirects the byte-count completion to the leader's mbarrier).
//
// Barriers (same offsets in both CTAs; "L" = only the leader's instance is used):
//   full[s]    L  operands that TMA writes in final form (w8a8, fp16, the fp16 A of w4a16), both CTAs
//   rawfull[s]    packed 4-bit operands of this CTA landed (local)
//   cvt[s]     L  converters of both CTAs finished stage s (256 arrivals)
//   empty[s]      stage s may be refilled (the leader's MMA commit, multicast to both CTAs)
//   tfull[b]      accumulator b complete (MMA commit, multicast)
//   tempty[b]  L  accumulator b drained by both CTAs (256 arrivals)
// full / rawfull / cvt complete a phase only on tiles that use them, so their parity is tracked per
// stage at each use; a waiter can then never be more than one phase away from the barrier.
#include <cuda.h>

#include "gg_common.cuh"

namespace mxb {

using namespace ptx;
using namespace ggc;

namespace {

constexpr int kThreads  = 320;
constexpr int kHalf     = 128;                 // rows of A, of B and of C per CTA
constexpr int kOpBytes  = kHalf * kRowBytes;   // 16 KiB: one operand half-tile
constexpr int kRawBytes = kHalf * 64;          // 8 KiB: packed int4 half-tile (w4a16 uses 4 KiB of the B one)
constexpr int kMaxStages = 6;

template <bool kCvt>
struct PCfg {
  static constexpr int kStages     = kCvt ? 4 : 6;
  static constexpr int kStageBytes = 2 * kOpBytes + (kCvt ? 2 * kRawBytes : 0);
  static constexpr int kRingBytes  = kStages * kStageBytes;
};

struct PCtrl {
  uint64_t full[kMaxStages];
  uint64_t rawfull[kMaxStages];
  uint64_t cvt[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tfull[2];
  uint64_t tempty[2];
  uint32_t tmem_base;
  int abort_flag;
  int pad[2];
  Sched sched;
  __half sb_stage[4][kBN];
};

template <bool kCvt>
constexpr int pair_smem_bytes() {
  return 1024 + PCfg<kCvt>::kRingBytes + (int)sizeof(PCtrl);
}

__device__ __forceinline__ void preport(GGStatus* status, int role, int tile) {
  atomicCAS(&status->error, 0, kDevErrTimeout);
  atomicCAS(&status->where, 0, (role << 24) | tile);
}

}  // namespace

template <bool kCvt>
__global__ void __launch_bounds__(kThreads, 1)
gg_pair_kernel(const GGProblemDev* __restrict__ problems, int count, GGStatus* __restrict__ status) {
  using C = PCfg<kCvt>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen        = smem_raw + (smem_base - smem_u32(smem_raw));
  PCtrl* ctrl              = reinterpret_cast<PCtrl*>(smem_gen + C::kRingBytes);
  Sched* sc                = &ctrl->sched;
  volatile int* abort_flag = &ctrl->abort_flag;

  const int tid  = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int rank = (int)cluster_ctarank();          // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;

  if (count > kMaxProblems) {                       // uniform over the grid: both CTAs of a pair leave
    if (tid == 0 && blockIdx.x == 0) atomicCAS(&status->error, 0, kDevErrTooMany);
    return;
  }

  auto opA  = [&](int s) { return smem_base + s * C::kStageBytes; };
  auto opB  = [&](int s) { return smem_base + s * C::kStageBytes + kOpBytes; };
  auto rawA = [&](int s) { return smem_base + s * C::kStageBytes + 2 * kOpBytes; };
  auto rawB = [&](int s) { return smem_base + s * C::kStageBytes + 2 * kOpBytes + kRawBytes; };

  // ------------------------------------------------------------------ setup
  if (tid == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->rawfull[s]), 1);
      mbar_init(smem_u32(&ctrl->cvt[s]), 256);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctrl->tfull[b]), 1);
      mbar_init(smem_u32(&ctrl->tempty[b]), 256);
    }
    ctrl->abort_flag = 0;
    fence_mbar_init();
  }
  build_sched(sc, problems, count, 2 * kHalf);
  if (warp == 1) {
    tmem_alloc2(smem_u32(&ctrl->tmem_base), 512);
    tmem_relinquish2();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                               // both CTAs' barriers exist before anyone signals them
  tc_fence_after_sync();

  const long long prof_t0 = clock64();
  const uint32_t tmem_base = ctrl->tmem_base;
  const int total_tiles    = sc->total_tiles;

  // ------------------------------------------------------------------ roles
  if (warp == 0) {
    // ===== TMA producer (both CTAs; each fetches its own halves) =====
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long w_prod = 0, n_stage = 0, n_tile = 0;
      for (int t = pair; ok && t < total_tiles; t += npairs) {
        const Tile ti          = find_tile(sc, count, t);
        const GGProblemDev* pr = problems + ti.p;
        ++n_tile;
        const int a_row        = sc->row0[ti.p] + ti.m_tile * 2 * kHalf + rank * kHalf;
        const int b_row        = ti.n_tile * kBN + rank * kHalf;
        for (int kb = 0; kb < ti.nkb; ++kb) {
          const long long c0 = clock64();
          const bool got = wait_bar(smem_u32(&ctrl->empty[stage]), phase ^ 1u, abort_flag);
          w_prod += clock64() - c0;
          ++n_stage;
          if (!got) {
            preport(status, 1, t);
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&ctrl->full[stage]);
          const uint32_t rawf = smem_u32(&ctrl->rawfull[stage]);
          if (ti.scheme == SCH_W8A8 || ti.scheme == SCH_FP16) {
            const int x = kb * (ti.scheme == SCH_W8A8 ? 128 : 64);
            if (rank == 0) mbar_expect_tx(full, 4 * kOpBytes);          // A + B halves of both CTAs
            tma_load_2d_pair(opA(stage), &pr->tmA, full, x, a_row);
            tma_load_2d_pair(opB(stage), &pr->tmB, full, x, b_row);
          } else if (kCvt && ti.scheme == SCH_W4A4_XA) {
            if (rank == 0) mbar_expect_tx(full, 2 * kOpBytes);          // expanded int8 A of both CTAs
            tma_load_2d_pair(opA(stage), &pr->tmA, full, kb * 128, a_row);
            mbar_expect_tx(rawf, kRawBytes);
            tma_load_2d(rawB(stage), &pr->tmB, rawf, kb * 64, b_row);
          } else if (kCvt && ti.scheme == SCH_W4A4) {
            mbar_expect_tx(rawf, 2 * kRawBytes);
            tma_load_2d(rawA(stage), &pr->tmA, rawf, kb * 64, a_row);
            tma_load_2d(rawB(stage), &pr->tmB, rawf, kb * 64, b_row);
          } else if (kCvt && ti.scheme == SCH_W4A16G128) {
            if (rank == 0) mbar_expect_tx(full, 2 * kOpBytes);          // fp16 A of both CTAs
            tma_load_2d_pair(opA(stage), &pr->tmA, full, kb * 64, a_row);
            mbar_expect_tx(rawf, (kHalf / 4) * 128);                    // 32 packed rows x 128 bytes
            tma_load_2d(rawB(stage), &pr->tmB, rawf, kb * 128, b_row / 4);
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
    // ===== MMA issuer (leader CTA only) =====
    if (lane == 0 && rank == 0) {
      int stage = 0;
      int acc = 0;
      uint32_t acc_phase = 0, full_parity = 0, cvt_parity = 0;
      bool ok = true;
      long long w_oper = 0, w_acc = 0, w_issue = 0;
      for (int t = pair; ok && t < total_tiles; t += npairs) {
        const Tile ti = find_tile(sc, count, t);
        const long long ca = clock64();
        const bool gota = wait_bar(smem_u32(&ctrl->tempty[acc]), acc_phase ^ 1u, abort_flag);
        w_acc += clock64() - ca;
        if (!gota) {
          preport(status, 2, t);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        const bool is_int     = (ti.scheme != SCH_FP16 && ti.scheme != SCH_W4A16G128);
        const bool has_cvt    = kCvt && (ti.scheme != SCH_FP16 && ti.scheme != SCH_W8A8);
        const bool has_full   = ti.scheme != SCH_W4A4;
        const uint32_t idesc  = is_int ? idesc_i8(2 * kHalf, kBN) : idesc_f16(2 * kHalf, kBN);
        for (int kb = 0; kb < ti.nkb; ++kb) {
          const long long c0 = clock64();
          bool w = true;
          if (has_full) {
            w = wait_bar(smem_u32(&ctrl->full[stage]), (full_parity >> stage) & 1u, abort_flag);
            full_parity ^= 1u << stage;
          }
          if (w && has_cvt) {
            w = wait_bar(smem_u32(&ctrl->cvt[stage]), (cvt_parity >> stage) & 1u, abort_flag);
            cvt_parity ^= 1u << stage;
          }
          if (!w) {
            preport(status, 3, t);
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
            const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
            if (is_int) mma_i8_ss2(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accum);
            else        mma_f16_ss2(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accum);
          }
          mma_commit2(smem_u32(&ctrl->empty[stage]), 3);
          w_issue += clock64() - c1;
          if (++stage == C::kStages) stage = 0;
        }
        if (!ok) break;
        mma_commit2(smem_u32(&ctrl->tfull[acc]), 3);
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
    // ===== epilogue (both CTAs; TMEM lane quarter = warp % 4) =====
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    __half* sbw = ctrl->sb_stage[warp - 2];
    long long w_epi = 0, w_store = 0;
    for (int t = pair; t < total_tiles; t += npairs) {
      const Tile ti          = find_tile(sc, count, t);
      const GGProblemDev* pr = problems + ti.p;
      const EpiCtx ec = epi_prefetch(pr, sc, ti, ti.m_tile * 2 * kHalf + rank * kHalf + q * 32 + lane, lane, sbw);
      const long long c0 = clock64();
      bool ok = wait_bar(smem_u32(&ctrl->tfull[acc]), acc_phase, abort_flag);
      ok      = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) preport(status, 4, t);
        break;
      }
      const long long c1 = clock64();
      w_epi += c1 - c0;
      tc_fence_after_sync();
      epi_store(ec, pr, tmem_base + acc * kBN + ((uint32_t)(q * 32) << 16), sbw);
      tc_fence_before_sync();
      mbar_arrive_leader(smem_u32(&ctrl->tempty[acc]));
      w_store += clock64() - c1;
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (blockIdx.x == 0 && warp == 2 && lane == 0) {
      status->prof[PROF_EPI_WAIT]  = w_epi;
      status->prof[PROF_EPI_STORE] = w_store;
    }
  } else if (kCvt) {
    // ===== converter (both CTAs, 128 threads each, own halves only) =====
    const int ct = tid - 192;
    int stage = 0;
    uint32_t raw_parity = 0;
    bool alive = true;
    long long w_cwait = 0, w_cwork = 0;
    const W4A16Lane<32, 128> ln(ct);
    for (int t = pair; alive && t < total_tiles; t += npairs) {
      const Tile ti = find_tile(sc, count, t);
      if (ti.scheme == SCH_FP16 || ti.scheme == SCH_W8A8) {
        stage = (stage + ti.nkb) % C::kStages;      // rawfull / cvt are not used by this tile
        continue;
      }
      const GGProblemDev* pr = problems + ti.p;
      const int N  = pr->N;
      const int gn = ti.n_tile * kBN + rank * kHalf + ln.n_lo;
      __half2 sz_lo = __float2half2_rn(0.f), sz_hi = __float2half2_rn(0.f);
      for (int kb = 0; kb < ti.nkb; ++kb) {
        if (ti.scheme == SCH_W4A16G128 && (kb & 1) == 0) {
          const __half2* sz = reinterpret_cast<const __half2*>(pr->scale_b) + (int64_t)(kb >> 1) * N;
          if (gn < N) sz_lo = __ldg(sz + gn);
          if (gn + 8 < N) sz_hi = __ldg(sz + gn + 8);
        }
        const long long c0 = clock64();
        bool ok = wait_bar(smem_u32(&ctrl->rawfull[stage]), (raw_parity >> stage) & 1u, abort_flag);
        raw_parity ^= 1u << stage;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) preport(status, 5, t);
          alive = false;
          break;
        }
        const long long c1 = clock64();
        w_cwait += c1 - c0;
        if (ti.scheme == SCH_W4A4_XA) {
          convert_w4a4<128>(rawB(stage), opB(stage), kHalf, ct);
        } else if (ti.scheme == SCH_W4A4) {
          // rawA | rawB-half are contiguous (2 x 128 packed rows), and so are opA | opB-half
          convert_w4a4<128>(rawA(stage), opA(stage), 2 * kHalf, ct);
        } else {
          convert_w4a16<32, 128>(ln, rawB(stage), opB(stage), sz_lo, sz_hi);
        }
        fence_proxy_async_all();
        mbar_arrive_leader(smem_u32(&ctrl->cvt[stage]));
        w_cwork += clock64() - c1;
        if (++stage == C::kStages) stage = 0;
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
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();            // the peer may still signal this CTA's barriers / read its shared memory
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc2(tmem_base, 512);
  }
}

cudaError_t gg_configure_pair() {
  cudaError_t e = cudaFuncSetAttribute(gg_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       pair_smem_bytes<false>());
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(gg_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              pair_smem_bytes<true>());
}

cudaError_t gg_launch_pair(const GGProblemDev* problems, int count, GGStatus* status, int cvt_mode, int num_ctas,
                           cudaStream_t stream) {
  const bool needs_cvt   = cvt_mode != 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim            = dim3((unsigned)(num_ctas & ~1), 1, 1);
  cfg.blockDim           = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes   = needs_cvt ? pair_smem_bytes<true>() : pair_smem_bytes<false>();
  cfg.stream             = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id               = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs    = attr;
  cfg.numAttrs = 1;
  if (needs_cvt) return cudaLaunchKernelEx(&cfg, gg_pair_kernel<true>, problems, count, status);
  return cudaLaunchKernelEx(&cfg, gg_pair_kernel<false>, problems, count, status);
}

}  // namespace mxb
