// Persistent mixed-precision grouped GEMM for sm_100a with swapped operands, one CTA per SM.
//
// Same contract as gg_kernel.cu (one launch walks a device-side list of problems
// C[M,N] = A[M,K] x B[N,K]^T, each with its own quantisation scheme; reference:
// mxmoe/kernels/compose_kernel.py:150-295, cta_gemm.cuh:7-107, :291-421, :423-608), but the MMA
// computes C^T: the WEIGHTS are the M side (tiles of 128 output channels) and the TOKENS the
// N side (tiles of up to 176 rows, any multiple of 16).  Consequences:
//   * 4-bit weights are unpacked / dequantised by the converter warps from shared memory straight
//     into TENSOR MEMORY (tcgen05.st) and the MMA takes its A operand from there: the converted
//     weights never travel through shared memory again, which is the unit that limits the kernel
//     with the operands the other way round.
//   * a ragged expert costs MMA time for its rows rounded up to 16, not to 128.
//   * the weight-conversion work per MAC shrinks with the token tile (176 instead of 128 rows).
//
// TMEM columns: [0,176) and [176,352) two accumulators (128 channels x up to 176 tokens, fp32/int32),
// [352,512) five A-operand slots of 32 columns (128 channels x 128 bytes of K each), one per ring stage.
//
// One CTA (608 threads; 352 when no problem has 4-bit weights):
//   warp 0      TMA producer: weights (packed or plain) + activations into a ring of 5 stages.
//   warp 1      MMA issuer.  It never touches shared memory: while the tensor core streams its operands
//               from shared memory, a shared-memory round trip of a regular warp (an mbarrier.try_wait, a
//               plain load) takes hundreds of cycles, and one of them between two batches of MMAs leaves
//               the tensor pipe idle.  The warp is paced by NAMED barriers (bar.sync) instead.
//   warps 2-5, 7-10   epilogue: tcgen05.ld (lane = channel, columns = tokens) -> scales -> fp16 ->
//               transposed through shared memory -> 16-byte global stores along the channel axis.  Two warps
//               per TMEM lane quarter take the 32-token chunks of a tile in turn: a chunk is a chain of three
//               shared-memory round trips (scales, transpose out, transpose in) of several hundred cycles each
//               while the tensor core streams operands, and with one warp per quarter a tile of few K blocks
//               (the down projection) was bounded by its epilogue.
//   warp 6      watcher: waits on the mbarriers the TMA unit completes (xfull[s]; wfull[s] too when the CTA has no
//               converter warps) and forwards each stage to the MMA warp with bar.arrive.
//   warps 11-18 converters: two groups of four warps that take alternate stages; thread = one weight row
//               of the tile (its TMEM lane).  With packed 4-bit ACTIVATIONS in the launch (the reference
//               operator API's input format; token tiles are then 128 rows) the group also expands the
//               stage's packed activation rows into the swizzled int8 operand tile in shared memory.
//
// Barrier protocol (mbarriers).  wfull[s] "the weights of stage s (and packed activations, which the converters
// expand) have landed"; xfull[s] "the activation tile of stage s has landed"; empty[s] "stage s may be refilled"
// = the MMAs of the stage have completed (tcgen05.commit) and the stage's converter group has read its packed
// operands.  Every barrier completes once per use of its stage, whatever the tile's scheme, so parities follow
// from the stage counter and no waiter can be lapped.  A slot s of tensor memory needs no barrier of its own:
// wfull[s] completes only after the producer saw empty[s] of the previous use, i.e. after the MMAs that read
// the slot.  Named barriers: 1 + s "stage s is ready": the MMA warp syncs on it, the watcher arrives once the
// activation tile is there, and the stage's converter group arrives itself as soon as the converted weights
// are in tensor memory (no mbarrier and no third warp between the conversion and the MMA: the time from "weights
// landed" to "MMA issued" is on the critical path of the ring, which is latency bound).  The weights have a
// barrier of their own so that the conversion starts when the 4-16 KiB of weights are there, not when the
// 22 KiB activation tile is.  6 + b "accumulator b is drained" (epilogue warps arrive, MMA warp syncs).  Every
// mbarrier wait is bounded (1 s of %globaltimer); a role whose wait ran out raises the abort flag and keeps
// walking its loop without waiting or working, so that every bar.arrive another warp counts on is still made
// and the kernel ends.
#include "gg_common.cuh"

namespace mxb {

using namespace ptx;
using namespace ggc;

namespace {

constexpr int kWSlotBytes  = kWT * kRowBytes;   // 16 KiB: plain weights, or 8 / 4 KiB of packed ones
constexpr int kEpiStageS   = 2048;              // per epilogue warp: 16 token pairs x 32 channels x 4 bytes
// Converter warps: groups of four (one warp per TMEM lane quarter) that take the stages in turn.  Measured on
// 8 x [4096, 2816, 2048]: one group w4a4 1815 / w4a16 725 TFLOP/s, two groups 1974 / 924, three groups - / 830;
// 8- and 16-bit tiles of a launch that also holds 4-bit weights lose 4-7 % per group that is present.
constexpr int kCvtWarps    = 8;
constexpr int kCvtGroups   = kCvtWarps / 4;
constexpr uint32_t kASlotCols = 32;             // TMEM columns of one converted K block (128 bytes of K per channel)
constexpr int kCvtGroup    = 4;                 // warps per converter group (one per TMEM lane quarter)
constexpr int kEpiWarps    = 8;                 // two per TMEM lane quarter (warps 2-5 and 7-10)

// Two geometries of the same kernel.  Large: token tiles of up to 176 rows, ring of 5 stages - for launches
// with compute-bound problems.  Small: token tiles of up to 32 rows, ring of 10 stages - for launches whose
// problems all have few rows (decode): what matters there is how many weight bytes are in flight per SM, and a
// stage of such a tile carries only 4-16 KiB of weights.
// kTwo (32-token tiles of launches with 4-bit weights): a stage holds TWO K blocks of a problem with 4-bit weights
// (16 KiB of packed w4a4 weights, 8 KiB of w4a16, 8 KiB of activations), ring of 7 stages: the hand-offs of a stage
// cost the same 500-600 cycles whatever it carries, and a 32-token tile has nothing else to pay them with.
template <bool kSmall, bool kTwo = false>
struct Geo {
  static_assert(!kTwo || kSmall, "two K blocks per stage: 32-token tiles only");
  static constexpr int kTok        = kSmall ? 32 : kTT;          // tokens per tile (tcgen05 N, any multiple of 16 up to this)
  static constexpr int kStages     = kSmall ? (kTwo ? 7 : 10) : 5;
  static constexpr int kKbPerStage = kTwo ? 2 : 1;
  static constexpr uint32_t kASlotStride = kASlotCols * kKbPerStage;   // TMEM columns of the A slot of one stage
  static constexpr int kEpiBufs    = kSmall ? 4 : kEpiWarps;     // transpose buffers: a 32-token tile has one chunk, the second warp of a quarter never stores
  static constexpr int kXSlotBytes = kTok * kRowBytes * kKbPerStage;   // 22 KiB / 4 KiB / 8 KiB
  static constexpr int kStageBytes = kWSlotBytes + kXSlotBytes;
  static constexpr int kRingBytes  = kStages * kStageBytes;      // 190 KiB / 200 KiB
  static constexpr uint32_t kAccCols   = kTok;                   // TMEM columns per accumulator
  static constexpr uint32_t kASlotCol0 = 2 * kTok;               // A slot s (one per ring stage) at kASlotCol0 + 32 s
  static constexpr int kBarStage0 = 1;                           // named barriers 1 .. kStages: stage s is ready
  static constexpr int kBarAcc0   = 1 + kStages;                 // two more: accumulator b is drained
  static constexpr int kBarEpi0   = 3 + kStages;                 // two per group of four epilogue warps (row-wide stores)
  static constexpr int kEpiGroups = kEpiBufs / 4;
  static_assert(kASlotCol0 + kStages * kASlotStride <= 512, "tensor memory budget");
  static_assert(kBarEpi0 + 2 * kEpiGroups - 1 <= 15, "named barrier budget");
  static_assert((kTok + 32) % 8 == 0, "sa_stage rows must stay 16-byte aligned");
};

constexpr int kFirstCvtWarp = 11;
constexpr int kAccBarThreads = kEpiWarps * 32 + 32;   // "accumulator drained": epilogue warps arrive, MMA warp syncs

template <int kMode, bool kPair = false>
struct CfgS {
  static constexpr int kThreads = kFirstCvtWarp * 32 + (kMode ? kCvtWarps * 32 : 0);
  // threads that meet at a "stage s is ready" named barrier: MMA warp + watcher (+ one converter group; in a CTA
  // pair the converters of both CTAs report to an mbarrier of the leader that its watcher forwards)
  static constexpr int kStageBarThreads = 64 + ((kMode && !kPair) ? kCvtGroup * 32 : 0);
};

// What every role needs to know about one tile, precomputed once per CTA: looking a tile up in the
// scheduling tables is a chain of dependent shared-memory loads, each of which takes hundreds of cycles
// while the tensor core streams operands from shared memory.
struct TileRec {
  int pk;       // problem | scheme << 8 | k-blocks << 12
  int x_row;    // buffer row of the tile's first token (A and scale_a)
  int nt;       // channel tile | tokens in the tile (1 .. kTT) << 16
  int c_row;    // row of C of the tile's first token
};
constexpr int kMaxRecs = 512;   // tiles per CTA kept in the table; later ones are looked up on the fly

struct TileS {
  int p, scheme, nkb, x_row, n_tile, ntok, c_row;
  int odd;   // stages of two K blocks: the last stage holds one
};

template <typename G>
struct CtrlS {
  uint64_t wfull[G::kStages];
  uint64_t xfull[G::kStages];
  uint64_t empty[G::kStages];
  uint64_t tfull[2];
  uint64_t cvtdone[G::kStages];   // CTA pairs, leader's instance: the converters of both CTAs have filled A slot s
  uint64_t tempty[2];             // CTA pairs, leader's instance: both CTAs have drained accumulator b
  uint32_t tmem_base;
  int abort_flag;
  int pad[2];
  Sched sched;
  alignas(16) __half sa_stage[kEpiWarps][G::kTok + 32];   // per epilogue warp: per-token scales of the current tile (read 16 bytes at a time)
  alignas(16) TileRec recs[kMaxRecs];
};

template <typename G>
constexpr int smem_bytes_swap() { return 1024 + G::kRingBytes + G::kEpiBufs * kEpiStageS + (int)sizeof(CtrlS<G>); }

static_assert(smem_bytes_swap<Geo<false>>() <= 232448 && smem_bytes_swap<Geo<true>>() <= 232448 &&
                  smem_bytes_swap<Geo<true, true>>() <= 232448,
              "dynamic shared memory of one CTA (227 KiB)");

__device__ __forceinline__ void report_s(GGStatus* status, int role, int tile) {
  atomicCAS(&status->error, 0, kDevErrTimeout);
  atomicCAS(&status->where, 0, (role << 24) | tile);
}

__device__ __forceinline__ bool is_int_scheme(int s) { return s != SCH_FP16 && s != SCH_W4A16G128; }
__device__ __forceinline__ bool is_cvt_scheme(int s) { return s == SCH_W4A4_XA || s == SCH_W4A16G128 || s == SCH_W4A4; }

// Per-role cycle counters (mxmoe_gg_profile) are compiled in with -DMXMOE_PROF only: every tick is a branch inside
// the per-stage loops of the producer and of the MMA warp, which are on the critical path of the ring.
#ifdef MXMOE_PROF
__device__ __forceinline__ long long tick(bool on) { return on ? clock64() : 0ll; }
#else
__device__ __forceinline__ long long tick(bool) { return 0ll; }
#endif

// bytes per stage of a weight tile and its coordinates (x step per K block, y) in the weight tensor map
__device__ __forceinline__ void weight_coords(int scheme, int w_row, uint32_t& wbytes, int& wx_step, int& wy) {
  constexpr uint32_t kFull = kWT * kRowBytes;   // 128 channels x 128 bytes of K
  if (scheme == SCH_W8A8)         { wbytes = kFull;     wx_step = 128; wy = w_row; }
  else if (scheme == SCH_FP16)    { wbytes = kFull;     wx_step = 64;  wy = w_row; }
  else if (scheme == SCH_W4A4_XA || scheme == SCH_W4A4) { wbytes = kFull / 2; wx_step = 64;  wy = w_row; }   // 64 packed bytes per row
  else                            { wbytes = kFull / 4; wx_step = 128; wy = w_row / 4; }   // w4a16: 32 packed rows x 128 B
}

// `pair_rank` >= 0: the schedule counts channel tiles of 256 (a CTA pair); this CTA takes the pair_rank-th half
__device__ __forceinline__ TileRec make_rec(const Sched* sc, int count, int t, int tok, int tok_packed, int pair_rank = -1) {
  Tile ti            = find_tile(sc, count, t);
  if (pair_rank >= 0) ti.n_tile = 2 * ti.n_tile + pair_rank;
  const int tile_tok = ti.scheme == SCH_W4A4 ? tok_packed : tok;   // problems with packed activations: shorter tiles
  TileRec r;
  r.pk     = ti.p | (ti.scheme << 8) | (ti.nkb << 12) | (ti.odd << 30);
  r.x_row  = sc->row0[ti.p] + ti.m_tile * tile_tok;
  r.nt     = ti.n_tile | (min(tile_tok, sc->m_eff[ti.p] - ti.m_tile * tile_tok) << 16);
  r.c_row  = r.x_row + sc->c_shift[ti.p];
  return r;
}
__device__ __forceinline__ TileS decode_rec(const TileRec& r) {
  TileS t;
  t.p = r.pk & 0xff; t.scheme = (r.pk >> 8) & 15; t.nkb = (r.pk >> 12) & 0x3FFFF; t.odd = (r.pk >> 30) & 1;
  t.x_row = r.x_row; t.n_tile = r.nt & 0xffff; t.ntok = r.nt >> 16; t.c_row = r.c_row;
  return t;
}

// named barriers (ids in Geo): stage s is ready (watcher and the stage's converter group -> MMA warp);
// accumulator b is drained (epilogue warps -> MMA warp)
__device__ __forceinline__ void nbar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void nbar_arrive(int id, int nthreads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Optional per-stage timeline of CTA 0 (compile with -DMXMOE_TRACE; debugging aid, not built by default): the clock
// at which each role passed a point of stage `it` (stages counted from the start of the launch).
#ifdef MXMOE_TRACE
constexpr int kTraceEvents = 8, kTraceLen = 512;
__device__ long long g_trace[kTraceEvents][kTraceLen];
#define TRACE(ev, it) do { if (blockIdx.x == 0 && (it) < kTraceLen) g_trace[ev][it] = clock64(); } while (0)
#else
#define TRACE(ev, it) do { } while (0)
#endif
enum { TR_PROD_GOT = 0, TR_PROD_ISSUED, TR_CVT_GOT, TR_CVT_DONE, TR_WATCH, TR_MMA_GOT, TR_MMA_ISSUED, TR_EPI };

__device__ __forceinline__ void sts16(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((unsigned short)v) : "memory");
}
// one row of the output tile, shared memory -> global memory (this GPU's or a peer's), by the copy engine
__device__ __forceinline__ void bulk_store_row(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

}  // namespace

// One pipeline stage = four MMAs (32 bytes of K each) and the commit that releases the stage, as ONE block of
// straight-line PTX: the issuing warp shares its scheduler with an epilogue warp and converter warps of the same
// TMEM lane quarter, so every instruction it does not need (a predicate set-up per MMA, descriptor arithmetic
// recomputed per stage) delays the issue of the next stage.  `first` == 0: the first MMA overwrites D.
//   kV 0 int8 / weights from shared memory, 1 fp16 / shared memory, 2 int8 / tensor memory, 3 fp16 / tensor memory.
#define MXB_COMMIT1 "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n\t"
#define MXB_MMA_STAGE_SS(KIND)                                                                              \
  asm volatile(                                                                                             \
      "{\n\t"                                                                                               \
      ".reg .pred p, t;\n\t"                                                                                \
      ".reg .b64 w0, w1, w2, w3, x0, x1, x2, x3;\n\t"                                                       \
      ".reg .b32 a1, a2, a3, b1, b2, b3;\n\t"                                                               \
      "setp.ne.b32 p, %5, 0;\n\t"                                                                           \
      "setp.eq.b32 t, 0, 0;\n\t"                                                                            \
      "add.u32 a1, %1, 2;  add.u32 a2, %1, 4;  add.u32 a3, %1, 6;\n\t"                                      \
      "add.u32 b1, %2, 2;  add.u32 b2, %2, 4;  add.u32 b3, %2, 6;\n\t"                                      \
      "mov.b64 w0, {%1, %3}; mov.b64 w1, {a1, %3}; mov.b64 w2, {a2, %3}; mov.b64 w3, {a3, %3};\n\t"         \
      "mov.b64 x0, {%2, %3}; mov.b64 x1, {b1, %3}; mov.b64 x2, {b2, %3}; mov.b64 x3, {b3, %3};\n\t"         \
      "tcgen05.mma.cta_group::1.kind::" KIND " [%0], w0, x0, %4, p;\n\t"                                    \
      "tcgen05.mma.cta_group::1.kind::" KIND " [%0], w1, x1, %4, t;\n\t"                                    \
      "tcgen05.mma.cta_group::1.kind::" KIND " [%0], w2, x2, %4, t;\n\t"                                    \
      "tcgen05.mma.cta_group::1.kind::" KIND " [%0], w3, x3, %4, t;\n\t"                                    \
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n\t"                     \
      "}"                                                                                                   \
      :                                                                                                     \
      : "r"(d_tmem), "r"(wlo), "r"(xlo), "r"(desc_hi), "r"(idesc), "r"(first), "r"(empty_bar)               \
      : "memory")
#define MXB_MMA_STAGE_TS(KIND, COMMIT)                                                                      \
  asm volatile(                                                                                             \
      "{\n\t"                                                                                               \
      ".reg .pred p, t;\n\t"                                                                                \
      ".reg .b64 x0, x1, x2, x3;\n\t"                                                                       \
      ".reg .b32 a1, a2, a3, b1, b2, b3;\n\t"                                                               \
      "setp.ne.b32 p, %5, 0;\n\t"                                                                           \
      "setp.eq.b32 t, 0, 0;\n\t"                                                                            \
      "add.u32 a1, %1, 8;  add.u32 a2, %1, 16;  add.u32 a3, %1, 24;\n\t"                                    \
      "add.u32 b1, %2, 2;  add.u32 b2, %2, 4;  add.u32 b3, %2, 6;\n\t"                                      \
      "mov.b64 x0, {%2, %3}; mov.b64 x1, {b1, %3}; mov.b64 x2, {b2, %3}; mov.b64 x3, {b3, %3};\n\t"         \
      "tcgen05.mma.cta_group::1.kind::" KIND " [%0], [%1], x0, %4, p;\n\t"                                  \
      "tcgen05.mma.cta_group::1.kind::" KIND " [%0], [a1], x1, %4, t;\n\t"                                  \
      "tcgen05.mma.cta_group::1.kind::" KIND " [%0], [a2], x2, %4, t;\n\t"                                  \
      "tcgen05.mma.cta_group::1.kind::" KIND " [%0], [a3], x3, %4, t;\n\t"                                  \
      COMMIT                                                                                                \
      "}"                                                                                                   \
      :                                                                                                     \
      : "r"(d_tmem), "r"(a_tmem), "r"(xlo), "r"(desc_hi), "r"(idesc), "r"(first), "r"(empty_bar)            \
      : "memory")

// The same for a CTA pair: one M = 256 MMA over both CTAs' weights and token halves, and a commit that arrives at
// the "stage may be refilled" barrier of both CTAs.
#define MXB_MMA_STAGE_SS2(KIND)                                                                             \
  asm volatile(                                                                                             \
      "{\n\t"                                                                                               \
      ".reg .pred p, t;\n\t"                                                                                \
      ".reg .b64 w0, w1, w2, w3, x0, x1, x2, x3;\n\t"                                                       \
      ".reg .b32 a1, a2, a3, b1, b2, b3;\n\t"                                                               \
      "setp.ne.b32 p, %5, 0;\n\t"                                                                           \
      "setp.eq.b32 t, 0, 0;\n\t"                                                                            \
      "add.u32 a1, %1, 2;  add.u32 a2, %1, 4;  add.u32 a3, %1, 6;\n\t"                                      \
      "add.u32 b1, %2, 2;  add.u32 b2, %2, 4;  add.u32 b3, %2, 6;\n\t"                                      \
      "mov.b64 w0, {%1, %3}; mov.b64 w1, {a1, %3}; mov.b64 w2, {a2, %3}; mov.b64 w3, {a3, %3};\n\t"         \
      "mov.b64 x0, {%2, %3}; mov.b64 x1, {b1, %3}; mov.b64 x2, {b2, %3}; mov.b64 x3, {b3, %3};\n\t"         \
      "tcgen05.mma.cta_group::2.kind::" KIND " [%0], w0, x0, %4, p;\n\t"                                    \
      "tcgen05.mma.cta_group::2.kind::" KIND " [%0], w1, x1, %4, t;\n\t"                                    \
      "tcgen05.mma.cta_group::2.kind::" KIND " [%0], w2, x2, %4, t;\n\t"                                    \
      "tcgen05.mma.cta_group::2.kind::" KIND " [%0], w3, x3, %4, t;\n\t"                                    \
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%6], %7;\n\t" \
      "}"                                                                                                   \
      :                                                                                                     \
      : "r"(d_tmem), "r"(wlo), "r"(xlo), "r"(desc_hi), "r"(idesc), "r"(first), "r"(empty_bar),              \
        "h"((unsigned short)3)                                                                              \
      : "memory")
#define MXB_MMA_STAGE_TS2(KIND)                                                                             \
  asm volatile(                                                                                             \
      "{\n\t"                                                                                               \
      ".reg .pred p, t;\n\t"                                                                                \
      ".reg .b64 x0, x1, x2, x3;\n\t"                                                                       \
      ".reg .b32 a1, a2, a3, b1, b2, b3;\n\t"                                                               \
      "setp.ne.b32 p, %5, 0;\n\t"                                                                           \
      "setp.eq.b32 t, 0, 0;\n\t"                                                                            \
      "add.u32 a1, %1, 8;  add.u32 a2, %1, 16;  add.u32 a3, %1, 24;\n\t"                                    \
      "add.u32 b1, %2, 2;  add.u32 b2, %2, 4;  add.u32 b3, %2, 6;\n\t"                                      \
      "mov.b64 x0, {%2, %3}; mov.b64 x1, {b1, %3}; mov.b64 x2, {b2, %3}; mov.b64 x3, {b3, %3};\n\t"         \
      "tcgen05.mma.cta_group::2.kind::" KIND " [%0], [%1], x0, %4, p;\n\t"                                  \
      "tcgen05.mma.cta_group::2.kind::" KIND " [%0], [a1], x1, %4, t;\n\t"                                  \
      "tcgen05.mma.cta_group::2.kind::" KIND " [%0], [a2], x2, %4, t;\n\t"                                  \
      "tcgen05.mma.cta_group::2.kind::" KIND " [%0], [a3], x3, %4, t;\n\t"                                  \
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%6], %7;\n\t" \
      "}"                                                                                                   \
      :                                                                                                     \
      : "r"(d_tmem), "r"(a_tmem), "r"(xlo), "r"(desc_hi), "r"(idesc), "r"(first), "r"(empty_bar),           \
        "h"((unsigned short)3)                                                                              \
      : "memory")

// kCommit = false (weights from tensor memory, single CTAs): the first K block of a stage that holds two
template <int kV, bool kPair, bool kCommit = true>
__device__ __forceinline__ void mma_stage(uint32_t d_tmem, uint32_t wlo, uint32_t a_tmem, uint32_t xlo, uint32_t desc_hi,
                                          uint32_t idesc, uint32_t first, uint32_t empty_bar) {
  if (kPair) {
    if (kV == 0)      { MXB_MMA_STAGE_SS2("i8"); }
    else if (kV == 1) { MXB_MMA_STAGE_SS2("f16"); }
    else if (kV == 2) { MXB_MMA_STAGE_TS2("i8"); }
    else              { MXB_MMA_STAGE_TS2("f16"); }
  } else {
    if (kV == 0)      { MXB_MMA_STAGE_SS("i8"); }
    else if (kV == 1) { MXB_MMA_STAGE_SS("f16"); }
    else if (kV == 2) { if (kCommit) { MXB_MMA_STAGE_TS("i8", MXB_COMMIT1); } else { MXB_MMA_STAGE_TS("i8", ""); } }
    else              { if (kCommit) { MXB_MMA_STAGE_TS("f16", MXB_COMMIT1); } else { MXB_MMA_STAGE_TS("f16", ""); } }
  }
}

// The MMA warp's main loop over the K blocks of one tile, specialised on the operand kind and on where
// the weights come from so that the issue sequence of a stage is straight-line code: a branch per MMA made the
// issue of every MMA several times slower.  All lanes walk the loop and meet the named barrier of each
// stage; the elected lane issues.  One MMA consumes 32 bytes of K per row: 8 TMEM columns of A or 32 bytes of a
// shared-memory row.  The per-stage addresses (descriptor low words, A slot, barrier) are carried in registers and
// advanced by their strides.
struct MmaCursor {
  int stage;
  uint32_t wlo, xlo, a_tmem, ebar;
};
// `last_nb`: K blocks in the last stage of the tile (stages of two K blocks, weights from tensor memory: 1 or 2;
// otherwise 1): every other stage of such a tile holds two, issued as 4 + 4 MMAs and one commit.
template <int kV, typename G, int kBarThreads, bool kPair>
__device__ __forceinline__ void mma_tile_loop(int nkb, int last_nb, MmaCursor& c, const MmaCursor& c0, int lane,
                                              uint32_t d_tmem, uint32_t idesc, uint32_t desc_hi, int& sidx) {
  constexpr bool kTwo = G::kKbPerStage == 2 && kV >= 2;
  for (int kb = 0; kb < nkb; ++kb) {
    nbar_sync(G::kBarStage0 + c.stage, kBarThreads);   // operands of this stage are in place
    if (lane == 0) TRACE(TR_MMA_GOT, sidx);
    if (elect_one_sync()) {
      tc_fence_after_sync();
      if (kTwo && (kb + 1 < nkb || last_nb == 2)) {
        mma_stage<kV, kPair, false>(d_tmem, c.wlo, c.a_tmem, c.xlo, desc_hi, idesc, kb > 0 ? 1u : 0u, c.ebar);
        mma_stage<kV, kPair>(d_tmem, c.wlo, c.a_tmem + kASlotCols, c.xlo + ((G::kTok * kRowBytes) >> 4), desc_hi, idesc,
                             1u, c.ebar);
      } else {
        mma_stage<kV, kPair>(d_tmem, c.wlo, c.a_tmem, c.xlo, desc_hi, idesc, kb > 0 ? 1u : 0u, c.ebar);
      }
    }
    __syncwarp();
    if (lane == 0) TRACE(TR_MMA_ISSUED, sidx);
    ++sidx;
    if (++c.stage == G::kStages) {
      c = c0;
    } else {
      c.wlo += G::kStageBytes >> 4; c.xlo += G::kStageBytes >> 4; c.a_tmem += G::kASlotStride; c.ebar += 8;
    }
  }
}

// kPair: two CTAs of a cluster work on 256 channels x one token tile.  Each loads (and converts) its own 128 weight
// rows and HALF of the token tile by its own plain TMA loads, the leader (cluster rank 0) issues one M = 256 MMA
// for both (tcgen05 cta_group::2), each drains its own accumulator: per MAC a CTA writes and reads half as many
// activation bytes in shared memory, which is what bounds the single-CTA form.  Cross-CTA signals: the token
// halves complete on the leader's xfull (the cta_group::2 form of the load only redirects the byte count),
// converters and epilogue warps of both CTAs arrive at the leader's cvtdone / tempty, the leader's commits arrive
// at empty / tfull of both CTAs.
// kExt: the launch holds problems with one of the optional result forms (silu(gate) * up, row-wide stores, rows at
// given addresses); its weight tensor maps then have rank 4.  Launches without them run the instance in which all of
// that is compiled out: the extra per-tile loads and per-chunk branches cost the plain launch 2-7 %.
template <int kMode, bool kSmall, bool kPair = false, bool kExt = false>
__global__ void __launch_bounds__(CfgS<kMode>::kThreads, 1)
gg_swap_kernel(const GGSwapProblemDev* __restrict__ problems, int count, GGStatus* __restrict__ status) {
  constexpr bool kTwo = kSmall && kMode == 1;   // stages of two K blocks for problems with 4-bit weights
  using G = Geo<kSmall, kTwo>;
  constexpr bool kCvt = kMode != 0;
  static_assert(!kPair || (!kSmall && kMode != 2), "CTA pairs: large tiles, activations in their final form");
  constexpr int kStageBar = CfgS<kMode, kPair>::kStageBarThreads;
  const int rank  = kPair ? (int)cluster_ctarank() : 0;                      // 0 = the CTA that issues the MMAs
  const int cta   = kPair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;       // this walker (CTA or CTA pair) ...
  const int nctas = kPair ? (int)(gridDim.x >> 1) : (int)gridDim.x;         // ... of so many
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzled tiles need 1024-byte alignment
  uint8_t* smem_gen        = smem_raw + (smem_base - smem_u32(smem_raw));
  CtrlS<G>* ctrl              = reinterpret_cast<CtrlS<G>*>(smem_gen + G::kRingBytes + G::kEpiBufs * kEpiStageS);
  const uint32_t epi_base  = smem_base + G::kRingBytes;
  Sched* sc                = &ctrl->sched;
  volatile int* abort_flag = &ctrl->abort_flag;

  const int tid  = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if (count > kMaxProblems) {
    if (tid == 0 && blockIdx.x == 0) atomicCAS(&status->error, 0, kDevErrTooMany);
    return;
  }

  auto load_w = [&](uint32_t dst, const void* map, uint32_t bar, int x, int y, int z) {
    if (kExt) tma_load_4d(dst, map, bar, x, y, 0, z);
    else      tma_load_2d(dst, map, bar, x, y);
  };
  auto wslot = [&](int s) { return smem_base + s * G::kStageBytes; };
  auto xslot = [&](int s) { return smem_base + s * G::kStageBytes + kWSlotBytes; };

  // ------------------------------------------------------------------ setup
  if (tid == 0) {
    for (int s = 0; s < G::kStages; ++s) {
      mbar_init(smem_u32(&ctrl->wfull[s]), 1);
      mbar_init(smem_u32(&ctrl->xfull[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1 + (kCvt ? kCvtGroup : 0));
      mbar_init(smem_u32(&ctrl->cvtdone[s]), 2 * kCvtGroup);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctrl->tfull[b]), 1);
      mbar_init(smem_u32(&ctrl->tempty[b]), 2 * kEpiWarps);
    }
    ctrl->abort_flag = 0;
    fence_mbar_init();
  }
  // problems with packed 4-bit activations use token tiles of at most 128 rows: the packed rows of a stage
  // (128 x 64 B) then fit behind the packed weights in the stage's weight slot
  constexpr int kTokPacked = G::kTok > 128 ? 128 : G::kTok;
  build_sched(sc, problems, count, G::kTok, kPair ? 2 * kWT : kWT, kTokPacked, kTwo);
  const int total_tiles = sc->total_tiles;
  const int my_tiles    = total_tiles > cta ? (total_tiles - cta + nctas - 1) / nctas : 0;
  const int pair_rank   = kPair ? rank : -1;
  for (int i = tid; i < my_tiles && i < kMaxRecs; i += blockDim.x)
    ctrl->recs[i] = make_rec(sc, count, cta + i * nctas, G::kTok, kTokPacked, pair_rank);
  auto tile_rec = [&](int i) -> TileRec {
    if (i < kMaxRecs) return ctrl->recs[i];
    return make_rec(sc, count, cta + i * nctas, G::kTok, kTokPacked, pair_rank);
  };
  if (warp == 1) {
    if (kPair) {
      tmem_alloc2(smem_u32(&ctrl->tmem_base), 512);
      tmem_relinquish2();
    } else {
      tmem_alloc(smem_u32(&ctrl->tmem_base), 512);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (kPair) cluster_sync_all();   // both CTAs' barriers exist before either signals the other's
  tc_fence_after_sync();

  const bool prof_on = status->prof_on != 0;   // per-role cycle counters wanted (costs a few percent)
  const uint64_t tmo = status->timeout_ms > 0 ? (uint64_t)status->timeout_ms * 1000000ull : kTimeoutNs;
  const int skip_stage = blockIdx.x == 0 ? status->skip_stage - 1 : -1;   // test hook, see GGStatus
  const long long prof_t0  = clock64();
  const uint32_t tmem_base = ctrl->tmem_base;

  // ------------------------------------------------------------------ roles
  if (warp == 0) {
    // ===== TMA producer =====
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long w_prod = 0;
      int n_stage = 0, n_tile = 0;
      const uint32_t empty0 = smem_u32(&ctrl->empty[0]), wfull0 = smem_u32(&ctrl->wfull[0]), xfull0 = smem_u32(&ctrl->xfull[0]);
      TileRec nrec = tile_rec(0);
      for (int i = 0; ok && i < my_tiles; ++i) {
        const int t    = cta + i * nctas;
        const TileS ti = decode_rec(nrec);
        if (i + 1 < my_tiles) nrec = tile_rec(i + 1);   // issued now, needed at the next tile
        const GGSwapProblemDev* pr = problems + ti.p;
        ++n_tile;
        const int ntok  = ti.ntok;
        const int x_row = ti.x_row;
        const int w_row = ti.n_tile * kWT;
        // long token tiles take one 176-row box, short ones only the 32-row boxes they need
        const bool big  = ntok > 4 * kXBoxSmall;
        const int nbox  = (ntok + kXBoxSmall - 1) / kXBoxSmall;
        const uint32_t xbytes = (kMode == 2 && ti.scheme == SCH_W4A4) ? (uint32_t)(nbox * kXBoxSmall * 64)
                                : big ? (uint32_t)G::kXSlotBytes : (uint32_t)(nbox * kXBoxSmall * kRowBytes);
        // weights: bytes per stage and coordinates in the weight tensor map
        uint32_t wbytes;
        int wx_step, wy;
        weight_coords(ti.scheme, w_row, wbytes, wx_step, wy);
        // silu(gate) * up problems: the box gathers 16 gate + 16 up rows four times; its origin is the tile's first
        // group of 16 columns of C (the weight maps have rank 4, see encode_w)
        int wz = 0;
        if (kExt && pr->silu_inter) { wz = ti.n_tile * 4; wy = 0; }
        const int xx_step = (ti.scheme == SCH_FP16 || ti.scheme == SCH_W4A16G128) ? 64 : 128;   // (packed int4: see below)
        // this tile's K block for which the test hook (GGStatus::skip_stage) announces more weight bytes than will
        // arrive.  A select, not a branch: one more branch per stage in these loops cost the w4a4 layer 3.5 %, and the
        // per-role cycle counters (two more) another 3.5 %; a second producer thread for the activation tiles was
        // measured too and is no faster than one lean loop.
        const int skip_kb = (skip_stage >= n_stage && skip_stage < n_stage + ti.nkb) ? skip_stage - n_stage : -1;
        const bool packed_x = kMode == 2 && ti.scheme == SCH_W4A4;
        if (kPair) {
          // this CTA's weights and its half of the token tile: rows [rank * npad / 2, +88) of the tile, one box.
          // The token halves of both CTAs complete on the leader's barrier, which the leader arms for both.
          constexpr uint32_t kXHalf = (uint32_t)(kTT / 2) * kRowBytes;
          const int xr = x_row + rank * (((ntok + 15) & ~15) >> 1);
          for (int kb = 0; kb < ti.nkb; ++kb) {
            const bool got = wait_bar(empty0 + 8 * stage, phase ^ 1u, abort_flag, 0, tmo);
            if (!got) { report_s(status, 1, t); ok = false; break; }
            if (kCvt) {
              mbar_expect_tx(wfull0 + 8 * stage, wbytes);
              load_w(wslot(stage), &pr->tmW, wfull0 + 8 * stage, kb * wx_step, wy, wz);
              if (rank == 0) mbar_expect_tx(xfull0 + 8 * stage, 2 * kXHalf);
            } else {
              if (rank == 0) mbar_expect_tx(xfull0 + 8 * stage, 2 * (wbytes + kXHalf));
              if (kExt) tma_load_4d_pair(wslot(stage), &pr->tmW, xfull0 + 8 * stage, kb * wx_step, wy, 0, wz);
              else      tma_load_2d_pair(wslot(stage), &pr->tmW, xfull0 + 8 * stage, kb * wx_step, wy);
            }
            tma_load_2d_pair(xslot(stage), &pr->tmXh, xfull0 + 8 * stage, kb * xx_step, xr);
            if (++stage == G::kStages) { stage = 0; phase ^= 1u; }
          }
        } else if (big && !packed_x) {
          // the common case (a full token tile), straight-line: wait, announce, two loads
          for (int kb = 0; kb < ti.nkb; ++kb) {
            const long long c0 = tick(prof_on);
            const bool got = wait_bar(empty0 + 8 * stage, phase ^ 1u, abort_flag, 0, tmo);
            w_prod += tick(prof_on) - c0;
            TRACE(TR_PROD_GOT, n_stage + kb);
            if (!got) { report_s(status, 1, t); ok = false; break; }
            mbar_expect_tx(wfull0 + 8 * stage, wbytes + (kb == skip_kb ? 16u : 0u));
            load_w(wslot(stage), &pr->tmW, wfull0 + 8 * stage, kb * wx_step, wy, wz);
            mbar_expect_tx(xfull0 + 8 * stage, xbytes);
            tma_load_2d(xslot(stage), &pr->tmX, xfull0 + 8 * stage, kb * xx_step, x_row);
            TRACE(TR_PROD_ISSUED, n_stage + kb);
            if (++stage == G::kStages) { stage = 0; phase ^= 1u; }
          }
        } else {
          for (int kb = 0; kb < ti.nkb; ++kb) {
            const long long c0 = tick(prof_on);
            const bool got = wait_bar(empty0 + 8 * stage, phase ^ 1u, abort_flag, 0, tmo);
            w_prod += tick(prof_on) - c0;
            if (!got) { report_s(status, 1, t); ok = false; break; }
            const uint32_t wbar = wfull0 + 8 * stage;
            const uint32_t bar  = xfull0 + 8 * stage;
            if (packed_x) {
              // packed activation rows (64 bytes of K each) go behind the packed weights; the converters expand them
              mbar_expect_tx(wbar, wbytes + xbytes);
              load_w(wslot(stage), &pr->tmW, wbar, kb * wx_step, wy, wz);
              for (int b = 0; b < nbox; ++b)
                tma_load_2d(wslot(stage) + kWSlotBytes / 2 + b * kXBoxSmall * 64, &pr->tmXs, wbar, kb * 64, x_row + b * kXBoxSmall);
              mbar_arrive(bar);                     // no activation tile of its own: complete the phase
            } else if (kTwo) {
              // stages of two K blocks for problems with 4-bit weights: K block 2 kb (+ 1 unless the tile's K ends
              // there), weights back to back in the weight slot, activations as [K block][32 rows][128 bytes]
              const int nb = (is_cvt_scheme(ti.scheme) && !(ti.odd && kb + 1 == ti.nkb)) ? 2 : 1;
              const int k0 = is_cvt_scheme(ti.scheme) ? 2 * kb : kb;
              mbar_expect_tx(wbar, wbytes * nb + (kb == skip_kb ? 16u : 0u));
              mbar_expect_tx(bar, xbytes * nb);
              for (int b = 0; b < nb; ++b) {
                load_w(wslot(stage) + b * wbytes, &pr->tmW, wbar, (k0 + b) * wx_step, wy, wz);
                tma_load_2d(xslot(stage) + b * G::kTok * kRowBytes, &pr->tmXs, bar, (k0 + b) * xx_step, x_row);
              }
            } else {
              mbar_expect_tx(wbar, wbytes + (kb == skip_kb ? 16u : 0u));
              load_w(wslot(stage), &pr->tmW, wbar, kb * wx_step, wy, wz);
              mbar_expect_tx(bar, xbytes);
              if (big) {
                tma_load_2d(xslot(stage), &pr->tmX, bar, kb * xx_step, x_row);
              } else {
                for (int b = 0; b < nbox; ++b)
                  tma_load_2d(xslot(stage) + b * kXBoxSmall * kRowBytes, &pr->tmXs, bar, kb * xx_step, x_row + b * kXBoxSmall);
              }
            }
            if (++stage == G::kStages) { stage = 0; phase ^= 1u; }
          }
        }
        n_stage += ti.nkb;
      }
      if (blockIdx.x == 0) {
        status->prof[PROF_PROD_WAIT] = w_prod;
        status->prof[PROF_TILES]     = n_tile;
        status->prof[PROF_STAGES]    = n_stage;
      }
    }
  } else if (warp == 1 && rank == 0) {
    // ===== MMA issuer (all lanes walk the loop and meet the named barriers, the elected lane issues) =====
    int acc = 0;
    long long w_oper = 0, w_acc = 0, w_issue = 0;
    int sidx = 0;   // stages issued so far (timeline tracing only)
    // stage 0: low words of the two shared-memory descriptors (the high word is the same for every tile of the
    // ring: 128-byte swizzle, 1024 bytes between 8-row groups), first A slot, first "stage may be refilled" barrier
    const uint64_t desc0 = smem_desc_sw128(smem_base);
    const uint32_t desc_hi = (uint32_t)(desc0 >> 32);
    MmaCursor cur0;
    cur0.stage  = 0;
    cur0.wlo    = (uint32_t)desc0;
    cur0.xlo    = (uint32_t)smem_desc_sw128(smem_base + kWSlotBytes);
    cur0.a_tmem = tmem_base + G::kASlotCol0;
    cur0.ebar   = smem_u32(&ctrl->empty[0]);
    MmaCursor cur = cur0;
    TileRec nrec = tile_rec(0);
    for (int i = 0; i < my_tiles; ++i) {
      const TileS ti = decode_rec(nrec);
      if (i + 1 < my_tiles) nrec = tile_rec(i + 1);   // issued now, needed at the next tile
      const long long ca = tick(prof_on);
      // the epilogue has drained this accumulator (tile i - 2); in a CTA pair both CTAs' epilogues have
      if (kPair) {
        if (i >= 2 && !warp_wait_bar(smem_u32(&ctrl->tempty[acc]), (uint32_t)((i >> 1) - 1) & 1u, abort_flag, lane, tmo)) {
          if (lane == 0) report_s(status, 2, cta + i * nctas);
          break;
        }
        tc_fence_after_sync();
      } else if (i >= 2) {
        nbar_sync(G::kBarAcc0 + acc, kAccBarThreads);
      }
      w_acc += tick(prof_on) - ca;
      const int npad        = (ti.ntok + 15) & ~15;
      const uint32_t d_tmem = tmem_base + acc * G::kAccCols;
      const bool is_int     = is_int_scheme(ti.scheme);
      const bool from_tmem  = kCvt && is_cvt_scheme(ti.scheme);
      constexpr int kMmaM   = kPair ? 2 * kWT : kWT;
      const uint32_t idesc  = is_int ? idesc_i8(kMmaM, npad) : idesc_f16(kMmaM, npad);
      const int variant     = (from_tmem ? 2 : 0) + (is_int ? 0 : 1);
      const int last_nb     = (kTwo && from_tmem && !ti.odd) ? 2 : 1;
      if (variant == 0)      mma_tile_loop<0, G, kStageBar, kPair>(ti.nkb, last_nb, cur, cur0, lane, d_tmem, idesc, desc_hi, sidx);
      else if (variant == 1) mma_tile_loop<1, G, kStageBar, kPair>(ti.nkb, last_nb, cur, cur0, lane, d_tmem, idesc, desc_hi, sidx);
      else if (variant == 2) mma_tile_loop<2, G, kStageBar, kPair>(ti.nkb, last_nb, cur, cur0, lane, d_tmem, idesc, desc_hi, sidx);
      else                   mma_tile_loop<3, G, kStageBar, kPair>(ti.nkb, last_nb, cur, cur0, lane, d_tmem, idesc, desc_hi, sidx);
      if (elect_one_sync()) {
        if (kPair) mma_commit2(smem_u32(&ctrl->tfull[acc]), 3);
        else       mma_commit(smem_u32(&ctrl->tfull[acc]));
      }
      __syncwarp();
      acc ^= 1;
    }
    // consume the "drained" arrivals of the last two tiles, so that no named barrier is left half-way
    if (!kPair)
      for (int i = max(my_tiles - 2, 0); i < my_tiles; ++i) nbar_sync(G::kBarAcc0 + (i & 1), kAccBarThreads);
    if (blockIdx.x == 0 && lane == 0) {
      status->prof[PROF_MMA_WAIT_OPER] = w_oper;
      status->prof[PROF_MMA_WAIT_ACC]  = w_acc;
      status->prof[PROF_MMA_ISSUE]     = w_issue;
    }
  } else if (warp == 1) {
    // (the second CTA of a pair issues nothing)
  } else if (warp < 6 || (warp > 6 && warp < kFirstCvtWarp)) {
    // ===== epilogue (TMEM lane quarter = warp % 4; lane = output channel, columns = tokens) =====
    // warps 2-5 take the even 32-token chunks of a tile, warps 7-10 the odd ones
    const int q    = warp & 3;
    const int half = warp > 6 ? 1 : 0;
    const int ew   = half ? warp - 7 + 4 : warp - 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    __half* saw        = ctrl->sa_stage[ew];
    const uint32_t stg = epi_base + ew * kEpiStageS;
    long long w_epi = 0, w_store = 0;
    bool dead = false;   // a wait ran out: walk the remaining tiles without waiting or working
    TileRec nrec = tile_rec(0);
    for (int i = 0; i < my_tiles; ++i) {
      const int t    = cta + i * nctas;
      const TileS ti = decode_rec(nrec);
      if (i + 1 < my_tiles) nrec = tile_rec(i + 1);   // issued now, needed at the next tile
      const GGSwapProblemDev* pr = problems + ti.p;
      const int ntok      = ti.ntok;
      const int64_t grow0 = ti.x_row;   // buffer row of token 0 of the tile (A, scale_a)
      const int64_t crow0 = ti.c_row;   // its row in C
      const int N = pr->N, ldc = pr->ldc, out_mode = pr->out_mode;
      const bool bulk     = kExt && pr->bulk_out != 0;
      const int64_t* row_ptrs = kExt ? pr->c_row_ptrs : nullptr;
      const int silu      = kExt ? pr->silu_inter : 0;   // > 0: lanes 0-15 of the warp hold gate rows, lanes 16-31 the up rows of the same 16 columns of C
      const bool is_int   = is_int_scheme(ti.scheme);
      const int acc_shift = (ti.scheme == SCH_W4A4 || ti.scheme == SCH_W4A4_XA) ? 8 : 0;   // codes ride in the high nibbles
      const int c_col     = ti.n_tile * (kWT / 2) + q * 16 + (lane & 15);                   // silu: this thread's column of C
      const int n_ch      = silu ? (lane >> 4) * silu + c_col : ti.n_tile * kWT + q * 32 + lane;   // this thread's channel (weight row)
      __half2 sb2 = __float2half2_rn(0.f);
      if (!dead && is_int && out_mode != OUT_ACC && half * 32 < ntok) {
        // everything that does not depend on the accumulator is fetched before waiting for it
        if (n_ch < N) sb2 = __half2half2(__ldg(pr->scale_b + n_ch));
        __syncwarp();
        for (int i = lane; i < G::kTok + 32; i += 32)
          saw[i] = (i < ntok) ? pr->scale_a[(grow0 + i) * pr->sa_stride] : __float2half(0.f);
        __syncwarp();
      }
      const long long c0 = tick(prof_on);
      if (!dead) {
        // ONE epilogue warp polls the accumulator's mbarrier, the other seven wait for it at a named barrier (a
        // tile keeps them waiting for thousands of cycles; eight polling warps are eight streams of try_wait)
        if (ew == 0) {
          const bool ok = warp_wait_bar(smem_u32(&ctrl->tfull[acc]), acc_phase, abort_flag, lane, tmo);
          if (lane == 0) ctrl->pad[0] = ok ? 1 : 0;
          __syncwarp();
        }
        nbar_sync(15, kEpiWarps * 32);
        const bool ok = *reinterpret_cast<volatile int*>(&ctrl->pad[0]) != 0;
        if (!ok) {
          if (lane == 0 && ew == 0) report_s(status, 4, t);
          dead = true;
        }
      }
      if (dead) {
        // keep the MMA warp's bar.sync on this accumulator balanced, do nothing else
        if (kPair) { if (lane == 0) mbar_arrive_leader_relaxed(smem_u32(&ctrl->tempty[acc])); }
        else nbar_arrive(G::kBarAcc0 + acc, kAccBarThreads);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
        continue;
      }
      const long long c1 = tick(prof_on);
      w_epi += c1 - c0;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * G::kAccCols + ((uint32_t)(q * 32) << 16);
      const int nchunk     = (ntok + 31) >> 5;
      // read one transposed chunk back and store it: lane -> (token pair, 8 channels), 16-byte stores
      auto store_chunk = [&](uint32_t buf, int ch) {
        const int p8 = lane & 3;   // which 8 channels of the warp's 32
#pragma unroll
        for (int rd = 0; rd < 2; ++rd) {
          const int tp   = (lane >> 2) + 8 * rd;
          const uint4 a0 = lds128(buf + tp * 128 + (((2 * p8) ^ (tp & 7)) << 4));
          const uint4 a1 = lds128(buf + tp * 128 + (((2 * p8 + 1) ^ (tp & 7)) << 4));
          uint4 lo, hi;   // lo: token 2*tp, hi: token 2*tp + 1; 8 consecutive channels each
          lo.x = __byte_perm(a0.x, a0.y, 0x5410); hi.x = __byte_perm(a0.x, a0.y, 0x7632);
          lo.y = __byte_perm(a0.z, a0.w, 0x5410); hi.y = __byte_perm(a0.z, a0.w, 0x7632);
          lo.z = __byte_perm(a1.x, a1.y, 0x5410); hi.z = __byte_perm(a1.x, a1.y, 0x7632);
          lo.w = __byte_perm(a1.z, a1.w, 0x5410); hi.w = __byte_perm(a1.z, a1.w, 0x7632);
          const int tk   = ch * 32 + 2 * tp;
          const int ncol = ti.n_tile * kWT + q * 32 + 8 * p8;
          __half* dst    = reinterpret_cast<__half*>(pr->C) + (crow0 + tk) * ldc + ncol;
          if (ncol < N) {
            if (tk < ntok) *reinterpret_cast<uint4*>(dst) = lo;
            if (tk + 1 < ntok) *reinterpret_cast<uint4*>(dst + ldc) = hi;
          }
        }
      };
#pragma unroll 1
      for (int ch = half; ch < nchunk; ch += 2) {
        // row-wide stores to per-row addresses: this lane's row of the chunk, fetched before the accumulator load
        int64_t row_ptr = 0;
        if (row_ptrs && lane < 8 && ch * 32 + q * 8 + lane < ntok) row_ptr = __ldg(row_ptrs + crow0 + ch * 32 + q * 8 + lane);
        uint32_t v[32];
        tmem_ld_32x32(taddr + ch * 32, v);
        tmem_ld_wait();
        if (out_mode == OUT_ACC) {
          // raw accumulators (int32 / fp32): element (token, channel), used by the bit-exactness tests
          uint32_t* dst = reinterpret_cast<uint32_t*>(pr->C);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int tk = ch * 32 + j;
            if (tk < ntok && n_ch < N)
              dst[(crow0 + tk) * ldc + n_ch] = is_int ? (uint32_t)((int)v[j] >> acc_shift) : v[j];
          }
          continue;
        }
        // fp16 results of this channel for 32 tokens, two tokens per word
        uint32_t h[16];
        if (is_int) {
          // C = fp16_rn( float(acc) * float( fp16_rn(sa * sb) ) )   (mm_tile.cuh:490-493)
          // (loading the chunk's scales before waiting for the accumulator load was measured slower)
          const uint4* sap = reinterpret_cast<const uint4*>(saw + ch * 32);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const uint4 sv    = sap[g];
            const __half2* s2 = reinterpret_cast<const __half2*>(&sv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int j    = g * 4 + e;
              const float2 p = __half22float2(__hmul2(s2[e], sb2));
              const float f0 = (float)((int)v[2 * j] >> acc_shift) * p.x;
              const float f1 = (float)((int)v[2 * j + 1] >> acc_shift) * p.y;
              __half2 r      = __floats2half2_rn(f0, f1);
              h[j]           = *reinterpret_cast<uint32_t*>(&r);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            __half2 r = __floats2half2_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
            h[j]      = *reinterpret_cast<uint32_t*>(&r);
          }
        }
        if (silu) {
          // h = fp16( fp16(silu(gate)) * up ) on the fp16 results, the arithmetic of the stand-alone silu-mul kernel.
          // The gate lane keeps tokens 0-15 of the chunk and gets their up values; the up lane gets the gate values
          // of tokens 16-31: eight exchanges, then each lane finishes 16 tokens of its column and stores them.
          const bool up = lane >= 16;
          uint32_t other[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) other[i] = __shfl_xor_sync(0xffffffffu, up ? h[i] : h[8 + i], 16);
          __half* dst = reinterpret_cast<__half*>(pr->C) + (crow0 + ch * 32 + (up ? 16 : 0)) * ldc + c_col;
          const int tk0 = ch * 32 + (up ? 16 : 0);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t gw = up ? other[i] : h[i], uw = up ? h[8 + i] : other[i];
            const float2 gf   = __half22float2(*reinterpret_cast<const __half2*>(&gw));
            const float s0    = __fdividef(gf.x, 1.f + __expf(-gf.x));
            const float s1    = __fdividef(gf.y, 1.f + __expf(-gf.y));
            const __half2 r   = __hmul2(__floats2half2_rn(s0, s1), *reinterpret_cast<const __half2*>(&uw));
            if (c_col < silu) {
              if (tk0 + 2 * i < ntok) dst[(2 * i) * ldc] = __low2half(r);
              if (tk0 + 2 * i + 1 < ntok) dst[(2 * i + 1) * ldc] = __high2half(r);
            }
          }
          continue;
        }
        if (bulk) {
          // Row-wide stores: the four warps of a group (one per TMEM lane quarter) lay the chunk down as 32 token
          // rows of 256 bytes (128 channels) in their joint 8 KiB buffer and hand every row to the copy engine as
          // one piece.  This is the form for outputs that cross NVLink (the down projection of an expert-parallel
          // layer stores into the peers' buffers): 64-byte pieces from plain stores cost the launch 65 % more time.
          const uint32_t gb = epi_base + half * 4 * kEpiStageS;
          if (lane < 8) bulk_wait_read();                          // this thread's earlier rows have left the buffer
          nbar_sync(G::kBarEpi0 + 2 * half, 128);
          const uint32_t col = gb + (uint32_t)(q * 32 + lane) * 2;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            sts16(col + (2 * j) * 256, h[j]);
            sts16(col + (2 * j + 1) * 256, h[j] >> 16);
          }
          fence_proxy_async_smem();
          nbar_sync(G::kBarEpi0 + 2 * half + 1, 128);
          if (lane < 8) {
            const int row = q * 8 + lane, tk = ch * 32 + row;
            const int n0  = ti.n_tile * kWT;
            if (tk < ntok) {
              // the row's place: in C, or wherever the problem's table of row addresses says
              __half* dst = row_ptrs ? reinterpret_cast<__half*>(row_ptr) + n0
                                     : reinterpret_cast<__half*>(pr->C) + (crow0 + tk) * ldc + n0;
              bulk_store_row(dst, gb + row * 256, (uint32_t)min(kWT, N - n0) * 2u);
            }
            bulk_commit();
          }
          continue;
        }
        // transpose through the warp's 2 KiB buffer: row = token pair (128 bytes = 32 channels x 2 tokens),
        // 16-byte slots XOR-swizzled by the row so that writes and reads are conflict-free
        __syncwarp();   // the previous chunk's reads of the buffer are done
#pragma unroll
        for (int j = 0; j < 16; ++j) sts32(stg + j * 128 + (((lane >> 2) ^ (j & 7)) << 4) + (lane & 3) * 4, h[j]);
        __syncwarp();
        store_chunk(stg, ch);
      }
      tc_fence_before_sync();
      if (kPair) {
        __syncwarp();
        if (lane == 0) mbar_arrive_leader_relaxed(smem_u32(&ctrl->tempty[acc]));
      } else {
        nbar_arrive(G::kBarAcc0 + acc, kAccBarThreads);
      }
      w_store += tick(prof_on) - c1;
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (kExt && lane < 8) bulk_wait_all();   // rows handed to the copy engine have reached memory before the CTA ends
    if (blockIdx.x == 0 && warp == 2 && lane == 0) {
      status->prof[PROF_EPI_WAIT]  = w_epi;
      status->prof[PROF_EPI_STORE] = w_store;
    }
  } else if (warp == 6 && rank != 0) {
    // (the leader's watcher serves the pair)
  } else if (warp == 6) {
    // ===== watcher: forwards "stage ready" from the mbarriers to the MMA warp's named barriers =====
    int stage = 0;
    uint32_t phase = 0;
    bool dead = false;
    int wit = 0;   // stages forwarded so far (timeline tracing only)
    TileRec nrec = tile_rec(0);
    for (int i = 0; i < my_tiles; ++i) {
      const int t    = cta + i * nctas;
      const TileS ti = decode_rec(nrec);
      if (i + 1 < my_tiles) nrec = tile_rec(i + 1);
      for (int kb = 0; kb < ti.nkb; ++kb) {
        if (!dead) {
          // with converter warps in the CTA the stage's converter group waits for the weights (and arrives at the
          // named barrier itself); without them this warp does
          bool ok = warp_wait_bar(smem_u32(&ctrl->xfull[stage]), phase, abort_flag, lane, tmo);
          if (ok && !kCvt && !kPair) ok = warp_wait_bar(smem_u32(&ctrl->wfull[stage]), phase, abort_flag, lane, tmo);
          if (ok && kCvt && kPair) {   // the converter groups of both CTAs have filled their A slots
            ok = warp_wait_bar(smem_u32(&ctrl->cvtdone[stage]), phase, abort_flag, lane, tmo);
            tc_fence_after_sync();
          }
          if (!ok) {
            if (lane == 0) report_s(status, 3, t);
            dead = true;
          }
        }
        if (lane == 0) TRACE(TR_WATCH, wit);
        ++wit;
        nbar_arrive(G::kBarStage0 + stage, kStageBar);   // always: the MMA warp's bar.sync must complete
        if (++stage == G::kStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (kCvt) {
    // ===== converters: two groups of four warps take alternate stages, so that the chain of shared-memory
    // round trips of one stage (wait, load, store to tensor memory, arrive) overlaps the next stage's.
    // Thread = weight row (channel) 32*q + lane of the tile = its TMEM lane; it converts the row's 128 bytes
    // of K of the stage into A slot `stage`.  The slot is free when wfull[stage] has completed: the producer
    // refilled the stage only after the MMAs of its previous use (which read the slot) had completed.  When the
    // converted weights are in tensor memory the group arrives at the stage's named barrier itself.
    const int q     = warp & 3;               // TMEM lane quarter this warp may write
    const int group = (warp - kFirstCvtWarp) / kCvtGroup;
    const int row   = q * 32 + lane;
    int stage = 0;
    uint32_t phase = 0;
    uint32_t it = 0;                          // stages walked so far
    bool dead = false;   // a wait ran out: walk the remaining stages without waiting or working, but keep arriving
    long long w_cwait = 0, w_cwork = 0;
    TileRec nrec = tile_rec(0);
    for (int i = 0; i < my_tiles; ++i) {
      const int t    = cta + i * nctas;
      const TileS ti = decode_rec(nrec);
      if (i + 1 < my_tiles) nrec = tile_rec(i + 1);
      const GGSwapProblemDev* pr = problems + ti.p;
      const bool convert         = is_cvt_scheme(ti.scheme);
      const int N                = pr->N;
      const int gn               = ti.n_tile * kWT + row;
      // w4a16: (scale, zero) pairs, [K/128][N][2] fp16; one group of 128 k spans two 64-k stages.  The pair of
      // the group's NEXT stage (two K blocks on) is fetched while the current stage is converted: a global load
      // at the head of every stage's chain of waits would bound the whole pipeline.
      const bool has_sz   = ti.scheme == SCH_W4A16G128 && gn < N;
      const __half2* szp  = reinterpret_cast<const __half2*>(pr->scale_b) + gn;
      // K blocks per (scale, zero) group as a shift: 1 for groups of 128 (two 64-k stages); the per-channel scheme
      // (cta_gemm.cuh:112-286) has one group for the whole of K
      // (with stages of two K blocks a stage IS a group of 128)
      const int gsh       = pr->one_group ? 30 : (kTwo ? 0 : 1);
      const int kb_first  = (int)(((uint32_t)group + kCvtGroups - it % kCvtGroups) % kCvtGroups);   // first K block of this tile the group handles
      __half2 sz_next = __float2half2_rn(0.f);
      if (has_sz && kb_first < ti.nkb) sz_next = __ldg(szp + (int64_t)(kb_first >> gsh) * N);
      for (int kb = 0; kb < ti.nkb; ++kb, ++it) {
        const int s_cur       = stage;
        const uint32_t ph_cur = phase;
        if (++stage == G::kStages) { stage = 0; phase ^= 1u; }
        if ((int)(it % kCvtGroups) != group) continue;   // another group's stage
        const __half2 sz = sz_next;
        if (has_sz && kb + kCvtGroups < ti.nkb) sz_next = __ldg(szp + (int64_t)((kb + kCvtGroups) >> gsh) * N);
        const long long c0 = tick(prof_on);
        if (!dead) {
          const bool ok = warp_wait_bar(smem_u32(&ctrl->wfull[s_cur]), ph_cur, abort_flag, lane, tmo);
          if (!ok) {
            if (lane == 0) report_s(status, convert ? 5 : 6, t);
            dead = true;
          }
        }
        if (dead) {
          // the MMA warp's bar.sync (the leader's wait, in a pair) must complete
          if (kPair) { if (lane == 0) mbar_arrive_leader_relaxed(smem_u32(&ctrl->cvtdone[s_cur])); }
          else nbar_arrive(G::kBarStage0 + s_cur, kStageBar);
          continue;
        }
        const long long c1 = tick(prof_on);
        w_cwait += c1 - c0;
        if (q == 0 && lane == 0) TRACE(TR_CVT_GOT, (int)it);
        if (convert) {
          tc_fence_after_sync();
          // stages of two K blocks: the second block's packed weights lie behind the first's, its converted form
          // goes to the upper 32 columns of the stage's A slot
          const int nb = (kTwo && !(ti.odd && kb + 1 == ti.nkb)) ? 2 : 1;
#pragma unroll 1
          for (int b = 0; b < nb; ++b) {
          uint32_t o[32];
          if (ti.scheme == SCH_W4A4_XA || ti.scheme == SCH_W4A4) {
            // packed row: 64 bytes, 16-byte chunks swizzled by (row >> 1) & 3 (64-byte swizzle of the tensor map).
            // Chunk c becomes 32 int8 bytes: its high nibbles, then its low nibbles, each moved to the top of a
            // byte (code q -> byte 16*q; the accumulator is shifted back in the epilogue).
            const uint32_t src = wslot(s_cur) + b * (kWSlotBytes / 2) + row * 64;
            const int sw       = (row >> 1) & 3;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 w = lds128(src + ((j ^ sw) << 4));
              o[8 * j + 0] = w.x & 0xF0F0F0F0u; o[8 * j + 4] = (w.x << 4) & 0xF0F0F0F0u;
              o[8 * j + 1] = w.y & 0xF0F0F0F0u; o[8 * j + 5] = (w.y << 4) & 0xF0F0F0F0u;
              o[8 * j + 2] = w.z & 0xF0F0F0F0u; o[8 * j + 6] = (w.z << 4) & 0xF0F0F0F0u;
              o[8 * j + 3] = w.w & 0xF0F0F0F0u; o[8 * j + 7] = (w.w << 4) & 0xF0F0F0F0u;
            }
          } else {
            // w4a16 g128: channel n = 32*q + 8*f + r lives in packed row 8*q + r; the 16-k block kb16 of this
            // stage is the 16-byte chunk 2*kb16 + (f >> 1) (128-byte swizzle: XOR r), nibble 2*(f & 1) + c of
            // word d holds k = 16*kb16 + 8*c + d.
            const int f = lane >> 3, r = lane & 7;
            const uint32_t src = wslot(s_cur) + b * (kWSlotBytes / 4) + (8 * q + r) * 128;
            const __half2 s2 = __half2half2(__low2half(sz)), z2 = __half2half2(__high2half(sz));
#pragma unroll
            for (int kb16 = 0; kb16 < 4; ++kb16) {
              const uint4 w = lds128(src + (((2 * kb16 + (f >> 1)) ^ r) << 4));
#pragma unroll
              for (int c = 0; c < 2; ++c) {
                const int nib = 2 * (f & 1) + c;
                o[8 * kb16 + 4 * c + 0] = dequant_pair(w.x, nib, s2, z2);
                o[8 * kb16 + 4 * c + 1] = dequant_pair(w.y, nib, s2, z2);
                o[8 * kb16 + 4 * c + 2] = dequant_pair(w.z, nib, s2, z2);
                o[8 * kb16 + 4 * c + 3] = dequant_pair(w.w, nib, s2, z2);
              }
            }
          }
          tmem_st_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + G::kASlotCol0 + s_cur * G::kASlotStride + b * kASlotCols, o);
          }
          if (kMode == 2 && ti.scheme == SCH_W4A4) {
            // packed activation rows -> int8 rows of the swizzled operand tile (the same nibble -> byte 16*q map)
            const int rows32 = (ti.ntok + 31) & ~31;
            convert_w4a4<kCvtGroup * 32>(wslot(s_cur) + kWSlotBytes / 2, wslot(s_cur) + kWSlotBytes, rows32, q * 32 + lane);
            fence_proxy_async_smem();
          }
        }
        // the stage's packed weights are in registers (or not needed): release the stage
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctrl->empty[s_cur]));
        if (convert) {
          tmem_st_wait();
          tc_fence_before_sync();
          __syncwarp();
          w_cwork += tick(prof_on) - c1;
        }
        if (q == 0 && lane == 0) TRACE(TR_CVT_DONE, (int)it);
        if (kPair) {
          __syncwarp();
          if (lane == 0) mbar_arrive_leader_relaxed(smem_u32(&ctrl->cvtdone[s_cur]));
        } else {
          nbar_arrive(G::kBarStage0 + s_cur, kStageBar);
        }
      }
    }
    if (blockIdx.x == 0 && warp == kFirstCvtWarp && lane == 0) {
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
  if (kPair) cluster_sync_all();   // the other CTA may still signal this CTA's barriers or read its shared memory
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    if (kPair) tmem_dealloc2(tmem_base, 512);
    else       tmem_dealloc(tmem_base, 512);
  }
}

namespace {
template <int kMode, bool kSmall>
cudaError_t configure_one() {
  cudaError_t e = cudaFuncSetAttribute(gg_swap_kernel<kMode, kSmall, false, false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes_swap<Geo<kSmall>>());
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(gg_swap_kernel<kMode, kSmall, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              smem_bytes_swap<Geo<kSmall>>());
}
template <int kMode, bool kSmall>
void launch_one(const GGSwapProblemDev* problems, int count, GGStatus* status, bool ext, int num_ctas, cudaStream_t stream) {
  if (ext) gg_swap_kernel<kMode, kSmall, false, true><<<num_ctas, CfgS<kMode>::kThreads, smem_bytes_swap<Geo<kSmall>>(), stream>>>(problems, count, status);
  else     gg_swap_kernel<kMode, kSmall, false, false><<<num_ctas, CfgS<kMode>::kThreads, smem_bytes_swap<Geo<kSmall>>(), stream>>>(problems, count, status);
}
template <int kMode>
void launch_pair(const GGSwapProblemDev* problems, int count, GGStatus* status, bool ext, int num_ctas, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim            = dim3((unsigned)(num_ctas & ~1), 1, 1);
  cfg.blockDim           = dim3(CfgS<kMode>::kThreads, 1, 1);
  cfg.dynamicSmemBytes   = smem_bytes_swap<Geo<false>>();
  cfg.stream             = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id               = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs    = attr;
  cfg.numAttrs = 1;
  if (ext) cudaLaunchKernelEx(&cfg, gg_swap_kernel<kMode, false, true, true>, problems, count, status);
  else     cudaLaunchKernelEx(&cfg, gg_swap_kernel<kMode, false, true, false>, problems, count, status);
}
}  // namespace

#ifdef MXMOE_TRACE
extern "C" int mxmoe_gg_trace(long long* out) {   // out[kTraceEvents][kTraceLen]
  return (int)cudaMemcpyFromSymbol(out, g_trace, sizeof(g_trace));
}
#endif

cudaError_t gg_configure_swap() {
  cudaError_t e;
  if ((e = configure_one<0, false>()) != cudaSuccess) return e;
  if ((e = configure_one<1, false>()) != cudaSuccess) return e;
  if ((e = configure_one<2, false>()) != cudaSuccess) return e;
  if ((e = configure_one<0, true>()) != cudaSuccess) return e;
  if ((e = configure_one<1, true>()) != cudaSuccess) return e;
  if ((e = configure_one<2, true>()) != cudaSuccess) return e;
  constexpr int kBytes = smem_bytes_swap<Geo<false>>();
  if ((e = cudaFuncSetAttribute(gg_swap_kernel<0, false, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(gg_swap_kernel<0, false, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(gg_swap_kernel<1, false, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes)) != cudaSuccess) return e;
  return cudaFuncSetAttribute(gg_swap_kernel<1, false, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes);
}

// CTA pairs (cta_group::2): large token tiles, activations in their final form (cvt_mode 0 or 1)
void gg_launch_swap_pair(const GGSwapProblemDev* problems, int count, GGStatus* status, int cvt_mode, bool ext,
                         int num_ctas, cudaStream_t stream) {
  if (cvt_mode) launch_pair<1>(problems, count, status, ext, num_ctas, stream);
  else          launch_pair<0>(problems, count, status, ext, num_ctas, stream);
}

void gg_launch_swap(const GGSwapProblemDev* problems, int count, GGStatus* status, int cvt_mode, bool small_tiles,
                    bool ext, int num_ctas, cudaStream_t stream) {
  if (small_tiles) {
    if (cvt_mode == 2)  launch_one<2, true>(problems, count, status, ext, num_ctas, stream);
    else if (cvt_mode)  launch_one<1, true>(problems, count, status, ext, num_ctas, stream);
    else                launch_one<0, true>(problems, count, status, ext, num_ctas, stream);
  } else {
    if (cvt_mode == 2)  launch_one<2, false>(problems, count, status, ext, num_ctas, stream);
    else if (cvt_mode)  launch_one<1, false>(problems, count, status, ext, num_ctas, stream);
    else                launch_one<0, false>(problems, count, status, ext, num_ctas, stream);
  }
}

}  // namespace mxb
