// Device-side problem list of the grouped GEMM and the workspace layout shared
// by the host launcher (capi.cu) and the kernel (gg_kernel.cu).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace mxb {

// Quantisation scheme of one problem (one linear block of one expert).
enum Scheme : int {
  SCH_FP16      = 0,  // fp16 x fp16, fp32 accumulate
  SCH_W8A8      = 1,  // int8 codes, per-token / per-channel fp16 scales
  SCH_W4A4      = 2,  // int4 codes packed along K, per-token / per-channel fp16 scales
  SCH_W4A16G128 = 3,  // fp16 activations, 4-bit weights packed along N, (scale, zero) per 128-k group
  SCH_W4A4_XA   = 4,  // w4a4 whose activations are already expanded: one byte 16*q per code (see below)
};

enum OutMode : int {
  OUT_FP16 = 0,  // scaled fp16 result
  OUT_ACC  = 1,  // raw accumulators: int32 for w8a8 / w4a4, fp32 otherwise
  OUT_SILU = 2,  // B = [gate rows; up rows] (N = 2 I): C[M, I] = fp16( fp16(silu(gate)) * up ) of the scaled fp16 results
};

constexpr int kMaxProblems = 256;
constexpr int kBM          = 128;  // rows of C per tile (tcgen05 M)
constexpr int kBN          = 256;  // columns of C per tile (tcgen05 N)
constexpr int kRowBytes    = 128;  // bytes of K per operand row and pipeline stage (one 128-byte swizzle atom)

// One entry of the device-side problem list.  Written by the host, read-only in
// the kernel.  `row0` / `row0_dev` shift the rows of A, of scale_a and of C
// together, so that several problems can share one tensor map over a contiguous
// expert-sorted activation buffer; `m_dev` lets the row count come from device
// memory (routing result) without a host round trip.
struct alignas(128) GGProblemDev {
  CUtensorMap tmA;
  CUtensorMap tmB;
  const __half* scale_a;
  const __half* scale_b;
  void* C;
  const int* m_dev;
  const int* row0_dev;
  int M;       // rows (upper bound when m_dev is set)
  int N;
  int K;
  int row0;
  int scheme;
  int out_mode;
  int ldc;     // row pitch of C in elements
  int sa_stride;  // distance between per-token scales, in elements (>= 1)
};
static_assert(sizeof(GGProblemDev) == 384, "GGProblemDev layout");

// The same problem as seen by the kernel with swapped operands (gg_swap_kernel.cu): the weights are the
// M side of the MMA (tiles of 128 output channels), the tokens the N side (tiles of up to 176 rows).
constexpr int kWT = 128;   // output channels per tile (tcgen05 M)
constexpr int kTT = 176;   // tokens per tile (tcgen05 N, any multiple of 16 up to this)
constexpr int kXBoxSmall = 32;   // rows of the small activation box (short token tiles load only what they need)
struct alignas(128) GGSwapProblemDev {
  CUtensorMap tmW;    // weights: 128 channels x one stage of K (packed for the 4-bit schemes)
  CUtensorMap tmX;    // activations: kTT rows x 128 bytes of K
  CUtensorMap tmXs;   // activations: kXBoxSmall rows x 128 bytes of K
  CUtensorMap tmXh;   // activations: kTT / 2 rows x 128 bytes of K (each CTA of a pair loads half of the token tile)
  const __half* scale_a;
  const __half* scale_b;
  void* C;
  const int* m_dev;
  const int* row0_dev;
  int M, N, K, row0;
  int scheme, out_mode, ldc, sa_stride;
  const int64_t* c_row_ptrs;   // optional: result row r goes to the ADDRESS c_row_ptrs[r] (rows numbered like A's)
  const int* c_row0_dev;   // optional: rows of C start at *c_row0_dev instead of at row0
  int one_group;           // w4a16: one (scale, zero) pair per channel for the whole of K (per-channel scheme)
  int bulk_out;            // fp16 results leave as whole 256-byte rows through the copy engine (outputs in a peer's memory)
  int silu_inter;          // OUT_SILU: I (the weight tile interleaves 16 gate rows with 16 up rows, four times); else 0
  int pad[7];
};
static_assert(sizeof(GGSwapProblemDev) == 640, "GGSwapProblemDev layout");

// Workspace: [GGStatus (256 B)] [GGProblemDev x count] [GGSwapProblemDev x count]
struct alignas(256) GGStatus {
  int error;       // 0 = ok; otherwise an MXMOE_DEVERR_* code
  int where;       // role << 24 | tile index
  int count;       // problems prepared
  int needs_cvt;   // any problem needs the converter warps
  // cycle counters of CTA 0 of the last launch (clock64 deltas), see GGProf
  unsigned long long prof[16];
  int prof_on;      // per-role cycle counters wanted (costs a few percent)
  int timeout_ms;   // limit of every bounded wait of the kernel with swapped operands; 0 = 1000 ms
  int skip_stage;   // test hook: 1 + the pipeline stage (counted from the start of CTA 0's work) for which CTA 0's
                    // producer announces more weight bytes than it loads, so that the wait for them runs out; 0 = none
  int pad[25];
};

// indices into GGStatus::prof
enum GGProf : int {
  PROF_TOTAL = 0,        // kernel body
  PROF_PROD_WAIT,        // producer waiting for a free stage
  PROF_MMA_WAIT_OPER,    // MMA issuer waiting for operands (full / cvt)
  PROF_MMA_WAIT_ACC,     // MMA issuer waiting for a drained accumulator
  PROF_MMA_ISSUE,        // MMA issuer inside issue + commit
  PROF_EPI_WAIT,         // epilogue warp 2 waiting for the accumulator
  PROF_EPI_STORE,        // epilogue warp 2 draining + storing
  PROF_CVT_WAIT,         // converter warp 6 waiting for packed operands
  PROF_CVT_WORK,         // converter warp 6 converting
  PROF_TILES,            // tiles processed by CTA 0
  PROF_STAGES,           // pipeline stages processed by CTA 0
};
static_assert(sizeof(GGStatus) == 256, "GGStatus layout");

constexpr int kDevErrTimeout = 1;   // a bounded wait ran out
constexpr int kDevErrTooMany = 2;   // more problems than kMaxProblems

// cvt_mode: 0 no 4-bit operand in the launch; 1 only weights need converting (w4a16, w4a4 with expanded
// activations); 2 packed 4-bit activations are present as well.
// single-CTA kernel (gg_kernel.cu): tiles of 128 x 256, any number of CTAs
void gg_launch_single(const GGProblemDev* problems, int count, GGStatus* status, int cvt_mode, int num_ctas,
                      cudaStream_t stream);
cudaError_t gg_configure_single();
// CTA-pair kernel (gg_pair_kernel.cu): tiles of 256 x 256 on clusters of two CTAs; num_ctas must be even
cudaError_t gg_launch_pair(const GGProblemDev* problems, int count, GGStatus* status, int cvt_mode, int num_ctas,
                           cudaStream_t stream);
cudaError_t gg_configure_pair();
// kernel with swapped operands (gg_swap_kernel.cu): weights from tensor memory / shared memory as the M side,
// token tiles of up to 176 rows (ring of 5 stages) or, with `small_tiles`, of up to 32 rows (ring of 10 stages)
// as the N side
// `ext`: the launch holds problems with an optional result form (weight maps of rank 4), see gg_swap_kernel
void gg_launch_swap_pair(const GGSwapProblemDev* problems, int count, GGStatus* status, int cvt_mode, bool ext,
                         int num_ctas, cudaStream_t stream);
void gg_launch_swap(const GGSwapProblemDev* problems, int count, GGStatus* status, int cvt_mode, bool small_tiles, bool ext,
                    int num_ctas, cudaStream_t stream);
cudaError_t gg_configure_swap();

}  // namespace mxb
