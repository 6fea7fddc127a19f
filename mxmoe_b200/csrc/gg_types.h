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
};

enum OutMode : int {
  OUT_FP16 = 0,  // scaled fp16 result
  OUT_ACC  = 1,  // raw accumulators: int32 for w8a8 / w4a4, fp32 otherwise
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

// Workspace: [GGStatus (256 B)] [GGProblemDev x count]
struct alignas(256) GGStatus {
  int error;       // 0 = ok; otherwise an MXMOE_DEVERR_* code
  int where;       // role << 24 | tile index
  int count;       // problems prepared
  int needs_cvt;   // any problem needs the converter warps
  int pad[60];
};
static_assert(sizeof(GGStatus) == 256, "GGStatus layout");

constexpr int kDevErrTimeout = 1;   // a bounded wait ran out
constexpr int kDevErrTooMany = 2;   // more problems than kMaxProblems

// single-CTA kernel (gg_kernel.cu): tiles of 128 x 256, any number of CTAs
void gg_launch_single(const GGProblemDev* problems, int count, GGStatus* status, bool needs_cvt, int num_ctas,
                      cudaStream_t stream);
cudaError_t gg_configure_single();
// CTA-pair kernel (gg_pair_kernel.cu): tiles of 256 x 256 on clusters of two CTAs; num_ctas must be even
cudaError_t gg_launch_pair(const GGProblemDev* problems, int count, GGStatus* status, bool needs_cvt, int num_ctas,
                           cudaStream_t stream);
cudaError_t gg_configure_pair();

}  // namespace mxb
