// C ABI of libmxmoe_b200.so (declarations: include/mxmoe_b200.h).
//
// Host side of the grouped GEMM: validates a problem list, encodes one TMA
// descriptor per operand on the host (cuTensorMapEncodeTiled, looked up through
// the runtime so that the library has no link-time dependency on libcuda),
// uploads the device-side problem list into the caller's workspace and launches
// the persistent kernel.  No allocation happens on the launch path.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstddef>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/mxmoe_b200.h"
#include "act_kernels.h"
#include "gg_types.h"
#include "ep_kernels.h"
#include "route_kernels.h"
#include "had_kernels.h"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define CUDA_TRY(expr)                                                                              \
  do {                                                                                              \
    cudaError_t e__ = (expr);                                                                       \
    if (e__ != cudaSuccess)                                                                         \
      return fail(MXMOE_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, \
                  __LINE__);                                                                        \
  } while (0)

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct DeviceState {
  bool ready          = false;
  int sm_count        = 0;
  EncodeTiledFn encode = nullptr;
};
std::mutex g_mu;
DeviceState g_dev[64];

// Once per device: check the architecture, raise the dynamic shared-memory limit
// of the kernels and fetch the descriptor encoder.
int device_state(DeviceState** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return fail(MXMOE_ERR_NO_DEVICE, "no CUDA device available");
  }
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceState& st = g_dev[dev];
  if (!st.ready) {
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10) return fail(MXMOE_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", dev, prop.major, prop.minor);
    st.sm_count = prop.multiProcessorCount;
    void* fn    = nullptr;
    cudaDriverEntryPointQueryResult qres;
    CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || fn == nullptr)
      return fail(MXMOE_ERR_CUDA, "cuTensorMapEncodeTiled not available from the driver");
    st.encode = reinterpret_cast<EncodeTiledFn>(fn);
    CUDA_TRY(mxb::gg_configure_single());
    CUDA_TRY(mxb::gg_configure_pair());
    CUDA_TRY(mxb::gg_configure_swap());
    st.ready = true;
  }
  *out = &st;
  return MXMOE_OK;
}

int scheme_of(const mxmoe_qparams& q, int* scheme) {
  if (q.a_bits >= 16 && q.w_bits >= 16) { *scheme = mxb::SCH_FP16; return MXMOE_OK; }
  if (q.a_bits == 8 && q.w_bits == 8 && q.gsize == -1 && q.sym) { *scheme = mxb::SCH_W8A8; return MXMOE_OK; }
  if (q.a_bits == 4 && q.w_bits == 4 && q.gsize == -1 && q.sym) { *scheme = mxb::SCH_W4A4; return MXMOE_OK; }
  if (q.a_bits >= 16 && q.w_bits == 4 && (q.gsize == 128 || q.gsize == -1) && !q.sym) { *scheme = mxb::SCH_W4A16G128; return MXMOE_OK; }
  return fail(MXMOE_ERR_UNSUPPORTED, "unsupported scheme w%da%d_g%d_%s (built: fp16, w8a8_g-1_sym, w4a4_g-1_sym, w4a16_g128_asym, w4a16_g-1_asym)",
              q.w_bits, q.a_bits, q.gsize, q.sym ? "sym" : "asym");
}

// 2-D row-major byte/half matrix [rows, row_bytes] -> tiled tensor map with a box of (box_inner x box_rows)
int encode_2d(EncodeTiledFn enc, CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes,
              uint64_t inner_elems, uint64_t rows, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle sw,
              const char* what, int idx, uint64_t pitch_bytes = 0) {
  if (rows == 0 || inner_elems == 0) return fail(MXMOE_ERR_INVALID, "problem %d: empty %s operand", idx, what);
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0)
    return fail(MXMOE_ERR_INVALID, "problem %d: %s pointer %p is not 16-byte aligned", idx, what, base);
  const uint64_t pitch = pitch_bytes ? pitch_bytes : inner_elems * (uint64_t)elem_bytes;
  if (pitch < inner_elems * (uint64_t)elem_bytes) return fail(MXMOE_ERR_INVALID, "problem %d: %s row pitch %llu B is smaller than a row", idx, what, (unsigned long long)pitch);
  if (pitch % 16 != 0) return fail(MXMOE_ERR_INVALID, "problem %d: %s row pitch %llu B is not a multiple of 16", idx, what, (unsigned long long)pitch);
  cuuint64_t gdim[2]    = {inner_elems, rows};
  cuuint64_t gstride[1] = {pitch};
  cuuint32_t box[2]     = {box_inner, box_rows};
  cuuint32_t estr[2]    = {1, 1};
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MXMOE_ERR_CUDA, "problem %d: cuTensorMapEncodeTiled(%s) failed with CUresult %d", idx, what, (int)r);
  return MXMOE_OK;
}

// Weight map of the kernel with swapped operands, always of rank 4 so that its producer has one form of load.
// Plain: [rows][inner] with two unit dimensions, box = box_rows x box_inner.  `silu_inter` = I > 0: the matrix is
// [gate rows (I); up rows (I)] and a box of 128 rows gathers, four times, 16 gate rows followed by the 16 up rows of
// the same columns of C: dimensions (inner, 16 rows, gate|up, I / 16 groups), box (box_inner, 16, 2, 4).
int encode_w(EncodeTiledFn enc, CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes,
             uint64_t inner_elems, uint64_t rows, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle sw,
             int silu_inter, int idx, bool rank4) {
  if (!rank4) return encode_2d(enc, out, base, dt, elem_bytes, inner_elems, rows, box_inner, box_rows, sw, "B", idx);
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0)
    return fail(MXMOE_ERR_INVALID, "problem %d: B pointer %p is not 16-byte aligned", idx, base);
  const uint64_t pitch = inner_elems * (uint64_t)elem_bytes;
  if (pitch % 16 != 0) return fail(MXMOE_ERR_INVALID, "problem %d: B row pitch %llu B is not a multiple of 16", idx, (unsigned long long)pitch);
  cuuint64_t gdim[4], gstride[3];
  cuuint32_t box[4], estr[4] = {1, 1, 1, 1};
  if (silu_inter > 0) {
    const uint64_t I = (uint64_t)silu_inter;
    gdim[0] = inner_elems; gdim[1] = 16; gdim[2] = 2; gdim[3] = I / 16;
    gstride[0] = pitch; gstride[1] = I * pitch; gstride[2] = 16 * pitch;
    box[0] = box_inner; box[1] = 16; box[2] = 2; box[3] = box_rows / 32;
  } else {
    gdim[0] = inner_elems; gdim[1] = rows; gdim[2] = 1; gdim[3] = 1;
    gstride[0] = pitch; gstride[1] = pitch * rows; gstride[2] = pitch * rows;
    box[0] = box_inner; box[1] = box_rows; box[2] = 1; box[3] = 1;
  }
  CUresult r = enc(out, dt, 4, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MXMOE_ERR_CUDA, "problem %d: cuTensorMapEncodeTiled(B, rank 4) failed with CUresult %d", idx, (int)r);
  return MXMOE_OK;
}

int build_problem(EncodeTiledFn enc, const mxmoe_gg_problem& p, int idx, mxb::GGProblemDev* d) {
  int scheme = 0;
  int rc     = scheme_of(p.q, &scheme);
  if (rc) return rc;
  if (p.a_expanded) {
    if (scheme != mxb::SCH_W4A4) return fail(MXMOE_ERR_INVALID, "problem %d: a_expanded is only defined for w4a4", idx);
    scheme = mxb::SCH_W4A4_XA;
  }
  if (!p.A || !p.B || !p.C) return fail(MXMOE_ERR_INVALID, "problem %d: null A/B/C pointer", idx);
  if (p.M < 0 || p.N <= 0 || p.K <= 0) return fail(MXMOE_ERR_INVALID, "problem %d: bad shape M=%d N=%d K=%d", idx, p.M, p.N, p.K);
  if (p.N % 8 != 0) return fail(MXMOE_ERR_INVALID, "problem %d: N=%d must be a multiple of 8", idx, p.N);
  if (p.row0 < 0) return fail(MXMOE_ERR_INVALID, "problem %d: negative row0", idx);
  // OUT_SILU: C has one column per (gate, up) pair of weight rows
  const int n_out = p.out_mode == mxb::OUT_SILU ? p.N / 2 : p.N;
  const int ldc   = p.ldc > 0 ? p.ldc : n_out;
  if (ldc < n_out || ldc % 8 != 0) return fail(MXMOE_ERR_INVALID, "problem %d: ldc=%d must be >= the %d columns of C and a multiple of 8", idx, ldc, n_out);
  if (p.out_mode == mxb::OUT_SILU) {
    if (scheme == mxb::SCH_W4A16G128) return fail(MXMOE_ERR_UNSUPPORTED, "problem %d: out_mode 2 (silu(gate) * up) is not available for weights packed along N", idx);
    if (p.N % 128 != 0) return fail(MXMOE_ERR_INVALID, "problem %d: out_mode 2 needs N = 2 I with I %% 64 == 0 (N=%d)", idx, p.N);
  }
  if ((reinterpret_cast<uintptr_t>(p.C) & 15) != 0) return fail(MXMOE_ERR_INVALID, "problem %d: C is not 16-byte aligned", idx);
  const bool wxax = scheme == mxb::SCH_W8A8 || scheme == mxb::SCH_W4A4 || scheme == mxb::SCH_W4A4_XA;
  if (wxax && p.out_mode != mxb::OUT_ACC) {
    if (!p.scale_a || !p.scale_b) return fail(MXMOE_ERR_INVALID, "problem %d: w%da%d needs scale_a and scale_b", idx, p.q.w_bits, p.q.a_bits);
    if ((reinterpret_cast<uintptr_t>(p.scale_b) & 15) != 0) return fail(MXMOE_ERR_INVALID, "problem %d: scale_b is not 16-byte aligned", idx);
  }
  if (p.out_mode != mxb::OUT_FP16 && p.out_mode != mxb::OUT_ACC && p.out_mode != mxb::OUT_SILU) return fail(MXMOE_ERR_INVALID, "problem %d: bad out_mode %d", idx, p.out_mode);
  const uint64_t a_rows = p.a_rows > 0 ? (uint64_t)p.a_rows : (uint64_t)p.row0 + (uint64_t)p.M;
  const uint64_t lda    = p.lda_bytes > 0 ? (uint64_t)p.lda_bytes : 0;
  if (!p.row0_dev && a_rows < (uint64_t)p.row0 + (uint64_t)p.M) return fail(MXMOE_ERR_INVALID, "problem %d: a_rows=%llu < row0+M", idx, (unsigned long long)a_rows);

  const uint64_t K = (uint64_t)p.K, N = (uint64_t)p.N;
  {
    // the kernels pack (channel tiles, K blocks, scheme) of a problem into one word: 15 and 12 bits
    const int kelems = (scheme == mxb::SCH_FP16 || scheme == mxb::SCH_W4A16G128) ? 64 : 128;
    if ((p.K + kelems - 1) / kelems > 4095)
      return fail(MXMOE_ERR_UNSUPPORTED, "problem %d: K=%d exceeds the limit of %d for this scheme", idx, p.K, 4095 * kelems);
    if ((p.N + mxb::kWT - 1) / mxb::kWT > 32767)
      return fail(MXMOE_ERR_UNSUPPORTED, "problem %d: N=%d exceeds the limit of %d", idx, p.N, 32767 * mxb::kWT);
  }
  switch (scheme) {
    case mxb::SCH_FP16:
      if (p.K % 8) return fail(MXMOE_ERR_INVALID, "problem %d: fp16 needs K %% 8 == 0 (K=%d)", idx, p.K);
      if ((rc = encode_2d(enc, &d->tmA, p.A, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, K, a_rows, 64, mxb::kBM, CU_TENSOR_MAP_SWIZZLE_128B, "A", idx, lda))) return rc;
      if ((rc = encode_2d(enc, &d->tmB, p.B, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, K, N, 64, mxb::kBN / 2, CU_TENSOR_MAP_SWIZZLE_128B, "B", idx))) return rc;
      break;
    case mxb::SCH_W8A8:
      if (p.K % 16) return fail(MXMOE_ERR_INVALID, "problem %d: w8a8 needs K %% 16 == 0 (K=%d)", idx, p.K);
      if ((rc = encode_2d(enc, &d->tmA, p.A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, a_rows, 128, mxb::kBM, CU_TENSOR_MAP_SWIZZLE_128B, "A", idx, lda))) return rc;
      if ((rc = encode_2d(enc, &d->tmB, p.B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, N, 128, mxb::kBN / 2, CU_TENSOR_MAP_SWIZZLE_128B, "B", idx))) return rc;
      break;
    case mxb::SCH_W4A4:
      if (p.K % 32) return fail(MXMOE_ERR_INVALID, "problem %d: w4a4 needs K %% 32 == 0 (K=%d)", idx, p.K);
      if ((rc = encode_2d(enc, &d->tmA, p.A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K / 2, a_rows, 64, mxb::kBM, CU_TENSOR_MAP_SWIZZLE_NONE, "A", idx, lda))) return rc;
      if ((rc = encode_2d(enc, &d->tmB, p.B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K / 2, N, 64, mxb::kBN / 2, CU_TENSOR_MAP_SWIZZLE_NONE, "B", idx))) return rc;
      break;
    case mxb::SCH_W4A4_XA:
      if (p.K % 32) return fail(MXMOE_ERR_INVALID, "problem %d: w4a4 needs K %% 32 == 0 (K=%d)", idx, p.K);
      if ((rc = encode_2d(enc, &d->tmA, p.A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, a_rows, 128, mxb::kBM, CU_TENSOR_MAP_SWIZZLE_128B, "A", idx, lda))) return rc;
      if ((rc = encode_2d(enc, &d->tmB, p.B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K / 2, N, 64, mxb::kBN / 2, CU_TENSOR_MAP_SWIZZLE_NONE, "B", idx))) return rc;
      break;
    case mxb::SCH_W4A16G128:
      if (p.K % (p.q.gsize == 128 ? 128 : 64)) return fail(MXMOE_ERR_INVALID, "problem %d: w4a16 needs K %% %d == 0 (K=%d)", idx, p.q.gsize == 128 ? 128 : 64, p.K);
      if (p.N % 32) return fail(MXMOE_ERR_INVALID, "problem %d: w4a16_g128 needs N %% 32 == 0 (N=%d)", idx, p.N);
      if (!p.scale_b) return fail(MXMOE_ERR_INVALID, "problem %d: w4a16_g128 needs scale_b (scale, zero) pairs", idx);
      if ((reinterpret_cast<uintptr_t>(p.scale_b) & 3) != 0) return fail(MXMOE_ERR_INVALID, "problem %d: scale_b is not 4-byte aligned", idx);
      if ((rc = encode_2d(enc, &d->tmA, p.A, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, K, a_rows, 64, mxb::kBM, CU_TENSOR_MAP_SWIZZLE_128B, "A", idx, lda))) return rc;
      // [N/4, K] uint16 words seen as bytes: 64 k = 128 bytes per stage, a box of 32 packed rows = 128 n
      if ((rc = encode_2d(enc, &d->tmB, p.B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K * 2, N / 4, 128, mxb::kBN / 8, CU_TENSOR_MAP_SWIZZLE_NONE, "B", idx))) return rc;
      break;
  }
  d->scale_a  = static_cast<const __half*>(p.scale_a);
  d->scale_b  = static_cast<const __half*>(p.scale_b);
  d->C        = p.C;
  d->m_dev    = p.m_dev;
  d->row0_dev = p.row0_dev;
  d->M        = p.M;
  d->N        = p.N;
  d->K        = p.K;
  d->row0     = p.row0;
  d->scheme   = scheme;
  d->out_mode = p.out_mode;
  d->ldc      = ldc;
  d->sa_stride = p.sa_stride > 1 ? p.sa_stride : 1;
  return MXMOE_OK;
}

// The same problem for the kernel with swapped operands: tensor maps with its boxes (weights: 128 channels per
// box; activations: 176-row and 32-row boxes).  `d` has been validated by build_problem already.
// `ext`: the launch runs the kernel instance with the optional result forms; its weight maps have rank 4
int build_problem_swap(EncodeTiledFn enc, const mxmoe_gg_problem& p, int idx, const mxb::GGProblemDev& d,
                       mxb::GGSwapProblemDev* o, bool bulk_everywhere, bool ext) {
  int rc;
  const uint64_t a_rows = p.a_rows > 0 ? (uint64_t)p.a_rows : (uint64_t)p.row0 + (uint64_t)p.M;
  const uint64_t lda    = p.lda_bytes > 0 ? (uint64_t)p.lda_bytes : 0;
  const uint64_t K = (uint64_t)p.K, N = (uint64_t)p.N;
  const auto f16 = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const auto u8  = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const auto s128 = CU_TENSOR_MAP_SWIZZLE_128B;
  const int silu = d.out_mode == mxb::OUT_SILU ? p.N / 2 : 0;
  switch (d.scheme) {
    case mxb::SCH_FP16:
      if ((rc = encode_w(enc, &o->tmW, p.B, f16, 2, K, N, 64, mxb::kWT, s128, silu, idx, ext))) return rc;
      break;
    case mxb::SCH_W8A8:
      if ((rc = encode_w(enc, &o->tmW, p.B, u8, 1, K, N, 128, mxb::kWT, s128, silu, idx, ext))) return rc;
      break;
    case mxb::SCH_W4A4:
    case mxb::SCH_W4A4_XA:
      // packed rows of 64 bytes per stage; the 64-byte swizzle spreads the rows a converter warp reads over the banks
      if ((rc = encode_w(enc, &o->tmW, p.B, u8, 1, K / 2, N, 64, mxb::kWT, CU_TENSOR_MAP_SWIZZLE_64B, silu, idx, ext))) return rc;
      break;
    case mxb::SCH_W4A16G128:
      // [N/4, K] uint16 words seen as bytes: 64 k = 128 bytes per stage, 32 packed rows = 128 channels
      if ((rc = encode_w(enc, &o->tmW, p.B, u8, 1, K * 2, N / 4, 128, mxb::kWT / 4, s128, 0, idx, ext))) return rc;
      break;
    default:
      break;
  }
  if (d.scheme == mxb::SCH_FP16 || d.scheme == mxb::SCH_W4A16G128) {
    if ((rc = encode_2d(enc, &o->tmX, p.A, f16, 2, K, a_rows, 64, mxb::kTT, s128, "A", idx, lda))) return rc;
    if ((rc = encode_2d(enc, &o->tmXs, p.A, f16, 2, K, a_rows, 64, mxb::kXBoxSmall, s128, "A", idx, lda))) return rc;
    if ((rc = encode_2d(enc, &o->tmXh, p.A, f16, 2, K, a_rows, 64, mxb::kTT / 2, s128, "A", idx, lda))) return rc;
  } else if (d.scheme == mxb::SCH_W4A4) {
    // packed rows: 64 bytes of K per stage, unswizzled (the converters expand them in shared memory); token tiles
    // of such launches have at most 128 rows, loaded as 32-row boxes
    if ((rc = encode_2d(enc, &o->tmXs, p.A, u8, 1, K / 2, a_rows, 64, mxb::kXBoxSmall, CU_TENSOR_MAP_SWIZZLE_NONE, "A", idx, lda))) return rc;
    o->tmX = o->tmXs;
    o->tmXh = o->tmXs;
  } else if (d.scheme == mxb::SCH_W8A8 || d.scheme == mxb::SCH_W4A4_XA) {
    if ((rc = encode_2d(enc, &o->tmX, p.A, u8, 1, K, a_rows, 128, mxb::kTT, s128, "A", idx, lda))) return rc;
    if ((rc = encode_2d(enc, &o->tmXs, p.A, u8, 1, K, a_rows, 128, mxb::kXBoxSmall, s128, "A", idx, lda))) return rc;
    if ((rc = encode_2d(enc, &o->tmXh, p.A, u8, 1, K, a_rows, 128, mxb::kTT / 2, s128, "A", idx, lda))) return rc;
  }
  o->scale_a = d.scale_a; o->scale_b = d.scale_b; o->C = d.C; o->m_dev = d.m_dev; o->row0_dev = d.row0_dev;
  o->M = d.M; o->N = d.N; o->K = d.K; o->row0 = d.row0;
  o->scheme = d.scheme; o->out_mode = d.out_mode; o->ldc = d.ldc; o->sa_stride = d.sa_stride;
  o->c_row0_dev = p.c_row0_dev;
  o->one_group  = (d.scheme == mxb::SCH_W4A16G128 && p.q.gsize == -1) ? 1 : 0;
  o->c_row_ptrs = p.c_row_ptrs;
  // results addressed through c_row0_dev are the expert-parallel combine: they land in a peer's buffer
  const bool aligned = p.N % 8 == 0 && d.ldc % 8 == 0 && ((uintptr_t)d.C & 15) == 0;
  o->bulk_out = (d.out_mode == mxb::OUT_FP16 && aligned && (p.c_row0_dev != nullptr || p.c_row_ptrs != nullptr || bulk_everywhere)) ? 1 : 0;
  if (p.c_row_ptrs && !o->bulk_out)
    return fail(MXMOE_ERR_INVALID, "problem %d: c_row_ptrs needs fp16 results with N and ldc multiples of 8", idx);
  if (p.c_row_ptrs && p.c_row0_dev) return fail(MXMOE_ERR_INVALID, "problem %d: c_row_ptrs and c_row0_dev exclude each other", idx);
  o->silu_inter = silu;
  return MXMOE_OK;
}

enum GGKernel { GGK_DEFAULT = 0, GGK_SINGLE = 1, GGK_PAIR = 2, GGK_SWAP = 3, GGK_SWAP2 = 4 };

// which kernel a launch that does not name one uses: MXMOE_GG_KERNEL = swap | single | pair, read when a workspace
// is prepared (never on the launch path) and kept in the plan
int default_kernel() {
  const char* e = getenv("MXMOE_GG_KERNEL");
  if (e && !strcmp(e, "pair")) return GGK_PAIR;
  if (e && !strcmp(e, "single")) return GGK_SINGLE;
  if (e && !strcmp(e, "swap")) return GGK_SWAP;
  if (e && !strcmp(e, "swap2")) return GGK_SWAP2;
  return GGK_SWAP;
}

// token-tile geometry of the SWAP kernel: chosen from the row counts unless MXMOE_GG_TILES = small | large overrides
// it (read when a workspace is prepared)
bool small_tiles_at_prepare(bool few_rows) {
  const char* e = getenv("MXMOE_GG_TILES");
  if (e && !strcmp(e, "small")) return true;
  if (e && !strcmp(e, "large")) return false;
  return few_rows;
}

struct ShimScratch {
  void* ws        = nullptr;
  size_t ws_bytes = 0;
};
ShimScratch g_shim[64];

}  // namespace

extern "C" {

const char* mxmoe_last_error(void) { return g_err; }
int mxmoe_version(void) { return 100; }

int mxmoe_device_sm_count(void) {
  DeviceState* st = nullptr;
  int rc          = device_state(&st);
  if (rc) return -rc;
  return st->sm_count;
}

size_t mxmoe_gg_workspace_bytes(int problem_count) {
  if (problem_count < 0) problem_count = 0;
  return sizeof(mxb::GGStatus) + (sizeof(mxb::GGProblemDev) + sizeof(mxb::GGSwapProblemDev)) * (size_t)problem_count;
}

int mxmoe_gg_prepare(const mxmoe_gg_problem* problems, int problem_count, void* workspace, size_t workspace_bytes,
                     void* stream, mxmoe_gg_plan* plan) {
  if (problem_count < 0 || (problem_count > 0 && !problems)) return fail(MXMOE_ERR_INVALID, "bad problem list");
  if (problem_count > mxb::kMaxProblems) return fail(MXMOE_ERR_INVALID, "%d problems exceed the limit of %d per launch", problem_count, mxb::kMaxProblems);
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return fail(MXMOE_ERR_WORKSPACE, "workspace must be a 256-byte aligned device pointer");
  if (workspace_bytes < mxmoe_gg_workspace_bytes(problem_count)) return fail(MXMOE_ERR_WORKSPACE, "workspace of %zu B is smaller than the %zu B needed", workspace_bytes, mxmoe_gg_workspace_bytes(problem_count));
  DeviceState* st = nullptr;
  int rc          = device_state(&st);
  if (rc) return rc;

  std::vector<unsigned char> host(mxmoe_gg_workspace_bytes(problem_count));
  std::memset(host.data(), 0, host.size());
  auto* status = reinterpret_cast<mxb::GGStatus*>(host.data());
  auto* dev    = reinterpret_cast<mxb::GGProblemDev*>(host.data() + sizeof(mxb::GGStatus));
  std::vector<mxb::GGSwapProblemDev> swp((size_t)problem_count);
  if (problem_count) std::memset(swp.data(), 0, swp.size() * sizeof(mxb::GGSwapProblemDev));
  int kept = 0, needs_cvt = 0;
  bool redirect = false;
  // MXMOE_GG_STORES = rows: every fp16 result leaves as whole rows through the copy engine, not only those that go
  // to a peer (read here, when the workspace is prepared)
  const char* stores_env     = getenv("MXMOE_GG_STORES");
  const bool bulk_everywhere = stores_env && !strcmp(stores_env, "rows");
  // does any problem use an optional result form?  Then the launch runs the kernel instance that has them.
  bool ext = bulk_everywhere;
  for (int i = 0; i < problem_count; ++i)
    if (problems[i].c_row0_dev || problems[i].c_row_ptrs || problems[i].out_mode == mxb::OUT_SILU) ext = true;
  int max_rows = 0;
  for (int i = 0; i < problem_count; ++i) {
    if (problems[i].M == 0 && !problems[i].m_dev) continue;  // empty expert (ref_bind.cu:345 skips them too)
    rc = build_problem(st->encode, problems[i], i, dev + kept);
    if (rc) return rc;
    rc = build_problem_swap(st->encode, problems[i], i, dev[kept], &swp[kept], bulk_everywhere, ext);
    if (rc) return rc;
    // redirected C rows and the per-channel 4-bit weight-only scheme exist in the SWAP kernel only
    if (problems[i].c_row0_dev || problems[i].c_row_ptrs || (dev[kept].scheme == mxb::SCH_W4A16G128 && problems[i].q.gsize == -1) ||
        problems[i].out_mode == mxb::OUT_SILU) redirect = true;
    if (problems[i].M > max_rows) max_rows = problems[i].M;
    if (dev[kept].scheme == mxb::SCH_W4A4) needs_cvt = 2;
    else if ((dev[kept].scheme == mxb::SCH_W4A4_XA || dev[kept].scheme == mxb::SCH_W4A16G128) && needs_cvt < 1) needs_cvt = 1;
    ++kept;
  }
  status->prof_on   = getenv("MXMOE_GG_PROFILE") ? atoi(getenv("MXMOE_GG_PROFILE")) : 0;   // per-role counters on
  status->count     = kept;
  status->needs_cvt = needs_cvt;
  // pageable source: the runtime stages the bytes before returning, so `host` may go out of scope
  // the list for the kernel with swapped operands follows the kept entries of the first list
  const size_t first = sizeof(mxb::GGStatus) + sizeof(mxb::GGProblemDev) * (size_t)kept;
  if (kept) std::memcpy(host.data() + first, swp.data(), sizeof(mxb::GGSwapProblemDev) * (size_t)kept);
  CUDA_TRY(cudaMemcpyAsync(workspace, host.data(), first + sizeof(mxb::GGSwapProblemDev) * (size_t)kept,
                           cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
  if (plan) {
    plan->count     = kept;
    plan->needs_cvt = needs_cvt;
    // few rows in every problem: token tiles of 32 rows and a deeper ring (more weight bytes in flight per SM)
    plan->flags     = (redirect ? 1 : 0) | (small_tiles_at_prepare(max_rows <= 32) ? 2 : 0) | (ext ? 4 : 0);
    plan->kernel    = default_kernel();
  }
  return MXMOE_OK;
}

namespace {
int run_kernel(void* workspace, const mxmoe_gg_plan* plan, int kernel, int num_ctas, void* stream) {
  if (!workspace || !plan) return fail(MXMOE_ERR_WORKSPACE, "null workspace or plan");
  DeviceState* st = nullptr;
  int rc          = device_state(&st);
  if (rc) return rc;
  const int count = plan->count, needs_cvt = plan->needs_cvt;
  if (count < 0 || count > mxb::kMaxProblems) return fail(MXMOE_ERR_WORKSPACE, "plan holds an invalid problem count %d", count);
  if (count == 0) return MXMOE_OK;
  auto* status = static_cast<mxb::GGStatus*>(workspace);
  auto* base   = static_cast<unsigned char*>(workspace) + sizeof(mxb::GGStatus);
  auto* probs  = reinterpret_cast<const mxb::GGProblemDev*>(base);
  auto* swp    = reinterpret_cast<const mxb::GGSwapProblemDev*>(base + sizeof(mxb::GGProblemDev) * (size_t)count);
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  if (kernel == GGK_DEFAULT) kernel = (plan->kernel >= GGK_SINGLE && plan->kernel <= GGK_SWAP2) ? plan->kernel : GGK_SWAP;
  if (plan->flags & 1) {
    if (kernel != GGK_SWAP && kernel != GGK_SWAP2) return fail(MXMOE_ERR_UNSUPPORTED, "problems that redirect their C rows or use w4a16_g-1_asym run on the SWAP kernel only");
  }
  int n = num_ctas;
  if (n <= 0 || n > st->sm_count) n = st->sm_count;
  if (kernel == GGK_PAIR && n < 2) kernel = GGK_SINGLE;
  // CTA pairs of the kernel with swapped operands: large token tiles and activations in their final form only
  if (kernel == GGK_SWAP2 && (n < 2 || (plan->flags & 2) || needs_cvt == 2)) kernel = GGK_SWAP;
  const bool ext = (plan->flags & 4) != 0;
  if (kernel == GGK_SWAP2)      mxb::gg_launch_swap_pair(swp, count, status, needs_cvt, ext, n & ~1, cs);
  else if (kernel == GGK_PAIR)  CUDA_TRY(mxb::gg_launch_pair(probs, count, status, needs_cvt, n & ~1, cs));
  else if (kernel == GGK_SWAP)  mxb::gg_launch_swap(swp, count, status, needs_cvt, (plan->flags & 2) != 0, ext, n, cs);
  else                          mxb::gg_launch_single(probs, count, status, needs_cvt, n, cs);
  CUDA_TRY(cudaGetLastError());
  return MXMOE_OK;
}
}  // namespace

int mxmoe_gg_run(void* workspace, const mxmoe_gg_plan* plan, int num_ctas, void* stream) {
  // num_ctas > 0: that many CTAs of the default kernel; < 0: CTA-pair kernel with -num_ctas CTAs; 0: every SM
  if (num_ctas < 0) return run_kernel(workspace, plan, GGK_PAIR, -num_ctas, stream);
  return run_kernel(workspace, plan, GGK_DEFAULT, num_ctas, stream);
}

int mxmoe_gg_run_kernel(void* workspace, const mxmoe_gg_plan* plan, int kernel, int num_ctas, void* stream) {
  if (kernel < GGK_DEFAULT || kernel > GGK_SWAP2) return fail(MXMOE_ERR_INVALID, "unknown kernel id %d", kernel);
  return run_kernel(workspace, plan, kernel, num_ctas < 0 ? -num_ctas : num_ctas, stream);
}

int mxmoe_gg_launch(const mxmoe_gg_problem* problems, int problem_count, void* workspace, size_t workspace_bytes,
                    void* stream) {
  mxmoe_gg_plan plan;
  int rc = mxmoe_gg_prepare(problems, problem_count, workspace, workspace_bytes, stream, &plan);
  if (rc) return rc;
  return mxmoe_gg_run(workspace, &plan, 0, stream);
}

int mxmoe_gg_check(void* workspace, void* stream) {
  if (!workspace) return fail(MXMOE_ERR_WORKSPACE, "null workspace");
  int words[2] = {0, 0};
  CUDA_TRY(cudaMemcpyAsync(words, workspace, sizeof(words), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  if (words[0] != 0) {
    static const char* roles[] = {"?", "producer", "mma(accumulator)", "mma(operands)", "epilogue", "converter", "converter(pacing)"};
    const int role = (words[1] >> 24) & 0xff;
    // the report is taken: clear it, so that the workspace can be launched again
    CUDA_TRY(cudaMemsetAsync(workspace, 0, sizeof(words), static_cast<cudaStream_t>(stream)));
    return fail(MXMOE_ERR_DEVICE, "kernel reported error %d (%s) in role %s at tile %d", words[0],
                words[0] == mxb::kDevErrTimeout ? "bounded wait ran out" : "too many problems",
                role < 7 ? roles[role] : "?", words[1] & 0xffffff);
  }
  return MXMOE_OK;
}

int mxmoe_gg_debug(void* workspace, int timeout_ms, int skip_stage, void* stream) {
  if (!workspace) return fail(MXMOE_ERR_WORKSPACE, "null workspace");
  if (timeout_ms < 0 || skip_stage < -1) return fail(MXMOE_ERR_INVALID, "bad debug setting");
  int words[2] = {timeout_ms, skip_stage + 1};
  auto* base = static_cast<unsigned char*>(workspace) + offsetof(mxb::GGStatus, timeout_ms);
  static_assert(offsetof(mxb::GGStatus, skip_stage) == offsetof(mxb::GGStatus, timeout_ms) + sizeof(int), "status layout");
  CUDA_TRY(cudaMemcpyAsync(base, words, sizeof(words), cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
  CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));   // `words` lives on this stack frame
  return MXMOE_OK;
}

int mxmoe_gg_profile(void* workspace, uint64_t* counters, void* stream) {
  if (!workspace || !counters) return fail(MXMOE_ERR_INVALID, "null argument");
  mxb::GGStatus h;
  CUDA_TRY(cudaMemcpyAsync(&h, workspace, sizeof(h), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  for (int i = 0; i < 16; ++i) counters[i] = h.prof[i];
  return MXMOE_OK;
}

int mxmoe_groupgemm_hz_fused(void** ptr_As, void** ptr_Bs, void** ptr_scale_a, void** ptr_scale_b, void** ptr_Cs,
                             void** ptr_Ds, int64_t*, int64_t*, int64_t*, int64_t*, const uint32_t*,
                             const uint32_t* host_problem_sizes, const mxmoe_qparams*,
                             const mxmoe_qparams* host_qparams, int problem_count) {
  (void)ptr_Ds;  // aliases ptr_Cs in every reference call site
  if (problem_count <= 0) return MXMOE_OK;
  if (!ptr_As || !ptr_Bs || !ptr_Cs || !host_problem_sizes || !host_qparams) return fail(MXMOE_ERR_INVALID, "null argument");
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  const size_t n = (size_t)problem_count;
  std::vector<void*> hA(n), hB(n), hSa(n, nullptr), hSb(n, nullptr), hC(n);
  CUDA_TRY(cudaMemcpy(hA.data(), ptr_As, n * sizeof(void*), cudaMemcpyDeviceToHost));
  CUDA_TRY(cudaMemcpy(hB.data(), ptr_Bs, n * sizeof(void*), cudaMemcpyDeviceToHost));
  CUDA_TRY(cudaMemcpy(hC.data(), ptr_Cs, n * sizeof(void*), cudaMemcpyDeviceToHost));
  if (ptr_scale_a) CUDA_TRY(cudaMemcpy(hSa.data(), ptr_scale_a, n * sizeof(void*), cudaMemcpyDeviceToHost));
  if (ptr_scale_b) CUDA_TRY(cudaMemcpy(hSb.data(), ptr_scale_b, n * sizeof(void*), cudaMemcpyDeviceToHost));
  std::vector<mxmoe_gg_problem> probs(n);
  std::memset(probs.data(), 0, n * sizeof(mxmoe_gg_problem));
  for (size_t i = 0; i < n; ++i) {
    probs[i].A = hA[i]; probs[i].B = hB[i]; probs[i].C = hC[i];
    probs[i].scale_a = hSa[i]; probs[i].scale_b = hSb[i];
    probs[i].M = (int)host_problem_sizes[3 * i + 0];
    probs[i].N = (int)host_problem_sizes[3 * i + 1];
    probs[i].K = (int)host_problem_sizes[3 * i + 2];
    probs[i].q = host_qparams[i];
  }
  // grow-only scratch owned by the shim (the reference launcher allocates and frees per call)
  ShimScratch& sc = g_shim[dev & 63];
  const size_t need = mxmoe_gg_workspace_bytes(problem_count);
  if (sc.ws_bytes < need) {
    if (sc.ws) cudaFree(sc.ws);
    sc.ws = nullptr; sc.ws_bytes = 0;
    CUDA_TRY(cudaMalloc(&sc.ws, need));
    sc.ws_bytes = need;
  }
  int rc = mxmoe_gg_launch(probs.data(), problem_count, sc.ws, sc.ws_bytes, nullptr);
  if (rc) return rc;
  return mxmoe_gg_check(sc.ws, nullptr);
}

static int to_act_args(const mxmoe_act_args* a, mxb::ActArgs* o, bool silu) {
  if (!a) return fail(MXMOE_ERR_INVALID, "null args");
  if (!a->in || !a->q_store || !a->exp_qtag || (!a->exp_row_start && a->rec_stride <= 0))
    return fail(MXMOE_ERR_INVALID, "null pointer in activation arguments");
  if (a->rows_routed > 0 && !a->row_expert) return fail(MXMOE_ERR_INVALID, "row_expert is required for routed rows");
  // quant_act without row_token: the rows of `in` (and of `in_shared`) are taken in place; no rotation then
  if (!silu && a->rows_routed > 0 && !a->row_token && a->rotate) return fail(MXMOE_ERR_INVALID, "row_token is required for rotated rows");
  if (a->rows_routed < 0 || a->rows_total < a->rows_routed) return fail(MXMOE_ERR_INVALID, "bad row counts");
  const bool has_shared = a->rows_total > a->rows_routed;
  const int ks = has_shared ? a->k_shared : a->k;
  if (a->k <= 0 || a->k % 8 || ks <= 0 || ks % 8) return fail(MXMOE_ERR_INVALID, "row length must be a positive multiple of 8 (k=%d, k_shared=%d)", a->k, ks);
  if (a->k > 16384 || ks > 16384) return fail(MXMOE_ERR_UNSUPPORTED, "row length above 16384 is not supported");
  if ((silu || !a->row_token) && has_shared && !a->in_shared) return fail(MXMOE_ERR_INVALID, "in_shared is required for shared-expert rows");
  if (!silu && a->rotate) {
    if ((a->k & (a->k - 1)) != 0 || a->k < 256) return fail(MXMOE_ERR_UNSUPPORTED, "rotation needs a power-of-two row length >= 256 (k=%d)", a->k);
    if (has_shared && ks != a->k) return fail(MXMOE_ERR_INVALID, "rotation needs k_shared == k");
  }
  o->in = static_cast<const __half*>(a->in);
  o->in_shared = static_cast<const __half*>(a->in_shared);
  o->q_store = static_cast<__half*>(a->q_store);
  o->s_store = static_cast<__half*>(a->s_store);
  o->row_expert = a->row_expert;
  o->row_token = a->row_token;
  o->exp_qtag = a->exp_qtag;
  o->exp_row_start = a->exp_row_start;
  o->exp_q_off = a->exp_q_off;
  o->exp_s_off = a->exp_s_off;
  o->signs = a->signs;
  o->k = a->k;
  o->k_shared = ks;
  o->rows_routed = a->rows_routed;
  o->rows_total = a->rows_total;
  o->num_experts = a->num_experts;
  o->rotate = silu ? 0 : a->rotate;
  o->rec_stride = a->rec_stride > 0 ? a->rec_stride : 0;
  o->rec_scale_off = a->rec_scale_off;
  o->rows_dev = nullptr;
  if (a->rows_dev) {
    if (!silu || has_shared) return fail(MXMOE_ERR_UNSUPPORTED, "rows_dev is for silu_mul_then_quant without shared-expert rows");
    o->rows_dev = a->rows_dev;
  }
  if (o->rec_stride > 0) {
    const int kmax = a->k > ks ? a->k : ks;
    if (o->rec_stride % 8) return fail(MXMOE_ERR_INVALID, "rec_stride must be a multiple of 8 fp16 elements");
    if (o->rec_scale_off >= o->rec_stride) return fail(MXMOE_ERR_INVALID, "rec_scale_off lies outside the record");
    if (o->rec_stride * 4 < kmax) return fail(MXMOE_ERR_INVALID, "rec_stride %d cannot hold a row of %d elements in any format", o->rec_stride, kmax);
  }
  return MXMOE_OK;
}

int mxmoe_quant_act(const mxmoe_act_args* args, void* stream) {
  mxb::ActArgs a;
  int rc = to_act_args(args, &a, false);
  if (rc) return rc;
  CUDA_TRY(mxb::launch_quant_act(a, static_cast<cudaStream_t>(stream)));
  return MXMOE_OK;
}

static int to_token_args(const mxmoe_token_quant_args* t, mxb::TokenQuantArgs* o) {
  if (!t) return fail(MXMOE_ERR_INVALID, "null args");
  if (!t->in) return fail(MXMOE_ERR_INVALID, "null input");
  if (t->k <= 0 || t->k % 8 || t->k > 16384) return fail(MXMOE_ERR_INVALID, "row length must be a multiple of 8 in (0, 16384] (k=%d)", t->k);
  if (t->num_tokens < 0) return fail(MXMOE_ERR_INVALID, "negative token count");
  if (t->q4x && t->k % 32) return fail(MXMOE_ERR_INVALID, "the expanded 4-bit format needs k %% 32 == 0 (k=%d)", t->k);
  if ((t->q8 && !t->s8) || ((t->q4 || t->q4x) && !t->s4)) return fail(MXMOE_ERR_INVALID, "a packed store needs its scale store");
  if (t->rotate && ((t->k & (t->k - 1)) != 0 || t->k < 256)) return fail(MXMOE_ERR_UNSUPPORTED, "rotation needs a power-of-two row length >= 256 (k=%d)", t->k);
  o->in = static_cast<const __half*>(t->in);
  o->f16 = static_cast<__half*>(t->f16);
  o->q8 = static_cast<__half*>(t->q8);
  o->s8 = static_cast<__half*>(t->s8);
  o->q4 = static_cast<__half*>(t->q4);
  o->s4 = static_cast<__half*>(t->s4);
  o->q4x = static_cast<__half*>(t->q4x);
  o->signs = t->signs;
  o->k = t->k;
  o->num_tokens = t->num_tokens;
  o->rotate = t->rotate;
  o->reserved = 0;
  return MXMOE_OK;
}

int mxmoe_quant_tokens(const mxmoe_token_quant_args* args, void* stream) {
  mxb::TokenQuantArgs t;
  int rc = to_token_args(args, &t);
  if (rc) return rc;
  CUDA_TRY(mxb::launch_quant_tokens(t, static_cast<cudaStream_t>(stream)));
  return MXMOE_OK;
}

int mxmoe_gather_rows(const mxmoe_act_args* rows, const mxmoe_token_quant_args* stores, void* stream) {
  mxb::TokenQuantArgs t;
  int rc = to_token_args(stores, &t);
  if (rc) return rc;
  if (!rows) return fail(MXMOE_ERR_INVALID, "null args");
  mxmoe_act_args r = *rows;
  r.in = stores->in;
  r.rotate = 0;
  if (r.rows_total > r.rows_routed) r.k_shared = r.k;
  mxb::ActArgs a;
  rc = to_act_args(&r, &a, false);
  if (rc) return rc;
  CUDA_TRY(mxb::launch_gather_rows(a, t, static_cast<cudaStream_t>(stream)));
  return MXMOE_OK;
}

int mxmoe_quant_tokens_scatter(const mxmoe_token_quant_args* stores, const mxmoe_act_args* rows, const int32_t* slot_row,
                               int topk, void* stream) {
  mxb::TokenQuantArgs t;
  int rc = to_token_args(stores, &t);
  if (rc) return rc;
  if (!rows || !slot_row) return fail(MXMOE_ERR_INVALID, "null args");
  if (topk < 1 || topk > 8) return fail(MXMOE_ERR_UNSUPPORTED, "the one-pass scatter serves top-k 1..8 (topk=%d): use mxmoe_quant_tokens + mxmoe_gather_rows", topk);
  if (rows->rows_total != rows->rows_routed) return fail(MXMOE_ERR_INVALID, "the scatter writes routed rows only (rows_total must equal rows_routed)");
  if (rows->k != stores->k) return fail(MXMOE_ERR_INVALID, "row length of the rows (%d) and of the tokens (%d) differ", rows->k, stores->k);
  // destinations travel between lanes as 32-bit offsets (in fp16 elements) from the stores
  const int64_t pitch = rows->rec_stride > 0 ? rows->rec_stride : rows->k;
  if ((int64_t)rows->rows_routed * pitch >= (int64_t)1 << 31) return fail(MXMOE_ERR_UNSUPPORTED, "activation store beyond 2^31 elements: use mxmoe_quant_tokens + mxmoe_gather_rows");
  mxmoe_act_args r = *rows;
  r.in = stores->in;
  r.rotate = 0;
  mxb::ActArgs a;
  rc = to_act_args(&r, &a, false);
  if (rc) return rc;
  CUDA_TRY(mxb::launch_quant_tokens_scatter(t, a, slot_row, topk, static_cast<cudaStream_t>(stream)));
  return MXMOE_OK;
}

int mxmoe_silu_mul_then_quant(const mxmoe_act_args* args, void* stream) {
  mxb::ActArgs a;
  int rc = to_act_args(args, &a, true);
  if (rc) return rc;
  CUDA_TRY(mxb::launch_silu_mul_quant(a, static_cast<cudaStream_t>(stream)));
  return MXMOE_OK;
}


size_t mxmoe_route_workspace_bytes(int num_tokens, int topk, int num_experts) {
  if (num_tokens < 0 || topk <= 0 || num_experts <= 0) return 0;
  return mxb::route_workspace_bytes(num_tokens, topk, num_experts);
}

int mxmoe_route_topk(const mxmoe_route_args* a, void* stream) {
  if (!a) return fail(MXMOE_ERR_INVALID, "null args");
  if (a->num_tokens < 0 || a->topk <= 0 || a->num_experts <= 0 || a->num_experts > 512)
    return fail(MXMOE_ERR_INVALID, "bad routing shape T=%d topk=%d E=%d (E <= 512)", a->num_tokens, a->topk, a->num_experts);
  if ((long long)a->num_tokens * a->topk > 0x3fffffffLL) return fail(MXMOE_ERR_INVALID, "too many (token, slot) pairs");
  if (!a->counts || !a->row_start || !a->workspace) return fail(MXMOE_ERR_INVALID, "null output or workspace pointer");
  if (a->num_tokens > 0 && (!a->topk_ids || !a->row_expert || !a->row_token || !a->slot_row))
    return fail(MXMOE_ERR_INVALID, "null pointer in routing arguments");
  if (a->workspace_bytes < mxb::route_workspace_bytes(a->num_tokens, a->topk, a->num_experts))
    return fail(MXMOE_ERR_WORKSPACE, "routing workspace of %zu B is too small", a->workspace_bytes);
  mxb::RouteArgs r;
  r.topk_ids = a->topk_ids; r.counts = a->counts; r.row_start = a->row_start; r.row_expert = a->row_expert;
  r.row_token = a->row_token; r.slot_row = a->slot_row; r.workspace = a->workspace;
  r.workspace_bytes = a->workspace_bytes;
  r.num_tokens = a->num_tokens; r.topk = a->topk; r.num_experts = a->num_experts;
  r.num_ids = a->num_ids > 0 ? a->num_ids : a->num_experts;
  r.id_map = a->id_map; r.rep_base = a->rep_base; r.rep_count = a->rep_count;
  if (r.rep_base && (!r.id_map || !r.rep_count)) return fail(MXMOE_ERR_INVALID, "rep_base needs id_map and rep_count");
  CUDA_TRY(mxb::launch_route(r, static_cast<cudaStream_t>(stream)));
  return MXMOE_OK;
}

int mxmoe_route_topk_static(const mxmoe_route_args* a, void* stream) {
  if (!a) return fail(MXMOE_ERR_INVALID, "null args");
  if (a->num_tokens < 0 || a->topk <= 0 || a->num_experts <= 0 || a->num_experts > 512)
    return fail(MXMOE_ERR_INVALID, "bad routing shape T=%d topk=%d E=%d (E <= 512)", a->num_tokens, a->topk, a->num_experts);
  if ((long long)a->num_tokens * a->topk > 0x3fffffffLL) return fail(MXMOE_ERR_INVALID, "too many (token, slot) pairs");
  if (!a->counts || !a->row_start) return fail(MXMOE_ERR_INVALID, "null output pointer");
  if (a->num_tokens > 0 && (!a->topk_ids || !a->row_expert || !a->row_token || !a->slot_row))
    return fail(MXMOE_ERR_INVALID, "null pointer in routing arguments");
  const size_t need = mxb::route_workspace_bytes(a->num_tokens, a->topk, a->num_experts) / sizeof(int);
  if (need > mxb::route_static_scratch_ints())
    return fail(MXMOE_ERR_WORKSPACE,
                "routing %d x %d pairs over %d experts needs %zu scratch words; the built-in scratch holds %zu "
                "(ceil(T*topk/1024) * E must not exceed it) - use mxmoe_route_topk with a workspace instead",
                a->num_tokens, a->topk, a->num_experts, need, mxb::route_static_scratch_ints());
  int* scratch = nullptr;
  CUDA_TRY(mxb::route_static_scratch_ptr(&scratch));
  mxb::RouteArgs r;
  r.topk_ids = a->topk_ids; r.counts = a->counts; r.row_start = a->row_start; r.row_expert = a->row_expert;
  r.row_token = a->row_token; r.slot_row = a->slot_row; r.workspace = scratch;
  r.workspace_bytes = mxb::route_static_scratch_ints() * sizeof(int);
  r.num_tokens = a->num_tokens; r.topk = a->topk; r.num_experts = a->num_experts;
  r.num_ids = a->num_ids > 0 ? a->num_ids : a->num_experts;
  r.id_map = a->id_map; r.rep_base = a->rep_base; r.rep_count = a->rep_count;
  if (r.rep_base && (!r.id_map || !r.rep_count)) return fail(MXMOE_ERR_INVALID, "rep_base needs id_map and rep_count");
  CUDA_TRY(mxb::launch_route(r, static_cast<cudaStream_t>(stream)));
  return MXMOE_OK;
}

namespace {
__global__ void fetch_host_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, size_t n16) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) dst[i] = src[i];
}
}  // namespace

int mxmoe_fetch_host(void* dst, const void* src, size_t bytes, void* stream) {
  if (bytes == 0) return MXMOE_OK;
  if (!dst || !src) return fail(MXMOE_ERR_INVALID, "null pointer");
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  cudaPointerAttributes at;
  const bool mapped = cudaPointerGetAttributes(&at, src) == cudaSuccess && at.type == cudaMemoryTypeHost &&
                      at.devicePointer != nullptr;
  if (!mapped) cudaGetLastError();   // an unregistered pointer leaves an error behind on older runtimes
  const bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | bytes) & 15) == 0;
  if (!mapped || !aligned || bytes > (size_t)(4 << 20)) {
    CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, cs));
    return MXMOE_OK;
  }
  const size_t n16 = bytes / 16;
  const int blocks = (int)std::min<size_t>(64, (n16 + 255) / 256);
  fetch_host_kernel<<<blocks, 256, 0, cs>>>(static_cast<uint4*>(dst), static_cast<const uint4*>(at.devicePointer), n16);
  CUDA_TRY(cudaGetLastError());
  return MXMOE_OK;
}

int mxmoe_combine_topk(const void* y, const int32_t* slot_row, const float* topk_weights, const void* y_shared,
                       void* out, int num_tokens, int topk, int hidden, void* stream) {
  if (!y || !slot_row || !out) return fail(MXMOE_ERR_INVALID, "null pointer in combine arguments");
  if (num_tokens < 0 || topk <= 0 || hidden <= 0 || hidden % 8) return fail(MXMOE_ERR_INVALID, "bad combine shape T=%d topk=%d H=%d (H %% 8 == 0)", num_tokens, topk, hidden);
  CUDA_TRY(mxb::launch_combine(y, slot_row, topk_weights, y_shared, out, num_tokens, topk, hidden,
                               static_cast<cudaStream_t>(stream)));
  return MXMOE_OK;
}


int mxmoe_gate_topk(const void* logits, int logits_fp16, int num_tokens, int num_experts, int topk, int renormalize,
                    int32_t* topk_ids, float* topk_weights, void* stream) {
  if (!logits || !topk_ids || !topk_weights) return fail(MXMOE_ERR_INVALID, "null pointer in gate arguments");
  if (num_tokens < 0 || num_experts <= 0 || num_experts > 512 || topk <= 0 || topk > 32 || topk > num_experts)
    return fail(MXMOE_ERR_INVALID, "bad gate shape T=%d E=%d topk=%d (E <= 512, topk <= min(32, E))", num_tokens, num_experts, topk);
  CUDA_TRY(mxb::launch_gate_topk(logits, logits_fp16 != 0, num_tokens, num_experts, topk, renormalize, topk_ids,
                                 topk_weights, static_cast<cudaStream_t>(stream)));
  return MXMOE_OK;
}

int mxmoe_hadamard_kron(const void* in, void* out, const void* had_k, int rows, int k, int m, float scale, int fwht8,
                        void* stream) {
  if (!in || !out || !had_k) return fail(MXMOE_ERR_INVALID, "null pointer in Hadamard arguments");
  if (rows < 0 || k < 1 || k > 176 || m < 8 || (m & (m - 1)) != 0)
    return fail(MXMOE_ERR_UNSUPPORTED, "Hadamard factor K=%d (1..176) with m=%d (a power of two >= 8) is not supported", k, m);
  if (fwht8 && m != 8) return fail(MXMOE_ERR_INVALID, "the fused 8-point transform needs m == 8 (m=%d)", m);
  if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return fail(MXMOE_ERR_INVALID, "Hadamard rows must be 16-byte aligned");
  CUDA_TRY(mxb::launch_had_kron(static_cast<const __half*>(in), static_cast<__half*>(out),
                                static_cast<const __half*>(had_k), rows, k, m, scale, fwht8 != 0,
                                static_cast<cudaStream_t>(stream)));
  return MXMOE_OK;
}

int mxmoe_ep_plan(const mxmoe_ep_plan_args* a, void* stream) {
  if (!a) return fail(MXMOE_ERR_INVALID, "null args");
  if (a->world <= 0 || a->world > 64 || a->rank < 0 || a->rank >= a->world || a->num_experts <= 0 ||
      a->num_experts > 4096 || a->experts_local < 0 || a->recv_capacity < 0)
    return fail(MXMOE_ERR_INVALID, "bad expert-parallel shape world=%d rank=%d experts=%d local=%d capacity=%d", a->world,
                a->rank, a->num_experts, a->experts_local, a->recv_capacity);
  if (!a->counts_all || !a->range_lo || !a->seg_m || !a->seg_row0 || !a->seg_src_row0 || !a->recv_row_expert ||
      !a->total_recv || !a->dst_row0 || !a->exp_owner)
    return fail(MXMOE_ERR_INVALID, "null table");
  if (a->layout != 0 && a->layout != 1) return fail(MXMOE_ERR_INVALID, "unknown receive-store layout %d", a->layout);
  const int n_opt = (a->exp_m != nullptr) + (a->exp_row0 != nullptr) + (a->row_dst != nullptr) + (a->peer_ret != nullptr);
  if (n_opt != 0 && (n_opt != 4 || a->layout != 1 || a->ret_row_bytes <= 0 || a->ret_row_bytes % 16))
    return fail(MXMOE_ERR_INVALID, "exp_m, exp_row0, row_dst and peer_ret go together, with layout 1 and a row size that is a multiple of 16");
  static_assert(sizeof(mxmoe_ep_plan_args) == sizeof(mxb::EpPlanArgs), "plan args layout");
  mxb::EpPlanArgs k;
  std::memcpy(&k, a, sizeof(k));
  CUDA_TRY(mxb::launch_ep_plan(k, static_cast<cudaStream_t>(stream)));
  return MXMOE_OK;
}

int mxmoe_ep_sync(const mxmoe_ep_sync_args* a, void* stream) {
  if (!a) return fail(MXMOE_ERR_INVALID, "null args");
  if (a->world <= 0 || a->world > 64 || a->rank < 0 || a->rank >= a->world || a->payload_len < 0 ||
      a->payload_len > a->payload_cap || !a->peer_sync || !a->local_sync)
    return fail(MXMOE_ERR_INVALID, "bad barrier arguments world=%d rank=%d payload=%d/%d", a->world, a->rank,
                a->payload_len, a->payload_cap);
  static_assert(sizeof(mxmoe_ep_sync_args) == sizeof(mxb::EpSyncArgs), "sync args layout");
  mxb::EpSyncArgs k;
  std::memcpy(&k, a, sizeof(k));
  CUDA_TRY(mxb::launch_ep_sync(k, static_cast<cudaStream_t>(stream)));
  return MXMOE_OK;
}

int mxmoe_ep_dispatch_rows(const mxmoe_ep_dispatch_args* a, const mxmoe_token_quant_args* stores, void* stream) {
  if (!a) return fail(MXMOE_ERR_INVALID, "null args");
  mxb::TokenQuantArgs t;
  int rc = to_token_args(stores, &t);
  if (rc) return rc;
  if (a->rows < 0 || a->k != t.k || a->rec_bytes <= 0 || a->rec_bytes % 16 || a->scale_off_bytes < 0 ||
      a->scale_off_bytes + 2 > a->rec_bytes || a->scale_off_bytes % 2)
    return fail(MXMOE_ERR_INVALID, "bad dispatch shape rows=%d k=%d rec_bytes=%d scale_off=%d", a->rows, a->k, a->rec_bytes,
                a->scale_off_bytes);
  if (!a->peer_base || !a->row_expert || !a->row_token || !a->exp_row_start || !a->exp_qtag || !a->dst_row0 || !a->exp_owner)
    return fail(MXMOE_ERR_INVALID, "null table");
  static_assert(sizeof(mxmoe_ep_dispatch_args) == sizeof(mxb::EpDispatchArgs), "dispatch args layout");
  mxb::EpDispatchArgs k;
  std::memcpy(&k, a, sizeof(k));
  CUDA_TRY(mxb::launch_ep_dispatch(k, t, static_cast<cudaStream_t>(stream)));
  return MXMOE_OK;
}

}  // extern "C"
