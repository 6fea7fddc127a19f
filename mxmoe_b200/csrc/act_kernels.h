// Arguments of the activation prologue kernels (act_kernels.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace mxb {

// Rows [0, rows_routed) are expert-sorted routed rows; rows [rows_routed,
// rows_total) belong to the shared expert (pseudo-expert index num_experts) and
// map one-to-one onto tokens.  The four per-expert tables have num_experts (+1
// with a shared expert) entries and mirror the host tables of
// mxmoe/kernels/src/ref_bind.cu:475-505.
struct ActArgs {
  const __half* in;          // quant_act: hidden [T, k]; silu_mul_quant: gate_up rows [rows_routed, 2k]
  const __half* in_shared;   // silu_mul_quant only: shared-expert gate_up rows [T, 2 k_shared]
  __half* q_store;           // packed activations (offsets in halfs)
  __half* s_store;           // per-token scales
  const int* row_expert;     // [rows_routed] expert of each sorted row
  const int64_t* row_token;  // [rows_routed] source token of each sorted row (quant_act only)
  const int* exp_qtag;       // 0 fp16 copy, 1 int8/token, 2 int4/token packed, 3 int4/token expanded to bytes
  const int* exp_row_start;  // first row of each expert
  const int* exp_q_off;      // write offset into q_store (halfs)
  const int* exp_s_off;      // write offset into s_store (halfs)
  const int8_t* signs;       // optional +-1 diagonal of the rotation (length k), or nullptr
  int k;                     // row length of routed rows
  int k_shared;              // row length of shared-expert rows
  int rows_routed;
  int rows_total;
  int num_experts;
  int rotate;                // 1: apply y = (x .* signs) H / sqrt(k) before quantising
  int rec_stride;            // > 0: record layout, row r at q_store + r * rec_stride (fp16 elements)
  int rec_scale_off;         // record layout: scale at this offset inside the record, or < 0: s_store[r]
  const int* rows_dev;       // optional live row count in device memory (quant_act, silu_mul_quant; no shared rows)
};

// Per-token quantisation into token-major stores; a store pointer that is null is not produced.
struct TokenQuantArgs {
  const __half* in;     // hidden [T, k]
  __half* f16;          // rotated fp16 rows [T, k]            (needed only when rotating)
  __half* q8;           // int8 rows  [T, k/2] uint16 words
  __half* s8;           // [T]
  __half* q4;           // int4 rows  [T, k/4] uint16 words
  __half* s4;           // [T]  (shared by q4 and q4x)
  __half* q4x;          // int4 rows expanded to one byte 16*q per code [T, k/2] (the GEMM's a_expanded format)
  const int8_t* signs;  // optional +-1 diagonal, length k
  int k;
  int num_tokens;
  int rotate;
  int reserved;
};

cudaError_t launch_quant_tokens(const TokenQuantArgs& t, cudaStream_t stream);
// rows of `a` (tables as for quant_act; a.in unused) are copied from the stores of `t`
cudaError_t launch_gather_rows(const ActArgs& a, const TokenQuantArgs& t, cudaStream_t stream);
// quant_tokens + gather_rows in one pass: rows of `r` (routed rows only) are written from registers, topk <= 8
cudaError_t launch_quant_tokens_scatter(const TokenQuantArgs& t, const ActArgs& r, const int* slot_row, int topk,
                                        cudaStream_t stream);
cudaError_t launch_quant_act(const ActArgs& a, cudaStream_t stream);
cudaError_t launch_silu_mul_quant(const ActArgs& a, cudaStream_t stream);

}  // namespace mxb
