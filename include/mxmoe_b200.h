/* mxmoe_b200 - C ABI of the B200 (sm_100a) mixed-precision MoE grouped GEMM.
 *
 * Plain C: pointers, sizes, CUDA stream handles (passed as void*).  Every entry
 * point returns an mxmoe_status (0 = ok); mxmoe_last_error() gives the text of
 * the last failure on the calling thread.  Nothing here terminates the process
 * (the reference's `checkCudaErrors` -> exit(1), mxmoe/kernels/src/include/helper.h:186-198,
 * becomes a status code) and nothing on the launch path allocates memory.
 *
 * "reference" paths below are relative to the MxMoE checkout.
 */
#ifndef MXMOE_B200_H_
#define MXMOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum mxmoe_status {
  MXMOE_OK              = 0,
  MXMOE_ERR_INVALID     = 1, /* bad argument (null pointer, misaligned buffer, bad shape) */
  MXMOE_ERR_UNSUPPORTED = 2, /* quantisation scheme not built into this library */
  MXMOE_ERR_CUDA        = 3, /* a CUDA runtime / driver call failed */
  MXMOE_ERR_WORKSPACE   = 4, /* workspace too small or not prepared */
  MXMOE_ERR_DEVICE      = 5, /* the kernel reported an error (bounded wait ran out, ...) */
  MXMOE_ERR_NO_DEVICE   = 6  /* no CUDA device / not an sm_100 device */
} mxmoe_status;

/* Per-problem quantisation descriptor.  Same 16-byte layout as the reference's
 * `mxmoe::QParams {int2 qbits(a_bits, w_bits); int gsize; bool sym;}`
 * (mxmoe/kernels/src/include/quantize.cuh:14-25). */
typedef struct mxmoe_qparams {
  int32_t a_bits;
  int32_t w_bits;
  int32_t gsize;
  uint8_t sym;
  uint8_t pad_[3];
} mxmoe_qparams;

/* One problem C[M,N] = A[M,K] x B[N,K]^T of a grouped launch; all pointers are
 * device pointers.  Layouts are the reference's (mxmoe/kernels/src/include/layout.cuh:26-31,
 * packed operands mxmoe/kernels/src/include/quantize.cuh:299-475):
 *   fp16   (16,16)          A fp16 [M,K],            B fp16 [N,K]
 *   w8a8   (8,8,-1,sym)     A u16 [M,K/2],           B u16 [N,K/2]   scale_a fp16 [M], scale_b fp16 [N]
 *   w4a4   (4,4,-1,sym)     A u16 [M,K/4],           B u16 [N,K/4]   scale_a fp16 [M], scale_b fp16 [N]
 *   w4a16  (16,4,128,asym)  A fp16 [M,K],            B u16 [N/4,K]   scale_b fp16 [K/128][N][2] (scale, zero)
 *   w4a16  (16,4,-1,asym)   A fp16 [M,K],            B u16 [N/4,K]   scale_b fp16 [N][2] (scale, zero), one pair per channel
 *                           (the reference's per-channel weight-only branch, cta_gemm.cuh:112-286; default kernel only)
 * C is fp16 [M,N] (row pitch ldc elements, 0 = N).  With out_mode 1 the raw
 * accumulators are stored instead (int32 for w8a8/w4a4, fp32 otherwise).
 * With out_mode 2 (default kernel, not for w4a16) B is a gate_up weight [gate rows (I); up rows (I)], N = 2 I with
 * I a multiple of 64, and C is fp16 [M, I] (ldc 0 = I): C = fp16(fp16(silu(gate)) * up) computed from the scaled
 * fp16 results in the epilogue -- the bits mxmoe_silu_mul_then_quant makes of the [M, 2 I] rows of out_mode 0
 * before it quantises (reference: the first half of silu_mul_then_quant_kernel, ref_bind.cu:701-716).
 *
 * Rows: the problem covers rows [row0, row0 + M) of A, scale_a and C.  `a_rows`
 * is the number of rows the A buffer holds (0 = row0 + M); it bounds what the
 * TMA unit may touch.  If `m_dev` is set, the live row count is read on the
 * device from *m_dev (clamped to M); if `row0_dev` is set, row0 is read from
 * *row0_dev.  Both let a launch follow a routing result that never visits the host.
 * `lda_bytes` / `sa_stride` describe activation stores made of fixed-size records (one per row,
 * possibly wider than the packed row, possibly carrying the row's scale): rows of different
 * formats then share one buffer and one row numbering. */
typedef struct mxmoe_gg_problem {
  const void* A;
  const void* B;
  const void* scale_a;
  const void* scale_b;
  void* C;
  const int32_t* m_dev;
  const int32_t* row0_dev;
  int32_t M, N, K;
  int32_t a_rows;
  int32_t row0;
  int32_t ldc;
  mxmoe_qparams q;
  int32_t out_mode;
  int32_t lda_bytes; /* row pitch of A in bytes; 0 = dense rows.  A multiple of 16. */
  int32_t sa_stride; /* distance between consecutive per-token scales in fp16 elements; 0 or 1 = contiguous */
  int32_t a_expanded; /* w4a4 only: A holds one byte per code, the byte 16*q, in the order the kernel's own
                         int4 -> int8 unpacking produces (see mxmoe_token_quant_args.q4x); A is then [M, K] bytes */
  int32_t reserved_;
  const int32_t* c_row0_dev; /* optional: the rows of C start at *c_row0_dev instead of at row0 (A and scale_a keep
                                row0).  Lets an expert-parallel rank store a segment's results straight into the
                                buffer of the rank the rows came from, at their place in that rank's order; C may
                                then be peer memory (plain stores). */
  const int64_t* c_row_ptrs; /* optional (default kernel, fp16 results, N and ldc multiples of 8): device table indexed
                                like the rows of A; row r of the result is stored at the ADDRESS c_row_ptrs[r] (+ the
                                column offset) instead of into C.  The rows of one problem may then go to different
                                buffers, e.g. to the ranks its rows came from; each row leaves in 256-byte pieces
                                through the copy engine.  Addresses must be 16-byte aligned. */
} mxmoe_gg_problem;

/* ---- library ---------------------------------------------------------------- */
const char* mxmoe_last_error(void);
int mxmoe_version(void);
/* Number of SMs of the current device, or a negative mxmoe_status. */
int mxmoe_device_sm_count(void);

/* ---- grouped GEMM ------------------------------------------------------------
 * Replaces the generated host launcher `groupgemm_hz_fused_<i>` and its kernel
 * (reference: mxmoe/kernels/kernel_sketch.py:82-145, mxmoe/kernels/compose_kernel.py:150-295).
 * The per-call cudaMalloc / cudaMemcpy / cudaFree of the reference launcher is
 * replaced by a caller-owned workspace. */

/* Bytes of device workspace needed for `problem_count` problems. */
size_t mxmoe_gg_workspace_bytes(int problem_count);

/* Host-side record of what mxmoe_gg_prepare put into a workspace. */
typedef struct mxmoe_gg_plan {
  int32_t count;     /* problems kept (empty ones are dropped) */
  int32_t needs_cvt; /* kernel variant: 0 no 4-bit operand, 1 4-bit weights only, 2 packed 4-bit activations too */
  int32_t flags;     /* bit 0: a problem redirects its C rows (c_row0_dev) or uses w4a16_g-1_asym: only the SWAP kernel can run it;
                        bit 2: a problem uses an optional result form (out_mode 2, c_row0_dev, c_row_ptrs): the launch runs the
                               kernel instance that has them, the weight tensor maps have rank 4;
                        bit 1: SWAP kernel with token tiles of 32 rows and a ring of 10 stages, 7 of two K blocks with 4-bit weights (set by prepare when no
                        problem has more than 32 rows; the caller may set or clear it before mxmoe_gg_run, e.g. set
                        it when the row counts come from device memory and are known to be small on average) */
  int32_t kernel;    /* the kernel mxmoe_gg_run launches (an mxmoe_gg_kernel value): chosen by mxmoe_gg_prepare from the
                        environment variable MXMOE_GG_KERNEL (swap | single | pair; default swap) */
} mxmoe_gg_plan;

/* Validate the problem list, encode the TMA descriptors on the host and copy the
 * device-side problem list into `workspace` (asynchronously on `stream`).
 * Problems with M == 0 (and no m_dev) are dropped.  `plan` receives what
 * mxmoe_gg_run needs to know about the prepared workspace. */
int mxmoe_gg_prepare(const mxmoe_gg_problem* problems, int problem_count, void* workspace, size_t workspace_bytes,
                     void* stream, mxmoe_gg_plan* plan);

/* Launch the persistent kernel over a prepared workspace; may be called any number of times after
 * one prepare.  `num_ctas` == 0: the plan's kernel on every SM; > 0: the plan's kernel with that
 * many CTAs; < 0: the CTA-pair kernel with -num_ctas CTAs (rounded down to even).  Nothing on this
 * path reads the environment or allocates.  All kernels give identical results. */
int mxmoe_gg_run(void* workspace, const mxmoe_gg_plan* plan, int num_ctas, void* stream);

/* The same with the kernel named explicitly. */
enum mxmoe_gg_kernel {
  MXMOE_GG_KERNEL_DEFAULT = 0,
  MXMOE_GG_KERNEL_SINGLE = 1, /* one CTA per tile of 128 rows x 256 channels, both operands from shared memory */
  MXMOE_GG_KERNEL_PAIR = 2,   /* tcgen05 cta_group::2, 256 x 256 tiles on clusters of two CTAs */
  MXMOE_GG_KERNEL_SWAP = 3,   /* swapped operands: 128 channels x up to 176 tokens per tile (128 when a problem has
                                 packed 4-bit activations), 4-bit weights converted into tensor memory */
  MXMOE_GG_KERNEL_SWAP2 = 4   /* the same on CTA pairs (tcgen05 cta_group::2): 256 channels x up to 176 tokens, each CTA
                                 loads half of the token tile; falls back to SWAP for launches with 32-token tiles or
                                 packed 4-bit activations */
};
int mxmoe_gg_run_kernel(void* workspace, const mxmoe_gg_plan* plan, int kernel, int num_ctas, void* stream);

/* prepare + run */
int mxmoe_gg_launch(const mxmoe_gg_problem* problems, int problem_count, void* workspace, size_t workspace_bytes,
                    void* stream);

/* Synchronise `stream` and read the device status block of the workspace:
 * MXMOE_OK, or MXMOE_ERR_DEVICE with the detail in mxmoe_last_error().  A reported error is cleared,
 * so that the workspace can be launched again. */
int mxmoe_gg_check(void* workspace, void* stream);

/* Test hook for the bounded waits of the kernel with swapped operands (no counterpart in the reference, whose
 * kernels cannot time out).  `timeout_ms` > 0 replaces the 1000 ms limit of every device-side wait of later
 * launches over `workspace`; `skip_stage` >= 0 makes the producer of CTA 0 announce more weight bytes than it
 * loads for that pipeline stage (counted from the start of its work), so that the wait for them runs out: the launch then ends
 * by itself and mxmoe_gg_check reports MXMOE_ERR_DEVICE with the role and the tile.  (0, -1) restores the
 * defaults.  Synchronises `stream`. */
int mxmoe_gg_debug(void* workspace, int timeout_ms, int skip_stage, void* stream);

/* Built-in tracing: cycle counters (clock64 deltas) that CTA 0 recorded during the last launch over
 * `workspace`.  counters[16]: 0 kernel body, 1 producer waiting for a free stage, 2 MMA issuer waiting
 * for operands, 3 MMA issuer waiting for a drained accumulator, 4 MMA issue, 5 epilogue waiting,
 * 6 epilogue draining + storing, 7 converter waiting, 8 converter working, 9 tiles, 10 stages.
 * Synchronises `stream`. */
int mxmoe_gg_profile(void* workspace, uint64_t* counters, void* stream);

/* Drop-in for the reference's function-pointer ABI `mxmoe::FuncType`
 * (mxmoe/kernels/src/include/registry.cuh:28-39): device arrays of device
 * pointers, host + device copies of the dim3 sizes (x=M, y=N, z=K) and QParams.
 * ld* are ignored as in the reference (mxmoe/kernels/src/ref_bind.cu:413 passes
 * nullptr); runs on the default stream and returns after the kernel finished. */
int mxmoe_groupgemm_hz_fused(void** ptr_As, void** ptr_Bs, void** ptr_scale_a, void** ptr_scale_b, void** ptr_Cs,
                             void** ptr_Ds, int64_t* ldas, int64_t* ldbs, int64_t* ldcs, int64_t* ldds,
                             const uint32_t* device_problem_sizes, const uint32_t* host_problem_sizes,
                             const mxmoe_qparams* device_qparams, const mxmoe_qparams* host_qparams,
                             int problem_count);

/* ---- activation prologues ----------------------------------------------------
 * Arguments common to both kernels.  Rows [0, rows_routed) are expert-sorted
 * routed rows, rows [rows_routed, rows_total) belong to the shared expert
 * (pseudo-expert `num_experts`).  The four per-expert device tables are the ones
 * the reference builds on the host at mxmoe/kernels/src/ref_bind.cu:475-505:
 * quantisation tag (0 fp16 copy, 1 int8 per token, 2 int4 per token, 3 int4 per token expanded to
 * one byte 16*q per code - an internal format of this library), first row,
 * write offset of the packed rows and of the scales (both in fp16 elements).
 * Record layout (rec_stride > 0): the three offset tables are not read; row r is written to
 * q_store + r * rec_stride whatever its format, and its scale to the same record at
 * rec_scale_off (or to s_store[r] if rec_scale_off < 0) - offsets that need no host knowledge
 * of the per-expert counts, and buffers that can be sent to another GPU as they are. */
typedef struct mxmoe_act_args {
  const void* in;             /* fp16 */
  const void* in_shared;      /* fp16, silu_mul_then_quant only */
  void* q_store;              /* packed activations */
  void* s_store;              /* fp16 per-token scales */
  const int32_t* row_expert;  /* [rows_routed] */
  const int64_t* row_token;   /* [rows_routed], quant_inp_act only; NULL (without rotation): row r of `in` is routed row r and
                                 the shared rows are the rows of `in_shared` -- the quantiser alone, rows_dev honoured */
  const int32_t* exp_qtag;
  const int32_t* exp_row_start;
  const int32_t* exp_q_off;
  const int32_t* exp_s_off;
  const int8_t* signs;        /* optional +-1 diagonal of the Hadamard rotation, length k */
  int32_t k;
  int32_t k_shared;
  int32_t rows_routed;
  int32_t rows_total;
  int32_t num_experts;
  int32_t rotate;             /* quant_inp_act only: rotate rows by diag(signs) H_k / sqrt(k) first */
  int32_t rec_stride;         /* > 0: record layout (see below), in fp16 elements */
  int32_t rec_scale_off;      /* record layout: offset of the scale inside the record, or < 0 for s_store[row] */
  const int32_t* rows_dev;    /* optional, quant_act / silu_mul_then_quant without shared rows: live row count in device memory;
                                 rows at or beyond it are skipped (rows_routed == rows_total is then an upper bound) */
} mxmoe_act_args;

/* Gather rows of `in` ([T,k] fp16) by expert, optionally rotate, quantise per
 * token and pack.  Replaces `quant_act_kernel` (launched at
 * mxmoe/kernels/src/ref_bind.cu:531-544). */
int mxmoe_quant_act(const mxmoe_act_args* args, void* stream);

/* Quantise once per token, then copy.  With top-k routing every token feeds topk experts, so the
 * rotation and the quantiser are evaluated once per token into token-major stores (one per
 * activation format in use; a NULL store is not produced) and mxmoe_gather_rows copies each routed
 * row from the store of its expert's format into the expert-sorted activation store.  The result is
 * bit-identical to mxmoe_quant_act. */
typedef struct mxmoe_token_quant_args {
  const void* in;      /* fp16 hidden [T, k] */
  void* f16;           /* rotated fp16 rows [T, k] (only needed when rotating and a 16-bit expert exists) */
  void* q8;            /* int8 rows [T, k/2] uint16 words */
  void* s8;            /* fp16 [T] */
  void* q4;            /* int4 rows [T, k/4] uint16 words */
  void* s4;            /* fp16 [T], shared by q4 and q4x */
  void* q4x;           /* int4 rows expanded to one byte 16*q per code, [T, k] bytes: the a_expanded operand
                          format of the grouped GEMM (tag 3 in exp_qtag); needs k % 32 == 0 */
  const int8_t* signs; /* optional +-1 diagonal, length k */
  int32_t k;
  int32_t num_tokens;
  int32_t rotate;
  int32_t reserved_;
} mxmoe_token_quant_args;

int mxmoe_quant_tokens(const mxmoe_token_quant_args* args, void* stream);
/* `rows` uses the tables of mxmoe_act_args (its `in` is ignored); every format tagged in
 * rows->exp_qtag must have its store in `stores` (tag 0 reads stores->f16, or stores->in if NULL). */
int mxmoe_gather_rows(const mxmoe_act_args* rows, const mxmoe_token_quant_args* stores, void* stream);
/* Both in one pass: every token's row is rotated and quantised once and written from registers to the
 * expert-sorted slot of each of its topk routing slots (slot_row[t * topk + s] = sorted row of slot s of token t,
 * as mxmoe_route_topk returns it; 1 <= topk <= 8; rows->rows_total == rows->rows_routed) in that expert's format,
 * and to the token-major stores of `stores` that are not NULL (a shared expert reads those).  Bit-identical to
 * mxmoe_quant_tokens followed by mxmoe_gather_rows; a store of a format only routed experts use may be NULL. */
int mxmoe_quant_tokens_scatter(const mxmoe_token_quant_args* stores, const mxmoe_act_args* rows, const int32_t* slot_row,
                               int32_t topk, void* stream);

/* h = silu(gate) * up over gate_up rows ([rows, 2k] fp16, gate first), then
 * quantise per token and pack for the down projection.  Replaces
 * `silu_mul_then_quant_kernel` (launched at mxmoe/kernels/src/ref_bind.cu:701-716). */
int mxmoe_silu_mul_then_quant(const mxmoe_act_args* args, void* stream);

/* Online Hadamard rotation of fp16 rows whose length n = k * m is not a power of two: `had_k` is a k x k Hadamard
 * matrix (fp16 +-1, row-major, device memory), m a power of two.  Replaces `matmul_hadU_cuda`
 * (mxmoe/quant/hadamard_utils.py:96-105), which the reference applies to the down-projection input when its online
 * rotation is on (mxmoe/quant/rotation.py:403-421):
 *     out[r, a*m + t] = scale * sum_a' had_k[a, a'] * z[r, a'*m + t]
 * with z = the rows after the natural-order Walsh-Hadamard transform over every group of m contiguous elements.
 * `fwht8` != 0 (m == 8 only): that transform is done here and scale is 1/sqrt(n); otherwise the caller has
 * already transformed the groups (mxmoe_quant_tokens with rotate over [rows * k, m], which scales by 1/sqrt(m))
 * and scale is 1/sqrt(k).  k <= 176; in == out is allowed. */
int mxmoe_hadamard_kron(const void* in, void* out, const void* had_k, int rows, int k, int m, float scale, int fwht8,
                        void* stream);

/* ---- device-side routing and combine -------------------------------------------
 * Stable counting sort of the (token, slot) pairs by expert, entirely on the
 * device.  Produces what the reference gets from torch::sort / floor_divide /
 * bincount(...).cpu() (mxmoe/kernels/src/ref_bind.cu:47-64, :449-453) without the
 * host round trip: counts[E], row_start[E+1] (exclusive prefix; row_start[E] is
 * the number of routed rows), row_expert / row_token per sorted row (the
 * reference's dst_exp_sorted / perm_indices) and slot_row, the inverse map. */
typedef struct mxmoe_route_args {
  const int32_t* topk_ids; /* [T, topk] */
  int32_t* counts;         /* [E] */
  int32_t* row_start;      /* [E + 1] */
  int32_t* row_expert;     /* [T * topk] */
  int64_t* row_token;      /* [T * topk] */
  int32_t* slot_row;       /* [T * topk]; -1 where the expert id is out of range */
  int32_t* workspace;      /* mxmoe_route_workspace_bytes() bytes */
  size_t workspace_bytes;
  int32_t num_tokens, topk, num_experts;
  int32_t num_ids;         /* with id_map: the ids in topk_ids lie in [0, num_ids); 0 = num_experts */
  /* Optional renumbering, applied to every id as it is read (NULL = none): id -> id_map[v] with
   * v = rep_base ? rep_base[id] + token % rep_count[id] : id.  An expert-parallel layer deals the rows of an expert
   * that is replicated on several ranks to its copies by token index and numbers the copies rank-major. */
  const int32_t* id_map;
  const int32_t* rep_base;
  const int32_t* rep_count;
} mxmoe_route_args;

size_t mxmoe_route_workspace_bytes(int num_tokens, int topk, int num_experts);
int mxmoe_route_topk(const mxmoe_route_args* args, void* stream);

/* Same routing as mxmoe_route_topk for callers that cannot allocate device memory where they
 * route (a serving loop whose memory pool is fixed at start-up, a plug-in that only receives
 * its input and output buffers): `workspace` / `workspace_bytes` of the arguments are ignored
 * and the per-block histograms go to a 256 KiB array built into the library.  This entry point
 * has no counterpart in the reference.
 *   limit     ceil(T * topk / 1024) * num_experts <= 65536, otherwise MXMOE_ERR_WORKSPACE;
 *   memory    every GPU that loads the library holds the 256 KiB until the process exits;
 *   set-up    the first call on each device looks up the array's device address (no allocation):
 *             make that first call outside of any stream capture;
 *   sharing   all calls on one device use the same array.  Nothing in it has to start at zero
 *             (each call rewrites every word it later reads), but two calls whose kernels overlap
 *             on the GPU - different streams without an ordering between them - race on it.
 * It calls no cudaMalloc / cudaFree and no allocating library routine. */
int mxmoe_route_topk_static(const mxmoe_route_args* args, void* stream);

/* Router gate on the device: softmax over the expert logits of every token (fp32 arithmetic), the top-k
 * probabilities and their experts, renormalised to sum 1 if `renormalize` (the softmax -> topk -> norm_topk_prob
 * sequence of the MoE blocks the reference quantises; the reference itself takes the routing result from the
 * framework, mxmoe/kernels/src/ref_bind.cu:47-64).  logits: fp32, or fp16 if `logits_fp16`, [T, E] with
 * E <= 512; outputs [T, topk], topk <= 32; ties go to the lower expert index. */
int mxmoe_gate_topk(const void* logits, int logits_fp16, int num_tokens, int num_experts, int topk, int renormalize,
                    int32_t* topk_ids, float* topk_weights, void* stream);

/* out[t] = sum_j topk_weights[t,j] * y[slot_row[t,j]] (+ y_shared[t]); y is the
 * fp16 [rows, hidden] output of the down projection, accumulation in fp32.  The
 * reference leaves this step unimplemented (`gg_unpermute_out(){}`,
 * mxmoe/kernels/src/ref_bind.cu:66); topk_weights may be NULL (all ones). */
int mxmoe_combine_topk(const void* y, const int32_t* slot_row, const float* topk_weights, const void* y_shared,
                       void* out, int num_tokens, int topk, int hidden, void* stream);

/* Small host -> device transfer done by a KERNEL that reads page-locked (mapped) host memory, for serving loops
 * whose copy engines are busy with large transfers: a 131 KB routing table queued as a DMA copy behind a 33 MB
 * one held the copy-in stream of the 8192-token layer for 50 us (measured).  `src` must be page-locked host memory
 * that the device can address (cudaHostAlloc / cudaHostRegister; what torch's pin_memory() returns) and must stay
 * unchanged until the stream reaches the call; dst, src and bytes are multiples of 16.  Anything else is handed to
 * cudaMemcpyAsync.  No counterpart in the reference. */
int mxmoe_fetch_host(void* dst, const void* src, size_t bytes, void* stream);

/* ---- expert parallel ----------------------------------------------------------
 * No reference counterpart: the reference has no distributed code.  One process per GPU; experts are
 * numbered so that rank r owns the contiguous range [range_lo[r], range_lo[r+1]).  mxmoe_ep_plan turns the
 * all-gathered routing counts into this rank's receive-side segment tables and send-side row offsets, on
 * the device; mxmoe_ep_dispatch_rows writes every quantised row of this rank (packed row + scale, one
 * record) straight into the receive store of the rank that owns its expert (plain stores to peer memory). */
typedef struct mxmoe_ep_plan_args {
  const int32_t* counts_all; /* [world][num_experts] */
  const int32_t* range_lo;   /* [world + 1] */
  int32_t world, rank, num_experts, experts_local, recv_capacity;
  int32_t layout;           /* order of the rows in a receive store: 0 = (source rank, expert), 1 = (expert, source rank) */
  int32_t* seg_m;           /* [world * experts_local] rows of segment (source rank, local expert), indexed source-major */
  int32_t* seg_row0;        /* first row of the segment in this rank's receive store */
  int32_t* seg_src_row0;    /* first row of the same rows in the source rank's expert-sorted order */
  int32_t* recv_row_expert; /* [recv_capacity] expert of every received row */
  int32_t* total_recv;      /* [0] rows received (clamped), [1] rows wanted when that exceeded the capacity */
  int32_t* dst_row0;        /* [num_experts] first row of this rank's rows for expert e in its owner's store */
  int32_t* exp_owner;       /* [num_experts] */
  /* layout 1, optional (all or none): with an expert's rows contiguous whatever rank sent them, the grouped GEMMs
   * take ONE problem per local expert (m_dev = exp_m + j, row0_dev = exp_row0 + j) instead of one per (source rank,
   * expert), and the down projection finds the destination of every row in row_dst (mxmoe_gg_problem.c_row_ptrs). */
  int32_t* exp_m;           /* [experts_local] */
  int32_t* exp_row0;        /* [experts_local] */
  int64_t* row_dst;         /* [recv_capacity] address of the row's result in the home-coming buffer of its source rank */
  const uint64_t* peer_ret; /* [world] device array: home-coming buffer of every rank as mapped here */
  int32_t ret_row_bytes;
  int32_t reserved_;
} mxmoe_ep_plan_args;

typedef struct mxmoe_ep_dispatch_args {
  const uint64_t* peer_base;   /* [world] device array: receive store of every rank as mapped here */
  const int32_t* row_expert;   /* [rows] */
  const int64_t* row_token;    /* [rows] */
  const int32_t* exp_row_start;
  const int32_t* exp_qtag;     /* activation format per expert, as in mxmoe_act_args */
  const int32_t* dst_row0;     /* from mxmoe_ep_plan */
  const int32_t* exp_owner;    /* from mxmoe_ep_plan */
  int32_t rows, k, rec_bytes, scale_off_bytes, recv_capacity;
  int32_t reserved_;
} mxmoe_ep_dispatch_args;

/* Stream-ordered barrier between the ranks (one process per GPU): every rank's earlier kernels on its stream, their
 * stores to peer memory included, have completed before any rank's later kernels start.  Each rank owns a "sync
 * block" of int32 in peer-mapped (symmetric) memory, zero-initialised once: [0, 64) arrival flags by rank, [64] error
 * word, [65] epoch, [128, 128 + world * payload_cap) payload slots by rank (mxmoe_ep_sync_block_ints gives the
 * size).  With `payload` set, payload_len int32 of this rank are written into slot `rank` of every peer before the
 * barrier: the all-gather of the per-expert row counts.  The wait for the peers is bounded (timeout_ms, 0 = 2000 ms);
 * when it runs out, local_sync[64] is set to 1 + the missing rank and the kernel returns.  No NCCL call, no host
 * involvement: a step built from it can be captured in a CUDA graph.  The ranks must run on different GPUs. */
typedef struct mxmoe_ep_sync_args {
  const uint64_t* peer_sync; /* [world] device array: every rank's sync block as mapped here */
  int32_t* local_sync;       /* this rank's sync block */
  const int32_t* payload;    /* optional */
  int32_t world, rank, payload_len, payload_cap;
  int32_t timeout_ms;
  int32_t reserved_;
} mxmoe_ep_sync_args;

int mxmoe_ep_sync(const mxmoe_ep_sync_args* args, void* stream);
int mxmoe_ep_plan(const mxmoe_ep_plan_args* args, void* stream);
int mxmoe_ep_dispatch_rows(const mxmoe_ep_dispatch_args* args, const mxmoe_token_quant_args* stores, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MXMOE_B200_H_ */
