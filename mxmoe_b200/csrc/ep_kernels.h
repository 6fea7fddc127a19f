// Arguments of the expert-parallel plan and dispatch kernels (ep_kernels.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "act_kernels.h"

namespace mxb {

// Experts are numbered so that rank r owns the contiguous range [range_lo[r], range_lo[r+1]).
struct EpPlanArgs {
  const int* counts_all;   // [world][num_experts] rows rank s routes to expert e (all-gathered)
  const int* range_lo;     // [world + 1]
  int world, rank, num_experts, experts_local, recv_capacity;
  int layout;              // order of the receive store: 0 = (source rank, expert), 1 = (expert, source rank)
  // receive side of this rank: segment i = (source rank i / experts_local, local expert i % experts_local)
  int* seg_m;              // [world * experts_local] rows of the segment
  int* seg_row0;           // first row of the segment in this rank's receive store
  int* seg_src_row0;       // first row of the same rows in the source rank's expert-sorted order
  int* recv_row_expert;    // [recv_capacity] expert of every received row
  int* total_recv;         // [0] rows received (clamped to the capacity), [1] rows wanted if that exceeded it
  // send side of this rank
  int* dst_row0;           // [num_experts] first row of this rank's rows for expert e in the owner's receive store
  int* exp_owner;          // [num_experts] rank that owns expert e
  // layout 1 (optional, all four or none): an expert's rows are contiguous whatever rank they came from
  int* exp_m;              // [experts_local] rows of local expert j
  int* exp_row0;           // [experts_local] its first row in the receive store
  int64_t* row_dst;        // [recv_capacity] where the result of received row r goes: address of its row in the
                           // home-coming buffer of the rank it came from
  const uint64_t* peer_ret;   // [world] home-coming buffer of every rank as mapped into this process
  int ret_row_bytes;       // bytes of one row of those buffers
  int pad_;
};

struct EpDispatchArgs {
  const uint64_t* peer_base;   // [world] receive store of every rank as mapped into this process
  const int* row_expert;       // [rows] expert of each expert-sorted row of this rank
  const int64_t* row_token;    // [rows] its token
  const int* exp_row_start;    // [num_experts] first sorted row of each expert
  const int* exp_qtag;         // [num_experts] activation format of each expert (see ActArgs::exp_qtag)
  const int* dst_row0;         // from the plan
  const int* exp_owner;        // from the plan
  int rows, k, rec_bytes, scale_off_bytes, recv_capacity;
  int pad_;
};

// Barrier between the ranks of an expert-parallel group that lives on the stream: every rank's kernels launched
// before it (their stores to peer memory included) have completed before any rank's kernels launched after it
// start.  Optionally carries a small payload (this rank's per-expert row counts) to every peer first, which makes it
// the all-gather of the counts as well.  All buffers are peer-mapped (symmetric) int32 memory.
struct EpSyncArgs {
  const uint64_t* peer_sync;   // [world] device array: address of every rank's sync block as mapped here
  int* local_sync;             // this rank's sync block: [0, 64) arrival flags by rank, [64] error word, [65] epoch,
                               // [128, 128 + world * payload_cap) payload slots by rank
  const int* payload;          // optional: payload_len int32 this rank publishes into slot `rank` of every peer
  int world, rank, payload_len, payload_cap;
  int timeout_ms;              // limit of the wait for the peers' flags; 0 = 2000 ms
  int pad_;
};

cudaError_t launch_ep_sync(const EpSyncArgs& a, cudaStream_t stream);
cudaError_t launch_ep_plan(const EpPlanArgs& a, cudaStream_t stream);
cudaError_t launch_ep_dispatch(const EpDispatchArgs& d, const TokenQuantArgs& t, cudaStream_t stream);

}  // namespace mxb
