// Device-side routing (token -> expert permutation) and weighted combine.
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

namespace mxb {

struct RouteArgs {
  const int* topk_ids;   // [T, topk] expert of every (token, slot)
  int* counts;           // [E]      rows per expert
  int* row_start;        // [E + 1]  exclusive prefix of counts; row_start[E] = routed rows
  int* row_expert;       // [T*topk] expert of every sorted row
  int64_t* row_token;    // [T*topk] source token of every sorted row
  int* slot_row;         // [T*topk] sorted row of every (token, slot); -1 for an invalid expert id
  int* workspace;        // per-block histograms
  size_t workspace_bytes;
  int num_tokens, topk, num_experts;
  int num_ids;           // range of the ids in topk_ids when id_map is given (0: num_experts)
  // optional renumbering applied to every id as it is read: id -> id_map[ rep_base ? rep_base[id] + token % rep_count[id] : id ]
  // (expert-parallel layers: an expert replicated on several ranks is dealt to its copies by token index, then the
  // copies are renumbered rank-major)
  const int* id_map;
  const int* rep_base;
  const int* rep_count;
};

size_t route_workspace_bytes(int num_tokens, int topk, int num_experts);
cudaError_t launch_route(const RouteArgs& a, cudaStream_t stream);
// static-scratch variant (see route_kernels.cu)
size_t route_static_scratch_ints();
cudaError_t route_static_scratch_ptr(int** out);
// softmax + top-k router gate (logits fp32 or fp16 [T, E]) -> expert ids and weights [T, topk]
cudaError_t launch_gate_topk(const void* logits, bool fp16, int num_tokens, int num_experts, int topk, int renorm,
                             int* ids, float* wts, cudaStream_t stream);
cudaError_t launch_combine(const void* y, const int* slot_row, const float* topk_w, const void* y_shared, void* out,
                           int num_tokens, int topk, int hidden, cudaStream_t stream);

}  // namespace mxb
