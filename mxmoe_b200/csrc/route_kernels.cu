// Device-side routing for the MoE grouped GEMM: a stable counting sort of the
// (token, slot) pairs by expert, and the weighted un-permute of expert outputs.
//
// The reference does the permutation with torch::sort / bincount and copies the
// per-expert counts to the host (mxmoe/kernels/src/ref_bind.cu:47-64, :449-453),
// which costs a host synchronisation per layer; its un-permute is an empty stub
// (`gg_unpermute_out(){}`, ref_bind.cu:66).  Here the counts, the row offsets and
// the permutation stay on the device and feed the grouped GEMM's problem list
// directly.  Rows of one expert keep the order of the flattened (token, slot)
// index, i.e. the result equals a stable sort.
#include "route_kernels.h"

#include <cuda_fp16.h>

#include <mutex>

namespace mxb {
namespace {

constexpr int kChunk   = 1024;  // (token, slot) pairs per block
constexpr int kThreads = 256;
constexpr int kMaxE    = 512;

// expert of pair `idx` = (token, slot), renumbered if the caller gave a map; -1 for an id out of range
__device__ __forceinline__ int read_id(const RouteArgs& a, int idx) {
  int e = a.topk_ids[idx];
  if (a.id_map) {
    if (e < 0 || e >= a.num_ids) return -1;
    if (a.rep_base) e = a.rep_base[e] + (idx / a.topk) % a.rep_count[e];
    e = a.id_map[e];
  }
  return (e < 0 || e >= a.num_experts) ? -1 : e;
}

__global__ void __launch_bounds__(kThreads) route_count_kernel(RouteArgs a) {
  __shared__ int hist[kMaxE];
  const int n = a.num_tokens * a.topk;
  for (int e = threadIdx.x; e < a.num_experts; e += kThreads) hist[e] = 0;
  __syncthreads();
  const int base = blockIdx.x * kChunk;
  for (int i = threadIdx.x; i < kChunk; i += kThreads) {
    const int idx = base + i;
    if (idx < n) {
      const int e = read_id(a, idx);
      if (e >= 0) atomicAdd(&hist[e], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < a.num_experts; e += kThreads) a.workspace[blockIdx.x * a.num_experts + e] = hist[e];
}

// one block: per-expert exclusive prefix over blocks, then exclusive prefix over experts.  A warp owns an
// expert and scans its per-block counts 32 at a time (independent loads + a shuffle scan); one thread walking
// the blocks with a load -> store chain per step cost a global-memory latency per block.
constexpr int kScanThreads = 1024;
__global__ void __launch_bounds__(kScanThreads) route_scan_kernel(RouteArgs a, int nblocks) {
  __shared__ int total[kMaxE];
  __shared__ int start[kMaxE + 1];
  const int E = a.num_experts;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = warp; e < E; e += kScanThreads / 32) {
    int carry = 0;
    for (int b0 = 0; b0 < nblocks; b0 += 32) {
      const int b = b0 + lane;
      const int c = b < nblocks ? a.workspace[b * E + e] : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
      }
      if (b < nblocks) a.workspace[b * E + e] = carry + incl - c;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      total[e] = carry;
      a.counts[e] = carry;
    }
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const int c = e < E ? total[e] : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
      }
      if (e < E) start[e] = carry + incl - c;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) start[E] = carry;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += kScanThreads) a.row_start[e] = start[e];
  for (int i = threadIdx.x; i < nblocks * E; i += kScanThreads) a.workspace[i] += start[i % E];
}

// kSingle: the whole input is this one block's chunk (a decode batch) - the block also produces the counts and
// the row offsets itself, so the count and scan launches are not needed and no workspace is read.
template <bool kSingle>
__global__ void __launch_bounds__(kThreads) route_scatter_kernel(RouteArgs a) {
  __shared__ int wbase[kThreads / 32][kMaxE];
  __shared__ int start[kSingle ? kMaxE + 1 : 1];
  const int n    = a.num_tokens * a.topk;
  const int E    = a.num_experts;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kWarps   = kThreads / 32;
  constexpr int kPerWarp = kChunk / kWarps;  // contiguous pairs per warp
  for (int i = threadIdx.x; i < kWarps * kMaxE; i += kThreads) (&wbase[0][0])[i] = 0;
  __syncthreads();
  const int wstart = blockIdx.x * kChunk + warp * kPerWarp;
  // pass 1: per-warp histogram
  for (int p = 0; p < kPerWarp; p += 32) {
    const int idx = wstart + p + lane;
    int e = -1;
    if (idx < n) e = read_id(a, idx);
    const unsigned m = __match_any_sync(0xffffffffu, e);
    if (e >= 0 && (m & ((1u << lane) - 1)) == 0) wbase[warp][e] += __popc(m);
    __syncwarp();
  }
  __syncthreads();
  if (kSingle) {
    for (int e = threadIdx.x; e < E; e += kThreads) {
      int t = 0;
      for (int w = 0; w < kWarps; ++w) t += wbase[w][e];
      start[e]    = t;
      a.counts[e] = t;
    }
    __syncthreads();
    if (warp == 0) {
      int carry = 0;
      for (int e0 = 0; e0 < E; e0 += 32) {
        const int e = e0 + lane;
        const int c = e < E ? start[e] : 0;
        int incl = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int u = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += u;
        }
        if (e < E) start[e] = carry + incl - c;
        carry += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) start[E] = carry;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += kThreads) a.row_start[e] = start[e];
  }
  // exclusive prefix over the warps of the block, on top of the block's base
  for (int e = threadIdx.x; e < E; e += kThreads) {
    int run = kSingle ? start[e] : a.workspace[blockIdx.x * E + e];
    for (int w = 0; w < kWarps; ++w) { const int c = wbase[w][e]; wbase[w][e] = run; run += c; }
  }
  __syncthreads();
  // pass 2: place
  for (int p = 0; p < kPerWarp; p += 32) {
    const int idx = wstart + p + lane;
    int e = -1;
    if (idx < n) e = read_id(a, idx);
    const unsigned m  = __match_any_sync(0xffffffffu, e);
    const unsigned lt = m & ((1u << lane) - 1);
    if (e >= 0) {
      const int dst = wbase[warp][e] + __popc(lt);
      a.row_expert[dst] = e;
      a.row_token[dst]  = idx / a.topk;
      a.slot_row[idx]   = dst;
    } else if (idx < n) {
      a.slot_row[idx] = -1;
    }
    __syncwarp();
    if (e >= 0 && lt == 0) wbase[warp][e] += __popc(m);
    __syncwarp();
  }
}

// out[t] = sum_j w[t,j] * y[slot_row[t,j]] (+ y_shared[t]); fp32 accumulation, fp16 result
__global__ void __launch_bounds__(kThreads) combine_kernel(const __half* __restrict__ y, const int* __restrict__ slot_row,
                                                           const float* __restrict__ w, const __half* __restrict__ ysh,
                                                           __half* __restrict__ out, int topk, int hidden) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < hidden / 8; c += kThreads) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int j = 0; j < topk; ++j) {
      const int r = slot_row[t * topk + j];
      if (r < 0) continue;
      const float wt = w ? w[t * topk + j] : 1.f;
      const uint4 v  = __ldg(reinterpret_cast<const uint4*>(y + (int64_t)r * hidden) + c);
      const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h[e]);
        acc[2 * e] += wt * f.x;
        acc[2 * e + 1] += wt * f.y;
      }
    }
    if (ysh) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(ysh + (int64_t)t * hidden) + c);
      const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) oh[e] = __floats2half2_rn(acc[2 * e], acc[2 * e + 1]);
    reinterpret_cast<uint4*>(out + (int64_t)t * hidden)[c] = o;
  }
}

// Router gate: softmax over the expert logits of a token in fp32, the top-k probabilities and their experts,
// optionally renormalised to sum 1 (the gate of the MoE blocks the reference quantises: softmax -> topk ->
// norm_topk_prob).  One warp per token, up to 16 experts per lane; ties go to the lower expert index.
template <typename T>
__global__ void __launch_bounds__(kThreads) gate_topk_kernel(const T* __restrict__ logits, int num_tokens, int E, int topk,
                                                             int renorm, int* __restrict__ ids, float* __restrict__ wts) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (kThreads / 32) + warp;
  if (t >= num_tokens) return;
  constexpr int kPer = kMaxE / 32;
  float v[kPer];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < E ? (float)logits[(int64_t)t * E + e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    v[i] = (i * 32 + lane) < E ? __expf(v[i] - mx) : -1.f;   // -1: not a candidate
    sum += fmaxf(v[i], 0.f);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
  float picked = 0.f, mine_w = 0.f;
  int mine_id = 0;
  for (int j = 0; j < topk; ++j) {
    // lane-local best, then the warp's best (larger value, then lower index)
    float bv = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int e = i * 32 + lane;
      if (v[i] > bv) { bv = v[i]; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi   = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((bi & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kPer; ++i)
        if (i * 32 + lane == bi) v[i] = -1.f;
    }
    picked += bv * inv;
    if (lane == j) { mine_w = bv * inv; mine_id = bi; }
  }
  if (lane < topk) {
    ids[(int64_t)t * topk + lane] = mine_id;
    wts[(int64_t)t * topk + lane] = renorm ? mine_w / picked : mine_w;
  }
}

}  // namespace

cudaError_t launch_gate_topk(const void* logits, bool fp16, int num_tokens, int num_experts, int topk, int renorm,
                             int* ids, float* wts, cudaStream_t stream) {
  if (num_tokens <= 0) return cudaSuccess;
  if (num_experts > kMaxE || topk > 32 || topk > num_experts) return cudaErrorInvalidValue;
  const int blocks = (num_tokens + kThreads / 32 - 1) / (kThreads / 32);
  if (fp16) gate_topk_kernel<__half><<<blocks, kThreads, 0, stream>>>(static_cast<const __half*>(logits), num_tokens, num_experts, topk, renorm, ids, wts);
  else      gate_topk_kernel<float><<<blocks, kThreads, 0, stream>>>(static_cast<const float*>(logits), num_tokens, num_experts, topk, renorm, ids, wts);
  return cudaGetLastError();
}

size_t route_workspace_bytes(int num_tokens, int topk, int num_experts) {
  const long long n = (long long)num_tokens * topk;
  const long long nblocks = (n + kChunk - 1) / kChunk;
  return (size_t)(nblocks > 0 ? nblocks : 1) * (size_t)num_experts * sizeof(int);
}

cudaError_t launch_route(const RouteArgs& a, cudaStream_t stream) {
  const int n = a.num_tokens * a.topk;
  const int nblocks = (n + kChunk - 1) / kChunk;
  if (a.num_experts > kMaxE) return cudaErrorInvalidValue;
  if (nblocks == 1) {   // a decode batch: one launch does all three steps
    route_scatter_kernel<true><<<1, kThreads, 0, stream>>>(a);
    return cudaGetLastError();
  }
  if (nblocks > 0) route_count_kernel<<<nblocks, kThreads, 0, stream>>>(a);
  route_scan_kernel<<<1, kScanThreads, 0, stream>>>(a, nblocks);
  if (nblocks > 0) route_scatter_kernel<false><<<nblocks, kThreads, 0, stream>>>(a);
  return cudaGetLastError();
}


// ---------------------------------------------------------------------------
// Routing without any caller-provided scratch.
//
// Some callers are not allowed to allocate device memory at the point where they
// route tokens: code running between the nodes of a fixed serving loop whose
// memory pool was sized at start-up, or a plug-in that is handed input and output
// buffers by its host application and nothing else.  For them the per-block
// histograms live in this file-scope device array instead of a workspace argument.
// Every GPU that loads the library keeps these 256 KiB resident until the process
// exits.
constexpr int kStaticScratchInts = 64 * 1024;
static __device__ __align__(256) int g_route_scratch[kStaticScratchInts];

size_t route_static_scratch_ints() { return kStaticScratchInts; }

// `g_route_scratch` names a host-side handle in host code, not a device address:
// the address a kernel may use is looked up once per device, with that device current.
cudaError_t route_static_scratch_ptr(int** out) {
  static int* ptrs[64] = {nullptr};
  static std::mutex mu;   // host threads that make the first call on a device together
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_route_scratch);
    if (e != cudaSuccess) return e;
    ptrs[dev] = static_cast<int*>(p);
  }
  *out = ptrs[dev];
  return cudaSuccess;
}

cudaError_t launch_combine(const void* y, const int* slot_row, const float* topk_w, const void* y_shared, void* out,
                           int num_tokens, int topk, int hidden, cudaStream_t stream) {
  if (num_tokens <= 0) return cudaSuccess;
  combine_kernel<<<num_tokens, kThreads, 0, stream>>>(static_cast<const __half*>(y), slot_row, topk_w,
                                                      static_cast<const __half*>(y_shared), static_cast<__half*>(out),
                                                      topk, hidden);
  return cudaGetLastError();
}

}  // namespace mxb
