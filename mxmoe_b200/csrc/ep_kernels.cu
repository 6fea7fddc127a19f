// Expert-parallel exchange without the host: the plan of a step (who sends how many rows where) is computed
// on the device from the all-gathered routing counts, and the quantised rows are written straight into the
// receive stores of the GPUs that own their experts (plain stores to peer memory over NVLink; no TMA and no
// multicast is involved).  The reference has no distributed code; this is the multi-GPU form of the path.
#include "ep_kernels.h"

namespace mxb {

namespace {

constexpr int kPlanThreads = 256;

__device__ __forceinline__ int owner_of(const int* range_lo, int world, int e) {
  int d = 0;
  while (d + 1 < world && e >= range_lo[d + 1]) ++d;
  return d;
}

// One block.  counts_all[s][e]: rows rank s routes to expert e; experts are numbered so that rank r owns
// [range_lo[r], range_lo[r+1]).
constexpr int kPlanSmemInts = 8192;   // counts of up to this many (rank, expert) pairs are staged in shared memory

__global__ void __launch_bounds__(kPlanThreads) ep_plan_kernel(EpPlanArgs a) {
  __shared__ int s_counts[kPlanSmemInts];
  const int tid = threadIdx.x;
  const int E = a.num_experts, G = a.world, me = a.rank;
  // every table below is a sum over a few hundred of the G x E counts: read them from HBM once
  const int* counts = a.counts_all;
  if (G * E <= kPlanSmemInts) {
    for (int i = tid; i < G * E; i += kPlanThreads) s_counts[i] = a.counts_all[i];
    __syncthreads();
    counts = s_counts;
  }
  const int lo = a.range_lo[me], hi = a.range_lo[me + 1];
  const int el = hi - lo;
  // where my rows for expert e start in the receive store of e's owner: behind the rows of the lower ranks
  // for the owner's experts, and behind my rows for the owner's earlier experts
  for (int e = tid; e < E; e += kPlanThreads) {
    const int d   = owner_of(a.range_lo, G, e);
    const int dlo = a.range_lo[d], dhi = a.range_lo[d + 1];
    int off = 0;
    if (a.layout == 0) {
      for (int s = 0; s < me; ++s)
        for (int j = dlo; j < dhi; ++j) off += counts[s * E + j];
      for (int j = dlo; j < e; ++j) off += counts[me * E + j];
    } else {
      // (expert, source rank): behind all rows of the owner's earlier experts and the lower ranks' rows for e
      for (int s = 0; s < G; ++s)
        for (int j = dlo; j < e; ++j) off += counts[s * E + j];
      for (int s = 0; s < me; ++s) off += counts[s * E + e];
    }
    a.dst_row0[e]  = off;
    a.exp_owner[e] = d;
  }
  // my receive store: segments (source rank s, local expert j), s-major
  const int nseg = G * el;
  for (int i = tid; i < nseg; i += kPlanThreads) {
    const int s = i / el, j = i - s * el;
    int row0 = 0;
    if (a.layout == 0) {
      for (int s2 = 0; s2 < s; ++s2)
        for (int j2 = lo; j2 < hi; ++j2) row0 += counts[s2 * E + j2];
      for (int j2 = lo; j2 < lo + j; ++j2) row0 += counts[s * E + j2];
    } else {
      for (int s2 = 0; s2 < G; ++s2)
        for (int j2 = lo; j2 < lo + j; ++j2) row0 += counts[s2 * E + j2];
      for (int s2 = 0; s2 < s; ++s2) row0 += counts[s2 * E + lo + j];
    }
    int src0 = 0;   // the same rows in rank s's expert-sorted order
    for (int e2 = 0; e2 < lo + j; ++e2) src0 += counts[s * E + e2];
    int m = counts[s * E + lo + j];
    // never let a segment reach past the store: the rows beyond the capacity are dropped and reported
    if (row0 >= a.recv_capacity) m = 0;
    else if (row0 + m > a.recv_capacity) m = a.recv_capacity - row0;
    a.seg_m[i]        = m;
    a.seg_row0[i]     = row0;
    a.seg_src_row0[i] = src0;
  }
  if (a.exp_m) {
    for (int j = tid; j < el; j += kPlanThreads) {
      int row0 = 0, m = 0;
      for (int s = 0; s < G; ++s) {
        for (int j2 = lo; j2 < lo + j; ++j2) row0 += counts[s * E + j2];
        m += counts[s * E + lo + j];
      }
      if (row0 >= a.recv_capacity) m = 0;
      else if (row0 + m > a.recv_capacity) m = a.recv_capacity - row0;
      a.exp_m[j]    = m;
      a.exp_row0[j] = row0;
    }
  }
  if (tid == 0) {
    int total = 0;
    for (int s = 0; s < G; ++s)
      for (int j = lo; j < hi; ++j) total += counts[s * E + j];
    a.total_recv[0] = total < a.recv_capacity ? total : a.recv_capacity;
    if (total > a.recv_capacity) atomicExch(&a.total_recv[1], total);   // overflow: rows wanted
  }
}

// One block.  Epoch e of the barrier: publish the payload into every peer, fence, write e into flag `rank` of every
// peer, then wait until all of this rank's flags show e.  The wait is bounded: when it runs out the error word of
// the local sync block is set and the kernel returns (the host reads the word; later kernels run on whatever
// arrived).  The ranks run on different GPUs, one process each, so the waiting kernels never share a GPU.
constexpr int kSyncFlags = 64, kSyncErr = 64, kSyncEpoch = 65, kSyncPayload0 = 128;

__device__ __forceinline__ uint64_t ep_globaltimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__global__ void __launch_bounds__(256) ep_sync_kernel(EpSyncArgs a) {
  const int tid = threadIdx.x;
  __shared__ int s_epoch;
  if (tid == 0) s_epoch = a.local_sync[kSyncEpoch] + 1;
  __syncthreads();
  const int epoch = s_epoch;
  if (a.payload && a.payload_len > 0) {
    for (int i = tid; i < a.world * a.payload_len; i += blockDim.x) {
      const int d = i / a.payload_len, j = i - d * a.payload_len;
      int* dst = reinterpret_cast<int*>(a.peer_sync[d]) + kSyncPayload0 + a.rank * a.payload_cap + j;
      *dst = a.payload[j];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid < a.world) {
    volatile int* flag = reinterpret_cast<int*>(a.peer_sync[tid]) + a.rank;
    *flag = epoch;
  }
  if (tid < a.world) {
    volatile int* mine = a.local_sync + tid;
    const uint64_t limit = (a.timeout_ms > 0 ? (uint64_t)a.timeout_ms : 2000ull) * 1000000ull;
    const uint64_t t0 = ep_globaltimer();
    unsigned spins = 0;
    // signed distance: a peer that is already one barrier ahead has written a larger epoch
    while (*mine - epoch < 0) {
      if ((++spins & 255u) == 0 && ep_globaltimer() - t0 > limit) {
        atomicExch(a.local_sync + kSyncErr, 1 + tid);      // 1 + the rank that did not arrive
        break;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid == 0) a.local_sync[kSyncEpoch] = epoch;
}

// block = segment: expert of every received row (the second quantiser picks its format by expert)
__global__ void ep_fill_row_expert_kernel(EpPlanArgs a) {
  const int lo = a.range_lo[a.rank], el = a.range_lo[a.rank + 1] - lo;
  const int i = blockIdx.x;
  const int e = lo + (i % el);
  const int row0 = a.seg_row0[i], m = a.seg_m[i];
  for (int r = threadIdx.x; r < m; r += blockDim.x) a.recv_row_expert[row0 + r] = e;
  if (a.row_dst) {
    const int64_t base = (int64_t)a.peer_ret[i / el] + (int64_t)a.seg_src_row0[i] * a.ret_row_bytes;
    for (int r = threadIdx.x; r < m; r += blockDim.x) a.row_dst[row0 + r] = base + (int64_t)r * a.ret_row_bytes;
  }
}

// One warp per expert-sorted row of this rank: packed row + its scale -> record in the owner's receive store.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(EpDispatchArgs d, TokenQuantArgs t) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  if (row >= d.rows) return;
  const int e       = d.row_expert[row];
  const int idx     = row - d.exp_row_start[e];
  const int dst_row = d.dst_row0[e] + idx;
  if (dst_row >= d.recv_capacity) return;   // reported by the owner's plan kernel
  const int tag     = d.exp_qtag[e];
  const int64_t tok = d.row_token[row];
  const int pack    = tag == 0 ? 1 : (tag == 2 ? 4 : 2);
  const __half* src = tag == 0 ? (t.f16 ? t.f16 : t.in) : (tag == 1 ? t.q8 : (tag == 2 ? t.q4 : t.q4x));
  const uint4* s    = reinterpret_cast<const uint4*>(src + tok * (d.k / pack));
  unsigned char* rec = reinterpret_cast<unsigned char*>(d.peer_base[d.exp_owner[e]]) + (int64_t)dst_row * d.rec_bytes;
  uint4* dst        = reinterpret_cast<uint4*>(rec);
  const int n16     = (d.k / pack) >> 3;
  // all loads of the record are issued before the first (peer) store
  for (int c0 = 0; c0 < n16; c0 += 32 * 8) {
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (c0 + j * 32 + lane < n16) v[j] = __ldg(s + c0 + j * 32 + lane);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (c0 + j * 32 + lane < n16) dst[c0 + j * 32 + lane] = v[j];
  }
  if (tag != 0 && lane == 0) *reinterpret_cast<__half*>(rec + d.scale_off_bytes) = (tag == 1 ? t.s8 : t.s4)[tok];
}

}  // namespace

cudaError_t launch_ep_sync(const EpSyncArgs& a, cudaStream_t stream) {
  ep_sync_kernel<<<1, 256, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_ep_plan(const EpPlanArgs& a, cudaStream_t stream) {
  ep_plan_kernel<<<1, kPlanThreads, 0, stream>>>(a);
  const int el = a.experts_local;
  if (a.world * el > 0) ep_fill_row_expert_kernel<<<a.world * el, 256, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_ep_dispatch(const EpDispatchArgs& d, const TokenQuantArgs& t, cudaStream_t stream) {
  if (d.rows <= 0) return cudaSuccess;
  ep_dispatch_kernel<<<(d.rows + 7) / 8, 256, 0, stream>>>(d, t);
  return cudaGetLastError();
}

}  // namespace mxb
