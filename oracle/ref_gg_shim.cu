// TEST INFRASTRUCTURE ONLY - never linked into the product library.
//
// Device oracle: the reference's OWN fused GroupGEMM kernel (mma.sync / cp.async code written for
// sm_80/sm_89), built for sm_100a.  The kernel and its host launcher are the strings the reference's
// generator returns (mxmoe/kernels/compose_kernel.py:503-530, launcher template
// mxmoe/kernels/kernel_sketch.py:82-145), written by oracle/gen_ref_gg.py to
// oracle/_ref/ref_gg_generated.cuh; the headers they use (cta_gemm.cuh, mm_tile.cuh, quantize.cuh,
// tile_scheduler.cuh, ...) are included from the reference checkout where it lies.  Nothing of the
// reference is copied here.  registry.cuh is left out (it needs the un-vendored fmt library and only
// registers the kernel under a name).
//
// extern "C" ref_gg_run: takes HOST arrays of device pointers, builds the device-side argument arrays
// the reference launcher expects (registry.cuh:28-39 FuncType), calls the launcher and synchronises.
// The reference launcher terminates the process on a CUDA error (helper.h:186-198): callers run this
// library in a child process.
#include <stdexcept>
#include <cstdint>
#include <cstdio>
#include <vector>

#include "cta_gemm.cuh"
#include "tile_scheduler.cuh"

namespace mxmoe {
using namespace tiled_gemm;
using MatricesInfo = RCR_FP16FP16FP16;

#include "ref_gg_generated.cuh"

}  // namespace mxmoe

namespace {
template <typename T>
T* to_device(const std::vector<T>& h) {
  T* d = nullptr;
  if (cudaMalloc(&d, h.size() * sizeof(T)) != cudaSuccess) return nullptr;
  if (cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess) return nullptr;
  return d;
}
}  // namespace

extern "C" {

// sizes: [count][3] = (M, N, K); qparams: [count][4] = (a_bits, w_bits, gsize, sym)
// A / B / scale_a / scale_b / C: host arrays of `count` device addresses (0 where the scheme has none).
// Returns 0, or a negative number for a failed allocation / a CUDA error code after the launch.
int ref_gg_run(const uint64_t* A, const uint64_t* B, const uint64_t* scale_a, const uint64_t* scale_b,
               const uint64_t* C, const int32_t* sizes, const int32_t* qparams, int count) {
  using mxmoe::QParams;
  std::vector<half*> hA(count), hB(count), hSa(count), hSb(count), hC(count);
  std::vector<dim3> hsz(count);
  std::vector<QParams> hq(count);
  for (int i = 0; i < count; ++i) {
    hA[i]  = reinterpret_cast<half*>(A[i]);
    hB[i]  = reinterpret_cast<half*>(B[i]);
    hSa[i] = reinterpret_cast<half*>(scale_a[i]);
    hSb[i] = reinterpret_cast<half*>(scale_b[i]);
    hC[i]  = reinterpret_cast<half*>(C[i]);
    hsz[i] = dim3(sizes[3 * i], sizes[3 * i + 1], sizes[3 * i + 2]);
    QParams q;
    q.qbits = make_int2(qparams[4 * i], qparams[4 * i + 1]);
    q.gsize = qparams[4 * i + 2];
    q.sym   = qparams[4 * i + 3] != 0;
    hq[i]   = q;
  }
  half** dA   = to_device(hA);
  half** dB   = to_device(hB);
  half** dSa  = to_device(hSa);
  half** dSb  = to_device(hSb);
  half** dC   = to_device(hC);
  dim3* dsz   = to_device(hsz);
  QParams* dq = to_device(hq);
  if (!dA || !dB || !dSa || !dSb || !dC || !dsz || !dq) return -1;
  try {
    mxmoe::groupgemm_hz_fused_oracle(dA, dB, dSa, dSb, dC, dC, nullptr, nullptr, nullptr, nullptr, dsz, hsz.data(), dq,
                                     hq.data(), count);
  } catch (const std::exception& e) {
    fprintf(stderr, "ref_gg_run: %s\n", e.what());
    return -2;
  }
  cudaError_t e = cudaDeviceSynchronize();
  cudaFree(dA); cudaFree(dB); cudaFree(dSa); cudaFree(dSb); cudaFree(dC); cudaFree(dsz); cudaFree(dq);
  return e == cudaSuccess ? 0 : -(1000 + (int)e);
}

// the host-side operand packers of the same headers, so that the child process needs one library only
// quantize.cuh:424-475
int ref_gg_pack_wxax(const int* act, const int* weight, int M, int N, int K, int qbits, uint16_t* out_act,
                     uint16_t* out_weight) {
  try {
    host_vector<int> a(act, act + (size_t)M * K);
    host_vector<int> w(weight, weight + (size_t)N * K);
    if (qbits == 8) {
      auto [pa, pw] = pack_wxax<int8_t>(a, w, M, N, K, qbits);
      memcpy(out_act, pa.data(), pa.size() * 2);
      memcpy(out_weight, pw.data(), pw.size() * 2);
    } else if (qbits == 4) {
      auto [pa, pw] = pack_wxax<nv_precision::s4>(a, w, M, N, K, qbits);
      memcpy(out_act, pa.data(), pa.size() * 2);
      memcpy(out_weight, pw.data(), pw.size() * 2);
    } else {
      return 2;
    }
  } catch (const std::exception&) {
    return 1;
  }
  return 0;
}

// quantize.cuh:318-421
int ref_gg_permute_pack_weightonly(const int* weight, int N, int K, int qbits, int sym, uint16_t* out) {
  try {
    host_vector<int> w(weight, weight + (size_t)N * K);
    auto perm   = permute_weight(w, N, K, qbits);
    auto packed = pack_weightonly(perm, N, K, qbits, sym);
    memcpy(out, packed.data(), packed.size() * 2);
  } catch (const std::exception&) {
    return 1;
  }
  return 0;
}

}  // extern "C"
