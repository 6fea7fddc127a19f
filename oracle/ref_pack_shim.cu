// TEST INFRASTRUCTURE ONLY - never linked into the product library.
//
// Thin extern "C" shim around the reference's own host-side pack/permute
// functions (mxmoe/kernels/src/include/quantize.cuh:299-475).  The reference
// header is included from where it lies (REF_INCLUDE_DIR is passed by the
// Makefile); nothing of it is copied here.  The resulting shared object is
// written to oracle/_ref/ and is used to pin oracle/pack.py (the numpy
// restatement of the packed layouts) against the reference's real code.
#include <stdexcept>
#include <cstdint>
#include <cstring>

#include "quantize.cuh"

extern "C" {

// quantize.cuh:424-475  pack_wxax<int8_t | s4>
int ref_pack_wxax(const int* act, const int* weight, int M, int N, int K, int qbits,
                  uint16_t* out_act, uint16_t* out_weight) {
  try {
    host_vector<int> a(act, act + (size_t)M * K);
    host_vector<int> w(weight, weight + (size_t)N * K);
    if (qbits == 8) {
      auto [pa, pw] = pack_wxax<int8_t>(a, w, M, N, K, qbits);
      std::memcpy(out_act, pa.data(), pa.size() * 2);
      std::memcpy(out_weight, pw.data(), pw.size() * 2);
    } else if (qbits == 4) {
      auto [pa, pw] = pack_wxax<nv_precision::s4>(a, w, M, N, K, qbits);
      std::memcpy(out_act, pa.data(), pa.size() * 2);
      std::memcpy(out_weight, pw.data(), pw.size() * 2);
    } else {
      return 2;
    }
  } catch (const std::exception&) {
    return 1;
  }
  return 0;
}

// quantize.cuh:318-421  permute_weight (PermuteMode::Row) then pack_weightonly
int ref_permute_pack_weightonly(const int* weight, int N, int K, int qbits, int sym, uint16_t* out) {
  try {
    host_vector<int> w(weight, weight + (size_t)N * K);
    auto perm   = permute_weight(w, N, K, qbits);
    auto packed = pack_weightonly(perm, N, K, qbits, sym);
    std::memcpy(out, packed.data(), packed.size() * 2);
  } catch (const std::exception&) {
    return 1;
  }
  return 0;
}

// quantize.cuh:299-315  permute_scale
int ref_permute_scale(const uint16_t* scale, size_t count, int N, int K, int gsize, int qbits, int sym,
                      uint16_t* out) {
  try {
    host_vector<half> s(count);
    std::memcpy(s.data(), scale, count * 2);
    auto r = permute_scale(s, N, K, gsize, qbits, sym != 0);
    std::memcpy(out, r.data(), r.size() * 2);
  } catch (const std::exception&) {
    return 1;
  }
  return 0;
}

}  // extern "C"
