// Online Hadamard rotation for row lengths n = K * m with a K x K Hadamard factor (had_kernels.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace mxb {

// out[r, a*m + t] = scale * sum_a' hadK[a, a'] * z[r, a'*m + t]; z = in, or (fwht8, m == 8) the natural-order
// Walsh-Hadamard transform of every group of 8 contiguous elements of in.  K <= 176, m a multiple of 8.
// in == out is allowed (a block reads its tile completely before it writes it).
cudaError_t launch_had_kron(const __half* in, __half* out, const __half* hadK, int rows, int K, int m, float scale,
                            bool fwht8, cudaStream_t stream);

}  // namespace mxb
