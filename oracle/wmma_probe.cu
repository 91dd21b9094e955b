// TEST INFRASTRUCTURE ONLY.  Dumps the register layout that nvcuda::wmma gives, on the GPU it runs on, to the two
// fragment kinds the reference kernel indexes by hand (inc/fmha_i8.cuh:183-196 accumulator, :239-253 matrix_a):
// a 16x16 matrix whose element (r, c) holds 16 r + c is loaded into an int32 accumulator fragment and into an int8
// row-major matrix_a fragment, and every lane writes out its x[0..7].  One warp, valid inputs, nothing else.
// The WMMA API leaves these layouts unspecified; the reference's arithmetic is only right where they are the
// mma.m16n8k16 ones (accumulator x[4 tc_xi + 2 tc_yi + e] = (lane/4 + 8 tc_yi, 8 tc_xi + 2 (lane%4) + e),
// matrix_a x[4 tc_yi + t] = (lane/4 + 8 tc_yi, 4 (lane%4) + t)), which is what tests compare this dump with.
#include <cuda_runtime_api.h>
#include <mma.h>
#include <cstdint>

namespace {
__global__ void wmma_layout_probe_kernel(int* acc_out, int* a_out) {
  using namespace nvcuda;
  __shared__ int acc_src[256];
  __shared__ __align__(32) int8_t a_src[256];
  for (int i = threadIdx.x; i < 256; i += 32) {
    acc_src[i] = i;                               // element (r, c) = 16 r + c
    a_src[i] = static_cast<int8_t>(i - 128);      // element (r, c) = 16 r + c - 128 (fits int8)
  }
  __syncwarp();
  wmma::fragment<wmma::accumulator, 16, 16, 16, int> acc;
  wmma::fragment<wmma::matrix_a, 16, 16, 16, int8_t, wmma::row_major> a;
  wmma::load_matrix_sync(acc, acc_src, 16, wmma::mem_row_major);
  wmma::load_matrix_sync(a, a_src, 16);
  for (int i = 0; i < 8; ++i) {
    acc_out[threadIdx.x * 8 + i] = (i < acc.num_elements) ? acc.x[i] : -1;
    a_out[threadIdx.x * 8 + i] = (i < a.num_elements) ? static_cast<int>(a.x[i]) + 128 : -1;
  }
}
}  // namespace

// acc_out, a_out: device arrays of 32 x 8 ints; entry [lane][i] = 16 r + c of the matrix element that x[i] of that lane holds.
extern "C" int wmma_layout_probe(int* acc_out, int* a_out) {
  wmma_layout_probe_kernel<<<1, 32>>>(acc_out, a_out);
  return static_cast<int>(cudaGetLastError());
}
