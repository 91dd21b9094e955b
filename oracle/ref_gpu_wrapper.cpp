// extern "C" door onto the reference project's own GPU entry point, gpuImpl::FMHAInferI8
// (inc/fmha_i8.h:5-17, src/fmha_i8.cu:157-173), built unchanged for sm_100a from the reference
// checkout by oracle/Makefile into oracle/_ref/libref_gpu.so.  TEST INFRASTRUCTURE ONLY: it pins
// the quantised CPU oracle against real reference output and gives the "reference WMMA kernel on
// the same box" timing.  Callers must keep to shapes the reference instantiates with a matching
// thread count: head_dim in {64,128} and seq_len in {128,256,384,512,1024,2048,4096}
// (its 64-row-tile variants are launched with twice the threads their tiles are sized for,
// src/fmha_i8.cu:42-59, and index out of bounds, so they are never run).
#include <cuda_runtime_api.h>
#include "fmha_i8.h"

extern "C" int ref_gpu_shape_ok(int seq_len, int head_dim) {
  if (head_dim != 64 && head_dim != 128) return 0;
  const int ok[] = {128, 256, 384, 512, 1024, 2048, 4096};
  for (int s : ok) if (s == seq_len) return 1;
  return 0;
}

extern "C" int ref_gpu_fmha(void* stream, const float* amax5, const int* desc4,
                            const void* q, const void* k, const void* v, const void* mask, void* o) {
  AttnDataDescriptor d;
  d.batch_num = desc4[0]; d.seq_len = desc4[1]; d.head_num = desc4[2]; d.head_dim = desc4[3];
  if (!ref_gpu_shape_ok(d.seq_len, d.head_dim)) return -1;
  FMHAParamI8 p;
  p.q_amax = amax5[0]; p.k_amax = amax5[1]; p.v_amax = amax5[2]; p.o_amax = amax5[3]; p.s_max = amax5[4];
  gpuImpl::FMHAInferI8(static_cast<cudaStream_t>(stream), p, d, q, k, v, mask, o, true);
  return static_cast<int>(cudaGetLastError());
}
