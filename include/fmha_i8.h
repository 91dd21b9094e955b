// Drop-in replacement for the reference project's host entry point (inc/fmha_i8.h:5-17, defined
// at src/fmha_i8.cu:157-173): same namespace, name, parameter list and void return, so a caller
// such as the reference's test_fmha_i8.cpp:204,219 links against this library unchanged.
//
// Behaviour kept: work is enqueued on `stream` and the call returns without synchronising; the
// caller owns all buffers; nothing is allocated.  Differences, all towards stricter behaviour:
//   * any head_dim in {64,128} with any seq_len that is a multiple of 64 (up to 32768) is served by
//     one runtime-shaped kernel (the reference silently launches nothing outside its table,
//     src/fmha_i8.cu:39-155);
//   * use_tcu == false is an error (the reference launches an empty kernel, inc/fmha_i8.cuh:337-342);
//   * a failed call stores a status readable through fmha_i8_sm100_last_status() and prints one
//     line to stderr; it never throws or aborts.
#ifndef FMHA_I8_H_
#define FMHA_I8_H_

#include <cuda_runtime_api.h>
#include "fmha_param_i8.h"

namespace gpuImpl {

// q, k, v : const int8 [B,H,S,D] device pointers (16-byte aligned)
// padding_mask : const int8 [B,S] device pointer (4-byte aligned); non-zero byte = key masked out
// o : int8 [B,H,S,D] device pointer (16-byte aligned)
void FMHAInferI8(cudaStream_t stream,
                 FMHAParamI8 fmha_param,
                 AttnDataDescriptor attn_desc,
                 const void* q,
                 const void* k,
                 const void* v,
                 const void* padding_mask,
                 void* o,
                 const bool use_tcu);

}  // namespace gpuImpl

#endif  // FMHA_I8_H_
