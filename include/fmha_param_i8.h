// Boundary types of the INT8 attention forward path.  Layout-identical (field order, types,
// defaults) to the reference project's inc/fmha_param_i8.h:3-17, so code written against the
// reference compiles and links unchanged.  Both structs are passed BY VALUE.
#ifndef FMHA_PARAM_I8_H_
#define FMHA_PARAM_I8_H_

// Problem shape.  Tensors q,k,v,o are int8 [batch_num, head_num, seq_len, head_dim], row-major
// and contiguous; the padding mask is int8 [batch_num, seq_len].  Note the member order:
// seq_len comes before head_num.  sizeof == 16.
struct AttnDataDescriptor {
  int batch_num = 1;
  int seq_len   = 64;
  int head_num  = 4;
  int head_dim  = 64;
};

// Per-tensor symmetric quantisation ranges: real value = int8 * amax / 127.
// s_max is carried for source compatibility and is not read.  sizeof == 20.
struct FMHAParamI8 {
  float q_amax = 0.0f;
  float k_amax = 0.0f;
  float v_amax = 0.0f;
  float o_amax = 1.0f;
  float s_max  = 1.0f;
};

#endif  // FMHA_PARAM_I8_H_
