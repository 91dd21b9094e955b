// Thin extern "C" wrapper around the reference project's own CPU headers, compiled from where
// they lie (the include path points into the reference checkout; nothing is copied).  The build
// recipe is oracle/Makefile and the result goes to oracle/_ref/.  TEST INFRASTRUCTURE ONLY: it
// validates the restatement in oracle.cpp, generates tests/golden/, and is the timed CPU baseline.
//
// Each function performs the calls of test_fmha_i8.cpp with the template arguments and flags
// used there (test_fmha_i8.cpp:142-161 for the fp32 path, :95-110 for quantisation).
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>
#include <unistd.h>

#include "cpuGEMM.hpp"
#include "cpuSoftmax.hpp"
#include "utils.hpp"

extern "C" {

float ref_abs_max(float* x, int len) { return abs_max(x, len); }

void ref_quantize(const float* x, int64_t n, float amax, int8_t* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = static_cast<int8_t>(float_quant2_int8(x[i], amax));
}

// Exact int32 Q.K^T through the reference GEMM template (same flags as the fp32 call).
void ref_qk_int32(int8_t* q, int8_t* k, int BH, int S, int D, int32_t* s) {
  cpuGEMM<int32_t, int32_t, int8_t, int32_t>(q, k, s, S, S, D, S * D, S * D, S * S, BH, 1, 0,
                                             GEMM_OP_T, GEMM_OP_N, nullptr, false);
}

// fp32 golden for heads [bh0, bh0+nbh) of a [B,H,S,D] problem; s_buf/p_buf hold nbh*S*S floats.
// mask_i32 is the [B,S] int mask of the reference (1 = masked key).
static void fp32_slice(float* q, float* k, float* v, int* mask_i32, int H, int S, int D,
                       int bh0, int nbh, float* s_buf, float* p_buf, float* o) {
  for (int bh = bh0; bh < bh0 + nbh; ++bh) {
    const int64_t off = static_cast<int64_t>(bh) * S * D;
    float* sb = s_buf + static_cast<int64_t>(bh - bh0) * S * S;
    float* pb = p_buf + static_cast<int64_t>(bh - bh0) * S * S;
    std::memset(sb, 0, sizeof(float) * S * S);
    std::memset(o + off, 0, sizeof(float) * S * D);
    cpuGEMM<float, float, float, float>(q + off, k + off, sb, S, S, D, S * D, S * D, S * S, 1,
                                        1.f, 0.f, GEMM_OP_T, GEMM_OP_N, nullptr, false);
    // one (batch, head) slice: batch_size = 1, head_num = 1, mask row of this head's batch
    cpuAttentionMaskedSoftmax<float, float>(sb, pb, mask_i32 + static_cast<int64_t>(bh / H) * S,
                                            1, S, S, 1, D);
    cpuGEMM<float, float, float, float>(pb, v + off, o + off, S, D, S, S * S, S * D, S * D, 1,
                                        1.f, 0.f, GEMM_OP_T, GEMM_OP_T, nullptr, false);
  }
}

// Whole problem in one set of batched calls, exactly as the reference test does it.
void ref_fp32_attention_batched(float* q, float* k, float* v, int* mask_i32, int B, int H, int S,
                                int D, float* s_buf, float* p_buf, float* o, float* s_max) {
  const int64_t len_sp = static_cast<int64_t>(B) * H * S * S;
  std::memset(s_buf, 0, sizeof(float) * len_sp);
  std::memset(p_buf, 0, sizeof(float) * len_sp);
  std::memset(o, 0, sizeof(float) * static_cast<int64_t>(B) * H * S * D);
  cpuGEMM<float, float, float, float>(q, k, s_buf, S, S, D, S * D, S * D, S * S, B * H, 1.f, 0.f,
                                      GEMM_OP_T, GEMM_OP_N, nullptr, false);
  cpuAttentionMaskedSoftmax<float, float>(s_buf, p_buf, mask_i32, B, S, S, H, D);
  if (s_max) *s_max = abs_max(p_buf, static_cast<int>(len_sp));
  cpuGEMM<float, float, float, float>(p_buf, v, o, S, D, S, S * S, S * D, S * D, B * H, 1.f, 0.f,
                                      GEMM_OP_T, GEMM_OP_T, nullptr, false);
}

// The same three calls with a different number of query rows (Sq) and keys (Sk): the reference templates
// take both lengths (inc/cpuGEMM.hpp:10-13 M,N,K; inc/cpuSoftmax.hpp:12 seq_len_q, seq_len_k) although
// its test only ever passes Sq == Sk.  q,o: [B,H,Sq,D]; k,v: [B,H,Sk,D]; mask [B,Sk]; s_buf/p_buf hold
// B*H*Sq*Sk floats.
void ref_fp32_attention_cross(float* q, float* k, float* v, int* mask_i32, int B, int H, int Sq, int Sk,
                              int D, float* s_buf, float* p_buf, float* o) {
  const int64_t len_sp = static_cast<int64_t>(B) * H * Sq * Sk;
  std::memset(s_buf, 0, sizeof(float) * len_sp);
  std::memset(p_buf, 0, sizeof(float) * len_sp);
  std::memset(o, 0, sizeof(float) * static_cast<int64_t>(B) * H * Sq * D);
  cpuGEMM<float, float, float, float>(q, k, s_buf, Sq, Sk, D, Sq * D, Sk * D, Sq * Sk, B * H, 1.f, 0.f,
                                      GEMM_OP_T, GEMM_OP_N, nullptr, false);
  cpuAttentionMaskedSoftmax<float, float>(s_buf, p_buf, mask_i32, B, Sq, Sk, H, D);
  cpuGEMM<float, float, float, float>(p_buf, v, o, Sq, D, Sk, Sq * Sk, Sk * D, Sq * D, B * H, 1.f, 0.f,
                                      GEMM_OP_T, GEMM_OP_T, nullptr, false);
}

// Exact int32 Q.K^T for Sq query rows against Sk keys.
void ref_qk_int32_cross(int8_t* q, int8_t* k, int BH, int Sq, int Sk, int D, int32_t* s) {
  cpuGEMM<int32_t, int32_t, int8_t, int32_t>(q, k, s, Sq, Sk, D, Sq * D, Sk * D, Sq * Sk, BH, 1, 0,
                                             GEMM_OP_T, GEMM_OP_N, nullptr, false);
}

// Same arithmetic, one unchanged single-slice call chain per (b,h), slices spread over threads.
// This is the timed CPU baseline; nbh may be a subset of B*H (heads [bh0, bh0+nbh)).
void ref_fp32_attention_threaded(float* q, float* k, float* v, int* mask_i32, int H, int S, int D,
                                 int bh0, int nbh, float* o, int n_threads) {
  if (n_threads < 1) n_threads = 1;
  if (n_threads > nbh) n_threads = nbh;
  std::vector<std::thread> pool;
  for (int t = 0; t < n_threads; ++t)
    pool.emplace_back([=]() {
      std::vector<float> s(static_cast<size_t>(S) * S), p(static_cast<size_t>(S) * S);
      for (int bh = bh0 + t; bh < bh0 + nbh; bh += n_threads)
        fp32_slice(q, k, v, mask_i32, H, S, D, bh, 1, s.data(), p.data(), o);
    });
  for (auto& th : pool) th.join();
}

// The reference's acceptance metric (inc/utils.hpp:59-89).  The function only prints its result,
// so stdout is captured around the call and the percentage parsed back.  Returns -1 on failure.
double ref_mean_rel_deviation(const int8_t* res, const float* ref, int len, float o_amax) {
  char path[] = "/tmp/ref_dev_XXXXXX";
  int fd = mkstemp(path);
  if (fd < 0) return -1.0;
  fflush(stdout);
  int saved = dup(1);
  dup2(fd, 1);
  compareResultsWithGoldenI8(res, ref, len, o_amax);
  fflush(stdout);
  dup2(saved, 1);
  close(saved);
  std::string text;
  lseek(fd, 0, SEEK_SET);
  char buf[512];
  ssize_t n;
  while ((n = read(fd, buf, sizeof buf)) > 0) text.append(buf, buf + n);
  close(fd);
  unlink(path);
  size_t pos = text.find("deviation:");
  if (pos == std::string::npos) return -1.0;
  return atof(text.c_str() + pos + 10);
}

}  // extern "C"
