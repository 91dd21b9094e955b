// CPU oracle for the INT8 attention forward path.  TEST INFRASTRUCTURE ONLY.
//
// This file restates, in plain C++, the arithmetic of the reference project
// (jundaf2/INT8-Flash-Attention-FMHA-Quantization) for the one path this
// repository accelerates.  It is never linked into, imported by or called from
// the product library; only the test-suite, the smoke check and the
// cpu-baseline leg of the benchmark may load it, and only as the checker.
//
// Three tiers are provided (reference citations are file:line in that project):
//   A  fp32 golden           cpuGEMM -> cpuAttentionMaskedSoftmax -> cpuGEMM as
//                            wired up in test_fmha_i8.cpp:142-159
//                            (inc/cpuGEMM.hpp:8-31, inc/cpuSoftmax.hpp:11-51)
//   B  exact int32 Q.K^T     the same GEMM template instantiated on int8 -> int32
//   C  quantised tile-128    the arithmetic of the device kernel
//                            inc/fmha_i8.cuh:71-72 (scales), :183-253 (tile
//                            softmax, P -> int8), :298-315 (online merge),
//                            :318-332 (epilogue), with the mask semantics of
//                            inc/cpuSoftmax.hpp:24 (masked key => -inf / p = 0)
// plus the input quantiser and acceptance metric of inc/utils.hpp:23-39,59-89.
//
// Parity pin: tiers A and B and the quantiser are checked bit-for-bit against
// outputs of the reference's own headers compiled here (oracle/_ref, see
// oracle/Makefile) and stored under tests/golden/.  Tier C has no CPU
// counterpart in the reference (the algorithm exists there only as a CUDA
// kernel); it is pinned through the reference's own acceptance criterion
// against tier A and, on a GPU box, against the reference kernel rebuilt
// unchanged for sm_100a (oracle/_ref/libref_gpu.so).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>
#include <algorithm>

namespace {

// The reference evaluates 1/sqrt(head_dim) through a constexpr Newton-Raphson
// square root (inc/fmha_i8.cuh:13-34): iterate in double, carry the value as
// float, stop when two successive float iterates are equal.
float newton_sqrt(float x) {
  float curr = x, prev = 0.f;
  while (curr != prev) {
    float next = static_cast<float>(0.5 * (static_cast<double>(curr) + static_cast<double>(x / curr)));
    prev = curr;
    curr = next;
  }
  return curr;
}

template <class F>
void parallel_for(int n, int n_threads, F f) {
  if (n_threads <= 1 || n <= 1) {
    for (int i = 0; i < n; ++i) f(i);
    return;
  }
  n_threads = std::min(n_threads, n);
  std::vector<std::thread> pool;
  for (int t = 0; t < n_threads; ++t)
    pool.emplace_back([=]() {
      for (int i = t; i < n; i += n_threads) f(i);
    });
  for (auto& th : pool) th.join();
}

inline int32_t clamp_round_even_i32(float x, float lo, float hi) {
  x = std::fmax(std::fmin(x, hi), lo);
  return static_cast<int32_t>(std::nearbyintf(x));  // default mode: round-half-even, like __float2int_rn
}
inline int8_t clamp_round_even(float x, float lo, float hi) { return static_cast<int8_t>(clamp_round_even_i32(x, lo, hi)); }

}  // namespace

extern "C" {

// inc/utils.hpp:31-39
float oracle_abs_max(const float* x, int64_t n) {
  float m = 0.f;
  for (int64_t i = 0; i < n; ++i) {
    float a = std::fabs(x[i]);
    if (a > m) m = a;
  }
  return m;
}

// inc/utils.hpp:23-29 : scale = 127/amax, floor(x*scale + 0.5), clamp to +-127
void oracle_quantize(const float* x, int64_t n, float amax, int8_t* out) {
  float scale = 127.0f / amax;
  for (int64_t i = 0; i < n; ++i) {
    float f = x[i] * scale;
    int32_t v = static_cast<int32_t>(floorf(static_cast<float>(f + 0.5)));  // 0.5 is a double literal there
    v = v < -127 ? -127 : (v > 127 ? 127 : v);
    out[i] = static_cast<int8_t>(v);
  }
}

// inc/utils.hpp:59-89 : mean over elements of |res*o_amax/127 - ref| / (|ref| + 0.01), in percent.
double oracle_mean_rel_deviation(const int8_t* res, const float* ref, int64_t n, float o_amax) {
  float acc = 0.f;  // the reference accumulates in float
  for (int64_t i = 0; i < n; ++i) {
    float r = static_cast<float>(res[i]) / 127.0f * o_amax;
    float d = std::fabs(r - ref[i]);
    acc += d / (std::fabs(ref[i]) + 0.01);
  }
  return static_cast<double>(acc) * 100.0 / static_cast<double>(n);
}

// Tier B.  S[bh, i, j] = sum_d q[bh,i,d] * k[bh,j,d], int32, row-major (test_fmha_i8.cpp:142-147
// with the template instantiated as cpuGEMM<int32_t,int32_t,int8_t,int32_t>).
void oracle_qk_int32(const int8_t* q, const int8_t* k, int BH, int S, int D, int32_t* s, int n_threads) {
  parallel_for(BH, n_threads, [=](int bh) {
    const int8_t* qb = q + static_cast<int64_t>(bh) * S * D;
    const int8_t* kb = k + static_cast<int64_t>(bh) * S * D;
    int32_t* sb = s + static_cast<int64_t>(bh) * S * S;
    for (int i = 0; i < S; ++i)
      for (int j = 0; j < S; ++j) {
        int32_t acc = 0;
        for (int d = 0; d < D; ++d) acc += static_cast<int32_t>(qb[i * D + d]) * static_cast<int32_t>(kb[j * D + d]);
        sb[static_cast<int64_t>(i) * S + j] = acc;
      }
  });
}

// Tier A.  fp32 attention on unquantised inputs with exactly the operation order of the
// reference CPU path: S = sum_d q*k (float accumulate, d ascending), then per row
// max(s*scale), sum of exp(s*scale - max), p = exp(..)/sum, O = sum_j p*v (j ascending).
// q and o have Sq rows per head, k and v have S (the reference CPU templates take both lengths,
// inc/cpuSoftmax.hpp:12).  mask[b, j] == 1 marks a masked key (inc/cpuSoftmax.hpp:9,24).  Rows whose keys are all
// masked produce 0 * (1/0)-free zeros in the reference (p is forced to 0), so O = 0.
// p_abs_max (optional) receives max |p| (the unused s_max of test_fmha_i8.cpp:152).
void oracle_fp32_attention_x(const float* q, const float* k, const float* v, const int8_t* mask,
                             int B, int H, int Sq, int S, int D, float* o, float* p_abs_max, int n_threads) {
  const float scale = 1 / std::sqrt(static_cast<float>(D));
  std::vector<float> pmax(static_cast<size_t>(B) * H, 0.f);
  parallel_for(B * H, n_threads, [&, scale](int bh) {
    const int b = bh / H;
    const float* qb = q + static_cast<int64_t>(bh) * Sq * D;
    const float* kb = k + static_cast<int64_t>(bh) * S * D;
    const float* vb = v + static_cast<int64_t>(bh) * S * D;
    const int8_t* mb = mask + static_cast<int64_t>(b) * S;
    float* ob = o + static_cast<int64_t>(bh) * Sq * D;
    std::vector<float> s(S), p(S);
    float local_pmax = 0.f;
    for (int i = 0; i < Sq; ++i) {
      for (int j = 0; j < S; ++j) {
        float acc = 0;
        for (int d = 0; d < D; ++d) acc += qb[i * D + d] * kb[j * D + d];
        s[j] = 1.0f * acc + 0.0f * 0.0f;  // alpha*sum + beta*C with alpha=1, beta=0 on a zeroed C
      }
      float mx = -INFINITY, sum = 0.0f;
      for (int j = 0; j < S; ++j) {
        float sv = (mb[j] == 1) ? -INFINITY : s[j];
        mx = std::max(sv * scale, mx);
      }
      for (int j = 0; j < S; ++j) sum += (mb[j] == 1) ? 0.0f : std::exp(s[j] * scale - mx);
      for (int j = 0; j < S; ++j) {
        p[j] = (mb[j] == 1) ? 0.0f : std::exp(s[j] * scale - mx) / sum;
        local_pmax = std::max(local_pmax, std::fabs(p[j]));
      }
      for (int d = 0; d < D; ++d) {
        float acc = 0;
        for (int j = 0; j < S; ++j) acc += p[j] * vb[j * D + d];
        ob[i * D + d] = 1.0f * acc + 0.0f * 0.0f;
      }
    }
    pmax[bh] = local_pmax;
  });
  if (p_abs_max) {
    float m = 0.f;
    for (float x : pmax) m = std::max(m, x);
    *p_abs_max = m;
  }
}

// Self-attention form (the only one the reference test exercises): Sq == S.
void oracle_fp32_attention(const float* q, const float* k, const float* v, const int8_t* mask,
                           int B, int H, int S, int D, float* o, float* p_abs_max, int n_threads) {
  oracle_fp32_attention_x(q, k, v, mask, B, H, S, S, D, o, p_abs_max, n_threads);
}

// Tier C ("Q128").  Quantised attention with key tiles of 128 starting at key 0 (the last tile
// is 64 wide when S % 128 == 64), P quantised to 8 bits against each tile's own row maximum,
// tiles merged in fp32 and the running output renormalised after every tile.
//   amax = {q_amax, k_amax, v_amax, o_amax}
//   rows = optional list of flattened row ids (bh * Sq + i); nullptr => every row.
//          Output is written at out[r * D ...] for the r-th listed row (or at the row's natural
//          position when rows == nullptr).
// Tiles whose keys are all masked contribute nothing and are skipped; a row with no unmasked key
// yields zeros.
void oracle_q128_x(const int8_t* q, const int8_t* k, const int8_t* v, const int8_t* mask,
                   int B, int H, int Sq, int S, int D, const float* amax, int p_levels,
                   const int64_t* rows, int64_t n_rows, int8_t* out, int n_threads) {
  // p_levels == 128: P8 = -rn(128 p) in [-128, 0], the reference kernel's quantisation (fmha_i8.cuh:241-250).
  // p_levels == 255: P8 = rn(255 p) in [0, 255], the unsigned variant the reference README plans
  //                  (README.md:137-143,186), with the final scale v_amax / (o_amax * 255).
  const float p_mul = (p_levels == 255) ? 255.f : -128.f;
  const float p_lo = std::min(p_mul, 0.f), p_hi = std::max(p_mul, 0.f);
  const float o_sign = (p_levels == 255) ? 1.f : -1.f;
  const float row_scale = 1.0f / newton_sqrt(static_cast<float>(D));          // fmha_i8.cuh:71
  const float scale_qk = amax[0] * amax[1] / (127.f * 127.f);                  // fmha_i8.cuh:72
  const float scale_v_out = amax[2] * (1.0f / (amax[3] * ((p_levels == 255) ? 255.f : 128.f)));   // fmha_i8.cuh:318
  const int64_t total = rows ? n_rows : static_cast<int64_t>(B) * H * Sq;
  const int chunks = static_cast<int>(std::min<int64_t>(total, 4096));
  parallel_for(chunks, n_threads, [=](int c) {
    std::vector<float> sf(128), o(D);
    std::vector<int32_t> ot(D);
    int32_t p8[128];
    for (int64_t idx = c; idx < total; idx += chunks) {
      const int64_t r = rows ? rows[idx] : idx;
      const int64_t bh = r / Sq;
      const int i = static_cast<int>(r % Sq);
      const int b = static_cast<int>(bh / H);
      const int8_t* qr = q + (bh * Sq + i) * D;
      const int8_t* kb = k + bh * S * D;
      const int8_t* vb = v + bh * S * D;
      const int8_t* mb = mask + static_cast<int64_t>(b) * S;
      float m_run = -1e6f, l_run = 0.f;                                        // fmha_i8.cuh:91-92
      std::fill(o.begin(), o.end(), 0.f);
      for (int j0 = 0; j0 < S; j0 += 128) {
        const int w = std::min(128, S - j0);
        bool any = false;
        for (int c2 = 0; c2 < w; ++c2) any |= (mb[j0 + c2] == 0);
        if (!any) continue;
        float m_t = -INFINITY;
        for (int c2 = 0; c2 < w; ++c2) {
          int32_t acc = 0;
          const int8_t* kr = kb + static_cast<int64_t>(j0 + c2) * D;
          for (int d = 0; d < D; ++d) acc += static_cast<int32_t>(qr[d]) * static_cast<int32_t>(kr[d]);
          sf[c2] = (row_scale * static_cast<float>(acc)) * scale_qk;          // fmha_i8.cuh:196,218
          if (mb[j0 + c2] == 0) m_t = std::max(m_t, sf[c2]);
        }
        float l_t = 0.f;
        for (int c2 = 0; c2 < w; ++c2) {
          float p = (mb[j0 + c2] != 0) ? 0.f : expf(sf[c2] - m_t);            // fmha_i8.cuh:218-221
          l_t += p;
          p8[c2] = clamp_round_even_i32(p_mul * p, p_lo, p_hi);                      // fmha_i8.cuh:241-250 (negated when signed)
        }
        std::fill(ot.begin(), ot.end(), 0);
        for (int c2 = 0; c2 < w; ++c2) {
          if (p8[c2] == 0) continue;
          const int8_t* vr = vb + static_cast<int64_t>(j0 + c2) * D;
          for (int d = 0; d < D; ++d) ot[d] += p8[c2] * static_cast<int32_t>(vr[d]);
        }
        const float m_new = std::max(m_run, m_t);                              // fmha_i8.cuh:301
        const float e_old = expf(m_run - m_new);
        const float e_cur = expf(m_t - m_new);
        const float l_new = e_old * l_run + e_cur * l_t;
        const float rcp = 1.0f / l_new;
        for (int d = 0; d < D; ++d)                                            // fmha_i8.cuh:309-310
          o[d] = rcp * (l_run * e_old * o[d] + e_cur * (o_sign * static_cast<float>(ot[d])));
        l_run = l_new;
        m_run = m_new;
      }
      int8_t* dst = out + (rows ? idx : r) * D;
      for (int d = 0; d < D; ++d) dst[d] = clamp_round_even(scale_v_out * o[d], -127.f, 127.f);  // :327-328
    }
  });
}

// The reference kernel's own case: self-attention, signed P with 128 levels.
void oracle_q128(const int8_t* q, const int8_t* k, const int8_t* v, const int8_t* mask,
                 int B, int H, int S, int D, const float* amax,
                 const int64_t* rows, int64_t n_rows, int8_t* out, int n_threads) {
  oracle_q128_x(q, k, v, mask, B, H, S, S, D, amax, 128, rows, n_rows, out, n_threads);
}

// Whole-row scaling policies for the 8-bit P, restated from the reference's accuracy study
// (fmha_i8_quant_deviation.py:57-121; the same three policies are swept over the sequence length in
// fmha_i8_quant_error_seqlen.py:21-130).  The study works on one 512 x 64 problem in numpy without tiles:
//   scores        f_s = i32_s * q_amax/127 * k_amax/127 / sqrt(D)                       (:57-58)
//   probabilities f_p = exp(f_s - row max) / row sum, the row NORMALISED                  (:63-68)
//   quantisation  P8 = clip(round(f_p * 127 / p_amax), 0, 127) as unsigned bytes          (:38-43, SOFTMAX_QUANT_SCALE = 127 at :7)
//   output        f_o = (P8 . V8) * p_amax/127 * v_amax/127                              (:72, :98, :118)
// with p_amax = 1 ("worst case", :61), = the largest probability of the whole problem ("static", :86; the number the
// reference test computes as s_max, test_fmha_i8.cpp:152) or = the largest probability of the row ("dynamic",
// :104-112).  Here: policy 1 = per row, 2 = static with p_amax = amax[4], 3 = worst case (p_amax = 1).
// Kept from the device path so that the result can be compared with it: the order in which the score scale is
// applied (inc/fmha_i8.cuh:72,196), the mask semantics (masked key: p = 0; row without keys: zeros) and the
// requantisation of the output to int8 against o_amax with round-half-even (inc/fmha_i8.cuh:318-328).
void oracle_policy_x(const int8_t* q, const int8_t* k, const int8_t* v, const int8_t* mask,
                     int B, int H, int Sq, int S, int D, const float* amax5, int policy,
                     const int64_t* rows, int64_t n_rows, int8_t* out, int n_threads) {
  const float levels = 127.f;
  const float row_scale = 1.0f / newton_sqrt(static_cast<float>(D));
  const float scale_qk = amax5[0] * amax5[1] / (127.f * 127.f);
  const int64_t total = rows ? n_rows : static_cast<int64_t>(B) * H * Sq;
  const int chunks = static_cast<int>(std::min<int64_t>(total, 4096));
  parallel_for(chunks, n_threads, [=](int c0) {
    std::vector<float> e(S);
    std::vector<int32_t> ot(D);
    for (int64_t idx = c0; idx < total; idx += chunks) {
      const int64_t r = rows ? rows[idx] : idx;
      const int64_t bh = r / Sq;
      const int i = static_cast<int>(r % Sq);
      const int b = static_cast<int>(bh / H);
      const int8_t* qr = q + (bh * Sq + i) * D;
      const int8_t* kb = k + bh * S * D;
      const int8_t* vb = v + bh * S * D;
      const int8_t* mb = mask + static_cast<int64_t>(b) * S;
      float m = -INFINITY;
      for (int c = 0; c < S; ++c) {
        int32_t acc = 0;
        const int8_t* kr = kb + static_cast<int64_t>(c) * D;
        for (int d = 0; d < D; ++d) acc += static_cast<int32_t>(qr[d]) * static_cast<int32_t>(kr[d]);
        e[c] = (row_scale * static_cast<float>(acc)) * scale_qk;
        if (mb[c] == 0) m = std::max(m, e[c]);
      }
      float l = 0.f, p_max = 0.f;
      for (int c = 0; c < S; ++c) {
        e[c] = (mb[c] != 0) ? 0.f : expf(e[c] - m);
        l += e[c];
      }
      int8_t* dst = out + (rows ? idx : r) * D;
      if (!(l > 0.f)) { std::memset(dst, 0, D); continue; }
      for (int c = 0; c < S; ++c) { e[c] = e[c] / l; p_max = std::max(p_max, e[c]); }          // :64-68 (:108-111)
      const float p_amax = policy == 1 ? p_max : (policy == 2 ? amax5[4] : 1.0f);
      const float scale = levels / p_amax;                                                       // :39
      std::fill(ot.begin(), ot.end(), 0);
      for (int c = 0; c < S; ++c) {
        const int32_t p8 = clamp_round_even_i32(e[c] * scale, 0.f, levels);                      // :41
        if (p8 == 0) continue;
        const int8_t* vr = vb + static_cast<int64_t>(c) * D;
        for (int d = 0; d < D; ++d) ot[d] += p8 * static_cast<int32_t>(vr[d]);
      }
      const float back = (p_amax / levels) * (amax5[2] / 127.f);                                 // :72 / :98 / :118
      const float to_int8 = 127.f / amax5[3];
      for (int d = 0; d < D; ++d) dst[d] = clamp_round_even((static_cast<float>(ot[d]) * back) * to_int8, -127.f, 127.f);
    }
  });
}

// Emulation of the reference CUDA kernel AS WRITTEN (inc/fmha_i8.cuh:87-332, the 128-key-tile variants), thread
// for thread where it matters, for pinning tier C against bytes the reference kernel really produces.
// It differs from tier C in exactly two places, both selectable so that each difference can be shown on its own:
//
//   mask_minus_1e6 != 0  a masked key enters the tile maximum as int(-1e6) before scaling (:191-193) and tiles whose
//                        keys are all masked are still processed (tier C: masked keys never enter the maximum,
//                        such tiles are skipped);
//   shuffle_as_written != 0  the accumulator-to-A-operand relayout of P (:239-253) is reproduced with the semantics
//                        CUDA gives __shfl_sync: every lane PUBLISHES p_fp32_frag[xi].x[which_val_idx] computed from
//                        ITS OWN lane id, and receives what lane `which_lane_x` published.  The index the receiving
//                        lane computed is only right when the publishing lane sits in the same half of the quad
//                        (lane%4 in {0,1} vs {2,3}), so within every block of 16 keys the A operand ends up holding
//                        P columns {0-3, 12-15, 0-3, 12-15} instead of {0-15}: keys 4-11 of each block are dropped
//                        from P.V and keys 0-3 and 12-15 counted twice, while the row sum still counts every key
//                        once.  (shuffle_as_written == 0: the relayout the code intends, identity.)
//
// Assumed register layouts (the ones the reference's index arithmetic assumes, :183-196): accumulator element
// x[tc_xi*4 + tc_yi*2 + e] of lane L is (row L/4 + 8 tc_yi, column 8 tc_xi + 2 (L%4) + e); matrix_a int8 element
// x[tc_yi*4 + t] of lane L is (row L/4 + 8 tc_yi, column 4 (L%4) + t).
// Summation orders follow the kernel (per-lane partial sums over its 4 columns of each block, then the xor-2 / xor-1
// butterfly); expf stands in for __expf and 1/x for __frcp_rn.  S must be a multiple of 128.
void oracle_refkernel_emulate(const int8_t* q, const int8_t* k, const int8_t* v, const int8_t* mask,
                              int B, int H, int S, int D, const float* amax, int mask_minus_1e6, int shuffle_as_written,
                              int8_t* out, int n_threads) {
  const float row_scale = 1.0f / newton_sqrt(static_cast<float>(D));          // fmha_i8.cuh:71
  const float scale_qk = amax[0] * amax[1] / (127.f * 127.f);                  // fmha_i8.cuh:72
  const float scale_v_out = amax[2] * (1.0f / (amax[3] * 128.f));             // fmha_i8.cuh:318
  // column of P (within a block of 16 keys) that lands in A-operand column a
  int perm[16];
  for (int a = 0; a < 16; ++a) {
    if (!shuffle_as_written) { perm[a] = a; continue; }
    const int lane_x = a / 4, tc_xi = a % 4;                                   // receiving lane (within its quad) and loop index
    const int c = lane_x * 4 + tc_xi;                                          // the column it wants (:246)
    const int src = (c % 8) / 2;                                               // which_lane_x (:246)
    const int src_idx = (src * 4 + tc_xi) / 8 * 4 + tc_xi % 2;                 // which_val_idx evaluated BY THE SOURCE lane (:247), without tc_yi*2
    perm[a] = 8 * (src_idx / 4) + 2 * src + (src_idx % 2);                     // accumulator layout: column of x[src_idx] in lane src
  }
  const int64_t total = static_cast<int64_t>(B) * H * S;
  const int chunks = static_cast<int>(std::min<int64_t>(total, 4096));
  parallel_for(chunks, n_threads, [=](int c0) {
    std::vector<float> sf(128), pf(128), o(D);
    std::vector<int32_t> ot(D), sraw(128);
    int32_t p8[128];
    for (int64_t r = c0; r < total; r += chunks) {
      const int64_t bh = r / S;
      const int i = static_cast<int>(r % S);
      const int b = static_cast<int>(bh / H);
      const int8_t* qr = q + (bh * S + i) * D;
      const int8_t* kb = k + bh * S * D;
      const int8_t* vb = v + bh * S * D;
      const int8_t* mb = mask + static_cast<int64_t>(b) * S;
      float m_run = -1e6f, l_run = 0.f;                                        // fmha_i8.cuh:91-92
      std::fill(o.begin(), o.end(), 0.f);
      for (int j0 = 0; j0 < S; j0 += 128) {
        if (!mask_minus_1e6) {
          bool any = false;
          for (int c2 = 0; c2 < 128; ++c2) any |= (mb[j0 + c2] == 0);
          if (!any) continue;
        }
        for (int c2 = 0; c2 < 128; ++c2) {
          int32_t acc = 0;
          const int8_t* kr = kb + static_cast<int64_t>(j0 + c2) * D;
          for (int d = 0; d < D; ++d) acc += static_cast<int32_t>(qr[d]) * static_cast<int32_t>(kr[d]);
          sraw[c2] = acc;
        }
        // tile maximum (:183-206): pairs of columns, masked values replaced before scaling
        float m_t = mask_minus_1e6 ? -1e6f : -INFINITY;
        for (int c2 = 0; c2 < 128; c2 += 2) {
          if (mask_minus_1e6) {
            const int v1 = mb[j0 + c2] ? static_cast<int>(-1e6) : sraw[c2];
            const int v2 = mb[j0 + c2 + 1] ? static_cast<int>(-1e6) : sraw[c2 + 1];
            m_t = std::max(m_t, row_scale * static_cast<float>(std::max(v1, v2)) * scale_qk);
          } else {
            if (!mb[j0 + c2]) m_t = std::max(m_t, row_scale * static_cast<float>(sraw[c2]) * scale_qk);
            if (!mb[j0 + c2 + 1]) m_t = std::max(m_t, row_scale * static_cast<float>(sraw[c2 + 1]) * scale_qk);
          }
        }
        // probabilities and the row sum in the kernel's order (:208-235): lane L of the quad owns columns
        // 16 xi + 8 tc_xi + 2 L + {0,1}; partial sums per lane, then (s0 + s2) + (s1 + s3)
        float lane_sum[4] = {0.f, 0.f, 0.f, 0.f};
        for (int xi = 0; xi < 8; ++xi)
          for (int tc_xi = 0; tc_xi < 2; ++tc_xi)
            for (int L = 0; L < 4; ++L) {
              const int c2 = 16 * xi + 8 * tc_xi + 2 * L;
              const float e0 = expf(row_scale * static_cast<float>(sraw[c2]) * scale_qk - m_t);
              const float e1 = expf(row_scale * static_cast<float>(sraw[c2 + 1]) * scale_qk - m_t);
              pf[c2] = mb[j0 + c2] ? 0.f : e0;
              pf[c2 + 1] = mb[j0 + c2 + 1] ? 0.f : e1;
              lane_sum[L] += (pf[c2] + pf[c2 + 1]);
            }
        const float l_t = (lane_sum[0] + lane_sum[2]) + (lane_sum[1] + lane_sum[3]);
        for (int c2 = 0; c2 < 128; ++c2)                                         // :241-250
          p8[c2] = clamp_round_even_i32(-128.f * pf[c2], -128.f, 0.f);
        std::fill(ot.begin(), ot.end(), 0);
        for (int xi = 0; xi < 8; ++xi)
          for (int a = 0; a < 16; ++a) {
            const int pv = p8[16 * xi + perm[a]];
            if (pv == 0) continue;
            const int8_t* vr = vb + static_cast<int64_t>(j0 + 16 * xi + a) * D;
            for (int d = 0; d < D; ++d) ot[d] += pv * static_cast<int32_t>(vr[d]);
          }
        const float m_new = std::max(m_run, m_t);                              // :301-310
        const float e_old = expf(m_run - m_new);
        const float e_cur = expf(m_t - m_new);
        const float l_new = e_old * l_run + e_cur * l_t;
        const float rcp = 1.0f / l_new;
        for (int d = 0; d < D; ++d)
          o[d] = rcp * (l_run * e_old * o[d] + e_cur * (-1.f * static_cast<float>(ot[d])));
        l_run = l_new;
        m_run = m_new;
      }
      int8_t* dst = out + r * D;
      for (int d = 0; d < D; ++d) dst[d] = clamp_round_even(scale_v_out * o[d], -127.f, 127.f);  // :327-328
    }
  });
}

// The constant the device kernel and tier C share for 1/sqrt(head_dim).
float oracle_row_scale(int D) { return 1.0f / newton_sqrt(static_cast<float>(D)); }

}  // extern "C"
