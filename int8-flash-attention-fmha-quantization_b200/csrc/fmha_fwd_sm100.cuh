// The INT8 flash-attention forward kernel for sm_100a.
//
// Replaces the reference project's FMHAInferKernel (inc/fmha_i8.cuh:43-334).  Same arithmetic
// contract -- key tiles of 128 starting at key 0, P quantised to 8 bits against each tile's own row
// maximum, tiles merged in fp32 -- on a different machine model:
//
//   work unit  = (batch*head, one 128-row query tile).  The kernel is persistent: min(units, SMs)
//                CTAs, one per SM, CTA c walks units c, c + grid, ...  A CTA's whole life is ONE
//                sequence of steps g = 0, 1, 2, ... (step = one live key tile of one unit); barrier
//                phases, the K/V ring and tensor memory carry on from one unit to the next, so no role
//                drains at a unit boundary.
//   two chains = the softmax warps form two teams; steps alternate between them (chain = g & 1).
//   S buffers  = S = Q.K^T of step g lands in accumulator g % n of tensor memory (n = 3 at head_dim 128, 4 at
//                head_dim 64), issued as soon as that accumulator is free, i.e. several steps ahead of the
//                softmax warps.  The same accumulator then carries the step through the rest of its life: once the
//                softmax threads have consumed S, P.V of the step writes its partial output there.  The 8-bit P row
//                goes into a 32-column annex of the accumulator (head_dim 128) or over the two ends of the
//                accumulator itself (head_dim 64, where the partial output needs only 64 columns in between).  So
//                every step in flight owns its whole set of buffers and no role ever waits for another STEP's
//                buffer, only for its own step's previous stage.
//
//   warp 0       loader: TMA brings Q (once per unit, in a small ring) and rings of K and of V tiles into
//                swizzled shared memory, running ahead into the next units.
//   warp 1       S issuer:  S_b = bias + Q . K_g^T  (tcgen05.mma smem x smem -> int32 in tensor memory).
//   warp 2       scanner: turns the coming units' padding-mask rows into per-tile bit masks and the list of
//                key tiles that hold at least one unmasked key (ring of four).
//   warp 3       P.V issuer:  O~ = bias + P_b . V_g  (tcgen05.mma tmem x smem -> int32 in tensor memory) when the
//                softmax warps have written P_b.
//                These four run warp-wide -- every lane waits and counts, one elected lane issues -- so that
//                descriptors and addresses are warp-uniform values; issued from a single divergent lane an MMA
//                cost about 100 cycles of issue time, this way about 70.
//   warps 4-11   merge: two threads per query row, each holding one half (D/2 columns) of the fp32 running
//                output row.  After P.V of a step they drain the partial output from tensor memory, rescale
//                and add it; at the end of a unit they normalise, requantise and store the row.  This keeps
//                the per-tile drain and the epilogue off the softmax warps.
//   warps 12-27  softmax: warps 12-19 serve chain 0, warps 20-27 chain 1.  TWO threads share one query row:
//                thread `half` owns keys [64*half, 64*half+64) of the tile.  Each reads its part of S twice
//                (integer max, then exp + requantise), the two exchange their maxima through shared memory,
//                and each writes its 8-bit P values into the annex or, at head_dim 64, over columns it has already
//                consumed (the lower half row walks up and leaves P in columns [0,16), the upper one walks down
//                and leaves it in [112,128)).
//                These threads hold no output row, so they are light (64 registers).
//
// The bias: every accumulator is first written by a one-step fp16 MMA whose operands hold 4096 and
// 3072, i.e. the fp32 value 1.5*2^23 (bits 0x4B400000); the int8 MMAs then add their integer result
// to that bit pattern.  Read back as a float the accumulator is exactly 1.5*2^23 + s, so no thread
// ever converts integers to floats: one fused multiply-add turns the raw accumulator into the
// exponent argument (or into the rescaled partial output).
//
// Tensor memory (512 columns x 128 lanes x 32 bit): accumulator b at columns [128 b, 128 b + 128).
// head_dim 128: annex b at [384 + 32 b, 384 + 32 b + 32) holds P (four int8 per column, keys in order), the partial
// output fills the accumulator.  head_dim 64: inside the accumulator, P of keys 0-63 in columns [0,16), P of keys
// 64-127 in columns [112,128), partial output in [16,80).
//
// Numerics kept equal to the reference kernel within the test tolerance: the running output is kept
// unnormalised (divided by the row sum once at the end) instead of renormalised after every tile,
// exp() is ex2.approx on an argument formed exactly from the integer accumulator, and masked keys
// contribute exactly zero (the reference adds a large negative number before scaling,
// inc/fmha_i8.cuh:191-193).  Key tiles with no unmasked key are skipped.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "ptx.cuh"
#include "../../include/fmha_i8_c.h"

// 1: the partial-output accumulators are preset to the bit pattern of 1.5*2^23 by a one-step fp16 MMA (as the S
//    accumulators are), so the merge threads read floats; 0: they add that bit pattern themselves, one integer
//    addition per element.
#ifndef FMHA_PV_BIAS_MMA
#define FMHA_PV_BIAS_MMA 1
#endif
// Ring depths can be overridden at compile time for tuning runs.
#ifndef FMHA_STAGES_K128
#define FMHA_STAGES_K128 3
#endif
#ifndef FMHA_STAGES_V128
#define FMHA_STAGES_V128 6
#endif
#ifndef FMHA_STAGES_K64
#define FMHA_STAGES_K64 4
#endif
#ifndef FMHA_STAGES_V64
#define FMHA_STAGES_V64 8
#endif

namespace fmha {

// Optional timeline tracing for performance work: with -DFMHA_TRACE the first CTA records clock64()
// stamps of its phase boundaries.  Compiled out of the product build.
#ifdef FMHA_TRACE
__device__ long long g_trace[48][512];
#define FMHA_STAMP(slot, idx) do { if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && (idx) < 512u) g_trace[slot][idx] = clock64(); } while (0)
#else
#define FMHA_STAMP(slot, idx) do { } while (0)
#endif

constexpr int kTile = 128;           // query rows per tile == keys per tile
constexpr int kHalf = 64;            // keys per softmax thread
constexpr int kMaxSeq = 32768;
constexpr int kMaxTiles = kMaxSeq / kTile;
constexpr int kSoftmaxWarps = 16;    // 2 chains x 2 key halves x 4 lane quarters
constexpr int kMergeWarps = 8;       // 2 column halves x 4 lane quarters
constexpr int kFwdWarps = kSoftmaxWarps + kMergeWarps + 4;
constexpr int kFwdThreads = kFwdWarps * 32;          // 896
// Warp numbering: the one-warp roles first, then the merge warps, then the softmax warps (a role's lane quarter of
// tensor memory is its warp number modulo 4; register targets are set per group of four warps).
constexpr int kWarpLoad = 0;
constexpr int kWarpMmaS = 1;
constexpr int kWarpScan = 2;
constexpr int kWarpMmaO = 3;
constexpr int kWarpMerge0 = 4;
constexpr int kWarpSoftmax0 = kWarpMerge0 + kMergeWarps;
// Tensor memory.  A buffer set is one 128-column accumulator that first holds S of a step and then, once the softmax
// threads have consumed it, the partial output P.V of the same step.
//   head_dim 128: three sets (384 columns) plus three 32-column annexes that take the P bytes of the step (480 columns);
//                 the partial output covers the whole accumulator, so P.V is one group of MMAs with N = 128.
//   head_dim 64:  four sets (512 columns); the P bytes stay inside the accumulator, keys 0-63 in its first 16 columns and
//                 keys 64-127 in its last 16, and the 64-column partial output sits between them from column 16 on.
//                 (Three sets with annexes, as at head_dim 128, run 5 % faster on sequences of 2048 and more and 5 %
//                 slower at sequence length 512, where the S issuer works several units ahead.)
template <int D> struct SBufs { static constexpr int n = (D == 128) ? 3 : 4; };
constexpr int kSBufsMax = 4;
template <int D> struct PLayout {
  static constexpr bool kAnnex = (D == 128);
  static constexpr int kOOff = kAnnex ? 0 : 16;        // first column of the partial output inside its accumulator
  static constexpr int kAnnexCols = 32;                // 128 keys x 1 byte
  // column (relative to the accumulator of the set, or to the set's annex) of the P bytes of keys [32 kk, 32 kk + 32)
  __host__ __device__ static constexpr int p_col(int kk) { return kAnnex ? 8 * kk : (kk >> 1) * 112 + (kk & 1) * 8; }
};
constexpr int kInfoBufs = 4;         // units whose mask information is resident at once
constexpr int kInfoConsumers = 3 + kSoftmaxWarps + kMergeWarps;   // loader, two issuers, softmax and merge warps release an info buffer once each
// setmaxnreg moves registers inside the CTA's own launch allocation (registers per thread at launch x
// threads), not inside the SM's whole register file: a request that does not fit blocks forever.  With
// 896 threads the launch allocation is 72 registers per thread (the host checks this before the first
// launch and refuses otherwise); the targets per role (FwdRegs) add up to 28 x 72.
constexpr int kLaunchRegs = 72;
template <int D> struct FwdRegs {
  // head_dim 128: the merge threads hold a 64-register half output row, the one-warp roles run lean (measured on C3:
  // 104/40 is 2 % faster than 96/56).  head_dim 64: the output row is 32 registers; 88/72 is the split at which
  // ptxas reports no spills at all, and C5 runs 5 % faster with it than with 80/88 or 96/56, which both spill.
  static constexpr int kSoftmax = 64, kMerge = (D == 128) ? 104 : 88, kOther = (D == 128) ? 40 : 72;
  static_assert(kSoftmaxWarps * kSoftmax + kMergeWarps * kMerge + 4 * kOther <= kFwdWarps * kLaunchRegs,
                "setmaxnreg targets exceed the CTA's register allocation: the kernel would hang");
  static_assert(kSoftmax <= kLaunchRegs && kMerge >= kLaunchRegs, "the softmax warps give registers, the merge warps gain");
};

constexpr uint32_t kTmemCols = 512;
constexpr float kMagic = 12582912.0f;          // 1.5 * 2^23: float whose ulp is 1 over [2^23, 2^24)
constexpr uint32_t kMagicBits = 0x4B400000u;
constexpr int kBiasBytes = 4096;               // 128 rows x 16 fp16, unswizzled core-matrix layout

template <int D> struct FwdCfg {
  static_assert(D == 64 || D == 128, "head_dim must be 64 or 128");
  static constexpr int kStagesK = (D == 128) ? FMHA_STAGES_K128 : FMHA_STAGES_K64;   // ring depth of K
  // ring depth of V: one thread loads K(g), V(g), K(g+1), ... in order, and V(g) is consumed a few steps (the number of S accumulators) after
  // K(g), so the V ring has to be that much deeper than the K ring
  static constexpr int kStagesV = (D == 128) ? FMHA_STAGES_V128 : FMHA_STAGES_V64;
  static_assert(kStagesV >= kStagesK + SBufs<D>::n, "V ring too shallow for the in-order loader");
  // Q tiles resident at once: the S cursor runs three steps ahead, which with one-tile units means three
  // units ahead, so short-sequence shapes want more than two (head_dim 128 has no shared memory to spare)
  static constexpr int kQBufs = (D == 128) ? 2 : 4;
  static constexpr int kTileBytes = kTile * D;              // one 128-row tile of int8
  static constexpr int kTilesBytesTotal = (kQBufs + kStagesK + kStagesV) * kTileBytes;
};

struct FwdParams {
  const int8_t* mask;   // [B,S] whole mask
  int8_t* o;            // first head of the slice
  int o_wide;           // o is 32-byte aligned: the epilogue may use 32-byte stores
  int S;                // keys per head (seq_len; seq_len_k when queries and keys differ in number)
  int Sq;               // query rows per head (== S for self-attention)
  int H, bh_begin, bh_count, q_tiles;
  int n_units;          // bh_count * q_tiles work units, taken round-robin by the resident CTAs
  float row_scale;      // 1/sqrt(D), the reference's constant (inc/fmha_i8.cuh:71)
  float scale_qk;       // q_amax*k_amax/127^2 (inc/fmha_i8.cuh:72)
  float scale_v_out;    // v_amax/(o_amax*128) (inc/fmha_i8.cuh:318)
  float c2;             // row_scale*scale_qk*log2(e)
  float p_mul;          // -128: P8 = -rn(128 p) signed, the reference's quantisation (inc/fmha_i8.cuh:241-250);
                        // +255: P8 = rn(255 p) unsigned (the reference README's planned UINT8 x INT8 variant)
  float o_sign;         // -1 when the accumulator holds -(P.V) (signed P), +1 when it holds +(P.V)
  unsigned p_unsigned;  // 1 = the tensor core reads P as unsigned bytes
  float* amax_out;      // calibration mode when not null: nothing is stored to o; instead the largest |output|
                        // in real units, max |O~ / l| * amax_scale, is folded into this device float
  float amax_scale;     // v_amax / (127 * 128)  (127 * 255 with unsigned P)
  unsigned* status;     // eight device status words
  // Whole-row P scaling policies (the reference's accuracy study, fmha_i8_quant_deviation.py:57-121), two launches:
  float2* row_stats_out;       // statistics launch: per query row {bits of the biased integer row maximum over ALL keys,
                               // sum over all keys of exp(score - row maximum)} is written here, nothing to o
  const float2* row_stats_in;  // policy launch (kernel instantiated with kPolicy): those statistics, read back
  float p_row_mul;      // policy launch: P8 = rn(p_row_mul * exp(score - row max))                  ("dynamic", per-row scale), or
  float p_static_mul;   //                P8 = min(rn(p_static_mul * exp(score - row max) / l), levels)  ("static" scale; 0 = dynamic)
  float p_levels;       // quantisation levels of P in a policy launch (127 in the reference's study)
                        // (a policy launch sets scale_v_out to the factor that turns sum_j P8 v8 [/ l] into int8 output units)
};

// What every role needs to know about one work unit's padding mask.  kInfoBufs of these live in shared
// memory: the scanner warp fills the ones of coming units while the current unit is being processed.
struct UnitInfo {
  int n_live;                         // key tiles with at least one unmasked key
  uint32_t maskbits[kMaxTiles * 4];   // bit set = key masked (or beyond seq_len)
  uint16_t live[kMaxTiles];           // indices of the live key tiles, ascending
  uint8_t mixed[kMaxTiles];           // 1 = that live tile has masked keys too
};

template <int NK, int NV> struct FwdCtl {
  uint64_t q_full[4], q_empty[4];      // Q ring (kQBufs used): rows have landed / the unit's last S = Q.K^T has completed
  uint64_t k_full[NK], k_empty[NK], v_full[NV], v_empty[NV];
  uint64_t s_full[kSBufsMax];          // per S accumulator: S = Q.K^T has completed
  uint64_t s_free[kSBufsMax];          // per S accumulator: the merge threads have drained the partial output that lived in it
  uint64_t o_full[kSBufsMax];          // per S accumulator: P.V of the step that owns it has completed
  uint64_t p_ready[4];                 // per step slot (g & 3): P written, row statistics published
  uint64_t xch[2][4];                  // per chain and lane quarter: the two half-row threads have published their maxima
  uint64_t info_full[kInfoBufs], info_empty[kInfoBufs];
  uint32_t tmem_base;
  int abort;
  // row statistics of a step, written by the softmax threads and read by the merge threads (slot = g & 3)
  float st_m[4][kTile], st_f[4][kTile], st_s0[4][kTile], st_s1[4][kTile];
  int st_i[4][kTile];                  // biased integer row maximum of the step's tile (for the statistics launch)
  int xmax[2][2][2][kTile];            // [chain][step parity][half][row]: biased integer maximum of that half row
  UnitInfo info[kInfoBufs];
};

// Device view of one word of mapped host memory (set by the host once per device; null until then).
// A wait that gives up writes 1 to it so that the next host call sees the failure without a synchronisation.
__device__ unsigned* g_host_flag_ptr;

__device__ __noinline__ void raise_status(volatile int* abort_flag, unsigned* status, unsigned code, unsigned tile) {
  *abort_flag = 1;
  if (atomicCAS(&status[0], 0u, code) == 0u) {
    status[1] = blockIdx.x;
    status[2] = threadIdx.x >> 5;
    status[3] = tile;
    unsigned* host_word = g_host_flag_ptr;
    if (host_word != nullptr) {
      *reinterpret_cast<volatile unsigned*>(host_word) = 1u;
      __threadfence_system();
    }
  }
}

__device__ __forceinline__ float clear_low2(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFFFFFFCu); }

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Builds one unit's view of its batch's padding mask: 128-bit masks per key tile, the list of live
// tiles and whether each needs the per-key path.  Executed by ONE warp.
__device__ __forceinline__ void scan_mask_warp(UnitInfo* info, const int8_t* mask_row, int S, int n_tiles) {
  const int lane = threadIdx.x & 31;
  const uint32_t* words = reinterpret_cast<const uint32_t*>(mask_row);
  for (int g = lane; g < n_tiles * 4; g += 32) {
    const int key0 = g * 32;
    uint32_t bits = 0xFFFFFFFFu;
    if (key0 < S) {  // S is a multiple of 64, so a 32-key group is entirely inside or outside
      bits = 0u;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t wv = __ldg(words + (key0 >> 2) + i);
#pragma unroll
        for (int b = 0; b < 4; ++b)
          if ((wv >> (8 * b)) & 0xFFu) bits |= 1u << (4 * i + b);
      }
    }
    info->maskbits[g] = bits;
  }
  __syncwarp();
  int n = 0;
  for (int base = 0; base < n_tiles; base += 32) {
    const int t = base + lane;
    bool is_live = false, is_mixed = false;
    if (t < n_tiles) {
      const uint32_t a = info->maskbits[4 * t], b = info->maskbits[4 * t + 1], c = info->maskbits[4 * t + 2], d = info->maskbits[4 * t + 3];
      is_live = (a & b & c & d) != 0xFFFFFFFFu;
      is_mixed = (a | b | c | d) != 0u;
    }
    const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, is_live);
    if (is_live) {
      const int pos = n + __popc(ballot & ((1u << lane) - 1u));
      info->live[pos] = static_cast<uint16_t>(t);
      info->mixed[pos] = is_mixed ? 1 : 0;
    }
    n += __popc(ballot);
  }
  if (lane == 0) info->n_live = n;
  __syncwarp();
}

// Writes the two constant fp16 operands of the bias MMA: A[m][0] = 4096, B[n][0] = 3072, all other
// elements zero, in the unswizzled K-major layout (core matrix = 8 rows x 16 bytes, the two K halves
// of a row group 128 bytes apart, row groups 256 bytes apart).
__device__ __forceinline__ void fill_bias_operands(uint8_t* bias_a, uint8_t* bias_b) {
  for (int i = threadIdx.x; i < 2 * kBiasBytes / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(bias_a)[i] = make_uint4(0u, 0u, 0u, 0u);   // bias_b follows bias_a
  __syncthreads();
  if (threadIdx.x < kTile) {
    const int m = threadIdx.x;
    const int off = (m >> 3) * 256 + (m & 7) * 16;
    *reinterpret_cast<uint16_t*>(bias_a + off) = 0x6C00u;   // 4096.0 in fp16
    *reinterpret_cast<uint16_t*>(bias_b + off) = 0x6A00u;   // 3072.0 in fp16
  }
  fence_proxy_async_smem();
}

// Row maximum over N raw accumulator words (biased integers compare like the integers themselves).
// mw: bit i set = key i of this chunk is masked.
template <bool kMixed, int N>
__device__ __forceinline__ void chunk_max(const uint32_t (&r)[N], uint32_t mw, int& max_a, int& max_b) {
#pragma unroll
  for (int i = 0; i < N; i += 4) {
    int a = static_cast<int>(r[i]), b = static_cast<int>(r[i + 1]), c = static_cast<int>(r[i + 2]), d = static_cast<int>(r[i + 3]);
    if (kMixed) {
      if ((mw >> i) & 1u) a = INT_MIN;
      if ((mw >> (i + 1)) & 1u) b = INT_MIN;
      if ((mw >> (i + 2)) & 1u) c = INT_MIN;
      if ((mw >> (i + 3)) & 1u) d = INT_MIN;
    }
    max_a = max(max_a, max(a, b));
    max_b = max(max_b, max(c, d));
  }
}

// N scores -> N probabilities (summed into two independent packed accumulators) -> N/4 words of
// packed bytes holding -rn(128 p) (or rn(255 p)).  x = raw accumulator read as float = kMagic + s.
// kCap: p is limited to p_cap before it is quantised (the static policy clips at its top level, fmha_i8_quant_deviation.py:38-43).
template <bool kMixed, int N, bool kCap = false>
__device__ __forceinline__ void chunk_exp_pack(const uint32_t (&r)[N], uint32_t mw, const float2 c2, const float2 neg_hi,
                                               const float2 p_mul_f, float2 (&sum)[2], uint32_t (&packed)[N / 4], const float p_cap = 0.f) {
  const float2 magic2 = make_float2(kMagic, kMagic);
#pragma unroll
  for (int g = 0; g < N / 4; ++g) {
    float2 x01 = make_float2(__uint_as_float(r[4 * g]), __uint_as_float(r[4 * g + 1]));
    float2 x23 = make_float2(__uint_as_float(r[4 * g + 2]), __uint_as_float(r[4 * g + 3]));
    if (kMixed) {
      if ((mw >> (4 * g)) & 1u) x01.x = -INFINITY;
      if ((mw >> (4 * g + 1)) & 1u) x01.y = -INFINITY;
      if ((mw >> (4 * g + 2)) & 1u) x23.x = -INFINITY;
      if ((mw >> (4 * g + 3)) & 1u) x23.y = -INFINITY;
    }
    const float2 a01 = __ffma2_rn(x01, c2, neg_hi);
    const float2 a23 = __ffma2_rn(x23, c2, neg_hi);
    float2 p01 = make_float2(ex2_approx(a01.x), ex2_approx(a01.y));
    float2 p23 = make_float2(ex2_approx(a23.x), ex2_approx(a23.y));
    if (kCap) {
      p01.x = fminf(p01.x, p_cap); p01.y = fminf(p01.y, p_cap);
      p23.x = fminf(p23.x, p_cap); p23.y = fminf(p23.y, p_cap);
    }
    sum[0] = __fadd2_rn(sum[0], p01);
    sum[1] = __fadd2_rn(sum[1], p23);
    const float2 y01 = __ffma2_rn(p01, p_mul_f, magic2);      // low byte = the two's-complement P8
    const float2 y23 = __ffma2_rn(p23, p_mul_f, magic2);
    packed[g] = __byte_perm(__byte_perm(__float_as_uint(y01.x), __float_as_uint(y01.y), 0x0040),
                            __byte_perm(__float_as_uint(y23.x), __float_as_uint(y23.y), 0x0040), 0x5410);
  }
}

// Constants of one row of one tile, derived from the biased integer row maximum.
struct RowConsts {
  float2 c2, neg_hi, p_mul_f;
  float f, m_tile;
};
__device__ __forceinline__ RowConsts row_consts(const int imax, const float c2s, const float row_scale, const float scale_qk, const float p_mul) {
  // exponent argument (s - smax) * c2 = x * c2 - M * c2 with x = kMagic + s and M = kMagic + smax.
  // M * c2 = hi + lo exactly (lo is the rounding residual); the factor 2^-lo is folded into the
  // quantisation constant and the row sum, so nothing is lost and nothing is paid per element.
  RowConsts k;
  const float M = __uint_as_float(static_cast<uint32_t>(imax));
  const float hi = M * c2s;
  const float lo = fmaf(M, c2s, -hi);
  k.f = fmaf(-lo, 0.6931471805599453f, 1.0f);
  k.c2 = make_float2(c2s, c2s);
  k.neg_hi = make_float2(-hi, -hi);
  k.p_mul_f = make_float2(p_mul * k.f, p_mul * k.f);        // -128 f (or +255 f): quantisation multiplier
  // the value the reference computes for the maximal element (inc/fmha_i8.cuh:196)
  k.m_tile = (row_scale * static_cast<float>(imax - static_cast<int>(kMagicBits))) * scale_qk;
  return k;
}

// o2 (+)= e_cur * (P8 . V) for N output columns.  r = accumulator: either preset by the bias MMA, so that it reads
// as the float kMagic + (P8 . V), or a raw int32 (|r| < 2^22) that becomes that float by adding the bit pattern
// of 1.5*2^23 -- no conversion instruction either way.
template <int N>
__device__ __forceinline__ void drain_chunk(const uint32_t (&r)[N], float2* o2, const float2 neg_ec, const float2 e_bias, const float2 e_old) {
#pragma unroll
  for (int i = 0; i < N / 2; ++i) {
#if FMHA_PV_BIAS_MMA
    const float2 x = make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
#else
    const float2 x = make_float2(__uint_as_float(r[2 * i] + kMagicBits), __uint_as_float(r[2 * i + 1] + kMagicBits));
#endif
    const float2 t = __ffma2_rn(x, neg_ec, e_bias);          // e_cur * (P8 . V), exact product before rounding
    o2[i] = __ffma2_rn(o2[i], e_old, t);
  }
}

// Geometry of work unit u.
struct UnitGeom {
  int bh_local, batch, q_row0;
};
__device__ __forceinline__ UnitGeom unit_geom(const FwdParams& p, int u) {
  UnitGeom g;
  g.bh_local = u / p.q_tiles;
  g.batch = (p.bh_begin + g.bh_local) / p.H;
  g.q_row0 = (u - g.bh_local * p.q_tiles) * kTile;
  return g;
}

// ---------------------------------------------------------------------------------------------- softmax role
// One thread = one half (64 keys) of one query row of one chain.  Walks the CTA's step sequence and
// handles the steps of its chain.
template <int D, bool kPolicy>
__device__ __forceinline__ void softmax_role(const FwdParams& p, FwdCtl<FwdCfg<D>::kStagesK, FwdCfg<D>::kStagesV>* ctl, const uint32_t tmem_base,
                                             const int first_unit, const int unit_step) {
  const int warp = (threadIdx.x >> 5) - kWarpSoftmax0, lane = threadIdx.x & 31;
  const int chain = warp >> 3, half = (warp >> 2) & 1, quad = warp & 3;
  const int row = quad * 32 + lane;
  // my 64 columns of S buffer 0; my P bytes go over their first 16 columns
  const uint32_t tS0 = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(half * kHalf);
  const uint32_t bar_x = smem_u32(&ctl->xch[chain][quad]);
  volatile int* abort_flag = &ctl->abort;
  const float c2s = p.c2, row_scale = p.row_scale, scale_qk = p.scale_qk, p_mul = p.p_mul;

  uint32_t n = 0;     // steps this chain has processed so far (phase of xch)
  uint32_t g0 = 0;    // global index of the current unit's first step
  int it = 0;
  for (int u = first_unit; u < p.n_units; u += unit_step, ++it) {
    const int buf = it % kInfoBufs;
    if (!__all_sync(0xFFFFFFFFu, mbar_wait_slow(smem_u32(&ctl->info_full[buf]), static_cast<uint32_t>((it / kInfoBufs) & 1), abort_flag))) {
      raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_INFO, it);
      return;
    }
    const UnitInfo* info = &ctl->info[buf];
    const int n_live = info->n_live;
    // Policy launch: the row's maximum over ALL keys and its exp-sum come from the statistics launch; one scale per
    // row for the whole unit, no tile maximum, no exchange (fmha_i8_quant_deviation.py:62-121).
    RowConsts kp;
    float p_cap = 0.f;
    if (kPolicy) {
      const UnitGeom geo = unit_geom(p, u);
      const int q_row = geo.q_row0 + row;
      float2 st = make_float2(__int_as_float(static_cast<int>(kMagicBits)), 1.f);
      if (q_row < p.Sq) st = __ldg(&p.row_stats_in[static_cast<int64_t>(geo.bh_local) * p.Sq + q_row]);
      const float l_row = st.y > 0.f ? st.y : 1.f;
      // dynamic: P8 = rn(levels * e); static: P8 = min(rn(levels * (e / l) / s_max), levels)
      const float mul = (p.p_static_mul != 0.f) ? p.p_static_mul / l_row : p.p_row_mul;
      kp = row_consts(__float_as_int(st.x), c2s, row_scale, scale_qk, mul);
      p_cap = p.p_levels / kp.p_mul_f.x;        // an exponential above this would quantise beyond the top level
    }
#pragma unroll 1
    for (int j = (chain ^ static_cast<int>(g0)) & 1; j < n_live; j += 2, ++n) {
      const uint32_t g = g0 + static_cast<uint32_t>(j);
      const uint32_t sb = g % SBufs<D>::n;                       // S accumulator of this step
      const uint32_t tS = tS0 + sb * kTile;
      // (read before the wait: none of it depends on S)
      const bool mixed = info->mixed[j] != 0;
      // the 64 mask bits of my keys (only looked at on the mixed path)
      const uint32_t* mwords = &info->maskbits[4 * info->live[j] + 2 * half];
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&ctl->s_full[sb]), (g / SBufs<D>::n) & 1u, abort_flag))) {
        raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_S_READY, g);
        return;
      }
      tc_fence_after();
      if (half == 0 && quad == 0) FMHA_STAMP(chain * 4 + 0, n);

      // Order of my four 16-column chunks: the lower half row walks up, the upper half row walks DOWN.  At head_dim 64
      // that lets each leave its P bytes over columns it has already consumed (the first 16 and the last 16 of the
      // accumulator); columns [16,112) stay untouched, and P.V of this step puts the partial output there.
      const int c0 = half ? 3 : 0, cs = half ? -1 : 1;                 // first chunk and direction
      // my 16 columns of P: inside the accumulator (head_dim 64) or in the annex of the buffer set (head_dim 128)
      const uint32_t tP = PLayout<D>::kAnnex
          ? tS0 - static_cast<uint32_t>(half * kHalf) + SBufs<D>::n * kTile + sb * PLayout<D>::kAnnexCols + static_cast<uint32_t>(half * 16)
          : tS + (half ? 48u : 0u);

      uint32_t ra[16], rb[16];
      RowConsts k;
      if (kPolicy) {
        k = kp;
        tmem_ld16_issue(tS + c0 * 16, ra);
      } else {
      // ---- pass 1: biased integer maximum of my 64 columns (inc/fmha_i8.cuh:183-206)
      int max_a = INT_MIN, max_b = INT_MIN;
      if (!mixed) {
        // two tensor-memory round trips (a round trip costs about as much as the whole arithmetic of this pass), two
        // 16-column loads in flight each time: 32 registers of data live instead of the 48 that one 32-column load
        // plus the prefetch for pass 2 would need
        tmem_ld16_issue(tS, ra);
        tmem_ld16_issue(tS + 16, rb);
        tmem_ld_fence(ra); tmem_ld_fence(rb);
        chunk_max<false, 16>(ra, 0u, max_a, max_b);
        tmem_ld16_issue(tS + 32, ra);
        chunk_max<false, 16>(rb, 0u, max_a, max_b);
        tmem_ld16_issue(tS + 48, rb);
        tmem_ld_fence(ra); tmem_ld_fence(rb);
        chunk_max<false, 16>(ra, 0u, max_a, max_b);
        tmem_ld16_issue(tS + c0 * 16, ra);                             // first chunk of pass 2, in flight during the exchange
        chunk_max<false, 16>(rb, 0u, max_a, max_b);
      } else {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          tmem_ld16_issue(tS + c * 16, ra);
          tmem_ld_fence(ra);
          chunk_max<true, 16>(ra, (mwords[c >> 1] >> ((c & 1) * 16)) & 0xFFFFu, max_a, max_b);
        }
        tmem_ld16_issue(tS + c0 * 16, ra);
      }
      const int mine = max(max_a, max_b);
      // ---- exchange with the thread that owns the other half of this row
      int* xrow = &ctl->xmax[chain][n & 1u][0][row];
      xrow[half * kTile] = mine;
      mbar_arrive(bar_x);
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(bar_x, n & 1u, abort_flag))) {
        tmem_ld_fence(ra);
        raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_S_READY, g);
        return;
      }
      const int imax = max(mine, xrow[(half ^ 1) * kTile]);
      k = row_consts(imax, c2s, row_scale, scale_qk, p_mul);
      if (half == 0) ctl->st_i[g & 3u][row] = imax;
      }
      if (half == 0 && quad == 0) FMHA_STAMP(chain * 4 + 1, n);

      // ---- pass 2: exp, row sum, requantise, P over columns already consumed (inc/fmha_i8.cuh:208-253)
      float2 sum[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      uint32_t packed[4];
      if (!mixed) {
        tmem_ld_fence(ra); tmem_ld16_issue(tS + (c0 + cs) * 16, rb);
        chunk_exp_pack<false, 16, kPolicy>(ra, 0u, k.c2, k.neg_hi, k.p_mul_f, sum, packed, p_cap); tmem_st4(tP + c0 * 4, packed);
        tmem_ld_fence(rb); tmem_ld16_issue(tS + (c0 + 2 * cs) * 16, ra);
        chunk_exp_pack<false, 16, kPolicy>(rb, 0u, k.c2, k.neg_hi, k.p_mul_f, sum, packed, p_cap); tmem_st4(tP + (c0 + cs) * 4, packed);
        tmem_ld_fence(ra); tmem_ld16_issue(tS + (c0 + 3 * cs) * 16, rb);
        chunk_exp_pack<false, 16, kPolicy>(ra, 0u, k.c2, k.neg_hi, k.p_mul_f, sum, packed, p_cap); tmem_st4(tP + (c0 + 2 * cs) * 4, packed);
        tmem_ld_fence(rb);
        chunk_exp_pack<false, 16, kPolicy>(rb, 0u, k.c2, k.neg_hi, k.p_mul_f, sum, packed, p_cap); tmem_st4(tP + (c0 + 3 * cs) * 4, packed);
      } else {
        tmem_ld_fence(ra);
#pragma unroll 1
        for (int i = 0; i < 4; ++i) {
          const int c = c0 + i * cs;
          if (i > 0) { tmem_ld16_issue(tS + c * 16, ra); tmem_ld_fence(ra); }
          chunk_exp_pack<true, 16, kPolicy>(ra, (mwords[c >> 1] >> ((c & 1) * 16)) & 0xFFFFu, k.c2, k.neg_hi, k.p_mul_f, sum, packed, p_cap);
          tmem_st4(tP + c * 4, packed);
        }
      }
      // ---- publish the row statistics of this step for the merge threads
      const int slot = static_cast<int>(g & 3u);
      const float part = (sum[0].x + sum[0].y) + (sum[1].x + sum[1].y);
      if (half == 0) {
        ctl->st_m[slot][row] = k.m_tile;
        ctl->st_f[slot][row] = k.f;
        ctl->st_s0[slot][row] = part;
      } else {
        ctl->st_s1[slot][row] = part;
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(smem_u32(&ctl->p_ready[slot]));
      if (half == 0 && quad == 0) FMHA_STAMP(chain * 4 + 2, n);
      FMHA_STAMP(16 + warp, n);
    }
    g0 += static_cast<uint32_t>(n_live);
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&ctl->info_empty[buf]));     // this warp is done with the unit's mask information
  }
}

// ---------------------------------------------------------------------------------------------- merge role
// One thread = one half (D/2 columns) of the fp32 running output row of one query row, plus the running
// maximum and the running sum of that row (kept by both threads of the row).
template <int D, bool kPolicy>
__device__ __forceinline__ void merge_role(const FwdParams& p, FwdCtl<FwdCfg<D>::kStagesK, FwdCfg<D>::kStagesV>* ctl, const uint32_t tmem_base,
                                           const int first_unit, const int unit_step) {
  constexpr int DH = D / 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad = warp & 3, ch = (warp - kWarpMerge0) >> 2;       // ch = which half of the output columns
  const int row = quad * 32 + lane;
  const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
  volatile int* abort_flag = &ctl->abort;

  uint32_t g0 = 0;
  int it = 0;
  for (int u = first_unit; u < p.n_units; u += unit_step, ++it) {
    const int buf = it % kInfoBufs;
    if (!__all_sync(0xFFFFFFFFu, mbar_wait_slow(smem_u32(&ctl->info_full[buf]), static_cast<uint32_t>((it / kInfoBufs) & 1), abort_flag))) {
      raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_INFO, it);
      return;
    }
    const int n_live = ctl->info[buf].n_live;
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&ctl->info_empty[buf]));     // only the tile count is needed here
    const UnitGeom geo = unit_geom(p, u);
    const int q_row = geo.q_row0 + row;

    float2 o2[DH / 2];
#pragma unroll
    for (int i = 0; i < DH / 2; ++i) o2[i] = make_float2(0.f, 0.f);
    float m_run = -INFINITY, l_run = 0.f;
    int imax_run = INT_MIN;                                 // statistics launch: biased integer row maximum over all tiles
    const bool stats_only = !kPolicy && p.row_stats_out != nullptr;

#pragma unroll 1
    for (int j = 0; j < n_live; ++j) {
      const uint32_t g = g0 + static_cast<uint32_t>(j);
      const int slot = static_cast<int>(g & 3u);
      const uint32_t sb = g % SBufs<D>::n;
      if (!__all_sync(0xFFFFFFFFu, mbar_wait_slow(smem_u32(&ctl->p_ready[slot]), (g >> 2) & 1u, abort_flag))) {
        raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_P_READY, g);
        return;
      }
      // ---- merge of tile statistics (inc/fmha_i8.cuh:301-304)
      float e_old = 1.f, e_cur = 1.f;                                  // policy launch: every tile of a row has the same scale
      if (!kPolicy) {
        const float m_tile = ctl->st_m[slot][row];
        const float l_tile = ctl->st_f[slot][row] * (ctl->st_s0[slot][row] + ctl->st_s1[slot][row]);
        const float m_new = fmaxf(m_run, m_tile);
        e_old = __expf(m_run - m_new);                                 // 0 on the first tile (m_run = -inf)
        e_cur = clear_low2(__expf(m_tile - m_new));                    // 22 significant bits: kMagic*e_cur is exact
        l_run = fmaf(e_old, l_run, e_cur * l_tile);
        m_run = m_new;
        imax_run = max(imax_run, ctl->st_i[slot][row]);
      }
      const float es = p.o_sign * e_cur;                               // the accumulator holds o_sign * (P.V)
      const float2 neg_ec = make_float2(es, es), e_bias = make_float2(-es * kMagic, -es * kMagic);
      const float2 e_old2 = make_float2(e_old, e_old);

      // ---- drain my half of O~ = bias -/+ (P8 . V) into the fp32 running row.  The partial output of step g lives in
      //      the accumulator S(g) came from: all of it at head_dim 128, columns [16,80) at head_dim 64.
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&ctl->o_full[sb]), (g / SBufs<D>::n) & 1u, abort_flag))) {
        raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_O_READY, g);
        return;
      }
      tc_fence_after();
      if (quad == 0) FMHA_STAMP(8 + 2 * ch, g);
      if (!stats_only) {
        // output column c of this step: tensor-memory column of 16-column chunk i of MY half
        auto chunk_col = [&](int i) -> uint32_t { return t_lane + sb * kTile + PLayout<D>::kOOff + ch * DH + i * 16; };
        // two loads in flight at a time: a round trip to tensor memory costs more than folding a chunk in
        uint32_t ra[16], rb[16];
        tmem_ld16_issue(chunk_col(0), ra);
        tmem_ld16_issue(chunk_col(1), rb);
#pragma unroll
        for (int c = 0; c < DH / 16; c += 2) {
          tmem_ld_fence(ra); tmem_ld_fence(rb);
          if (c + 2 >= DH / 16) {
            // the last two chunks are in registers: the accumulator can go back to the S issuer before they are folded in
            tc_fence_before();
            mbar_arrive(smem_u32(&ctl->s_free[sb]));
          }
          drain_chunk<16>(ra, o2 + c * 8, neg_ec, e_bias, e_old2);
          if (c + 2 < DH / 16) tmem_ld16_issue(chunk_col(c + 2), ra);
          drain_chunk<16>(rb, o2 + (c + 1) * 8, neg_ec, e_bias, e_old2);
          if (c + 3 < DH / 16) tmem_ld16_issue(chunk_col(c + 3), rb);
        }
      } else {
        tc_fence_before();
        mbar_arrive(smem_u32(&ctl->s_free[sb]));
      }
      if (quad == 0) FMHA_STAMP(9 + 2 * ch, g);
    }
    g0 += static_cast<uint32_t>(n_live);

    // ---- statistics launch: the row's maximum and exp-sum over all keys, for the policy launch that follows
    if (stats_only) {
      if (ch == 0 && q_row < p.Sq)
        p.row_stats_out[static_cast<int64_t>(geo.bh_local) * p.Sq + q_row] =
            make_float2(__int_as_float(n_live > 0 ? imax_run : static_cast<int>(kMagicBits)), n_live > 0 ? l_run : 0.f);
      continue;
    }
    if (kPolicy) {
      // the accumulated integer sum becomes the output through one factor per row: out_mul (/ l for the per-row policy)
      float l_row = 0.f;
      if (q_row < p.Sq) l_row = __ldg(&p.row_stats_in[static_cast<int64_t>(geo.bh_local) * p.Sq + q_row]).y;
      l_run = (p.p_static_mul != 0.f) ? (l_row > 0.f ? 1.f : 0.f) : l_row;
    }

    // ---- calibration mode: only the largest magnitude of the unquantised output is wanted (the reference
    //      takes o_amax from its fp32 CPU result, test_fmha_i8.cpp:161)
    if (p.amax_out != nullptr) {
      float mx = 0.f;
      if (q_row < p.Sq && n_live > 0 && l_run > 0.f) {
        const float inv = 1.0f / l_run;
#pragma unroll
        for (int i = 0; i < DH / 2; ++i) mx = fmaxf(mx, fmaxf(fabsf(o2[i].x * inv), fabsf(o2[i].y * inv)));
      }
      // non-negative floats order like their bit patterns
      const unsigned bits = __reduce_max_sync(0xFFFFFFFFu, __float_as_uint(mx * p.amax_scale));
      if (lane == 0 && bits != 0u) atomicMax(reinterpret_cast<unsigned*>(p.amax_out), bits);
      continue;
    }

    // ---- epilogue (inc/fmha_i8.cuh:318-332): normalise, requantise, store
    if (q_row < p.Sq) {
      const float inv = (n_live > 0 && l_run > 0.f) ? 1.0f / l_run : 0.f;
      int8_t* dst = p.o + (static_cast<int64_t>(geo.bh_local) * p.Sq + q_row) * D + ch * DH;
      // rn(clamp(x)) through the magic-number addition (the low byte of clamp(x) + 1.5*2^23 is the two's-complement
      // integer), bytes gathered with PRMT: conversions and shifts would cost three times the issue cycles
      const float2 inv2 = make_float2(inv, inv), sc2 = make_float2(p.scale_v_out, p.scale_v_out);
      const float2 zero2 = make_float2(0.f, 0.f), magic2 = make_float2(kMagic, kMagic);
      uint32_t wide[8];
#pragma unroll
      for (int c = 0; c < DH / 16; ++c) {
        uint32_t* wds = &wide[(c & 1) * 4];
#pragma unroll
        for (int gq = 0; gq < 4; ++gq) {
          float2 a = __ffma2_rn(sc2, __ffma2_rn(o2[c * 8 + gq * 2], inv2, zero2), zero2);        // scale_v_out * (o * inv), each product rounded
          float2 b = __ffma2_rn(sc2, __ffma2_rn(o2[c * 8 + gq * 2 + 1], inv2, zero2), zero2);
          a.x = fminf(fmaxf(a.x, -127.f), 127.f); a.y = fminf(fmaxf(a.y, -127.f), 127.f);
          b.x = fminf(fmaxf(b.x, -127.f), 127.f); b.y = fminf(fmaxf(b.y, -127.f), 127.f);
          const float2 ya = __fadd2_rn(a, magic2), yb = __fadd2_rn(b, magic2);
          wds[gq] = __byte_perm(__byte_perm(__float_as_uint(ya.x), __float_as_uint(ya.y), 0x0040),
                                __byte_perm(__float_as_uint(yb.x), __float_as_uint(yb.y), 0x0040), 0x5410);
        }
        // 32-byte stores: a warp's rows are 128 (or 64) bytes apart, so every store touches 32 lines whatever its
        // width, and the 16-byte version of this loop cost 5 % of the whole kernel at head_dim 128
        if (c & 1) {
          if (p.o_wide) {
            st_global_v8(dst + (c - 1) * 16, wide);
          } else {
            *reinterpret_cast<uint4*>(dst + (c - 1) * 16) = make_uint4(wide[0], wide[1], wide[2], wide[3]);
            *reinterpret_cast<uint4*>(dst + c * 16) = make_uint4(wide[4], wide[5], wide[6], wide[7]);
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------- loader
// One warp, run warp-wide (every lane waits and counts, one elected lane issues the copies): the Q tile of every
// non-empty unit, then per step the K tile and the V tile, in step order.
template <int D>
__device__ __forceinline__ void loader_role(const FwdParams& p, FwdCtl<FwdCfg<D>::kStagesK, FwdCfg<D>::kStagesV>* ctl,
                                            const CUtensorMap* map_q, const CUtensorMap* map_k, const CUtensorMap* map_v,
                                            const uint32_t q_smem, const uint32_t k_smem, const uint32_t v_smem,
                                            const int first_unit, const int unit_step) {
  using Cfg = FwdCfg<D>;
  constexpr uint32_t NK = Cfg::kStagesK, NV = Cfg::kStagesV, NQ = Cfg::kQBufs;
  volatile int* abort_flag = &ctl->abort;
  uint32_t g = 0;            // steps loaded so far: ring position and phase continue across units
  uint32_t qn = 0;           // non-empty units so far: Q buffer and phase
  uint32_t fail = 0u, fail_tile = 0u;
  int it = 0;
  for (int u = first_unit; u < p.n_units && fail == 0u; u += unit_step, ++it) {
    const int buf = it % kInfoBufs;
    if (!__all_sync(0xFFFFFFFFu, mbar_wait_slow(smem_u32(&ctl->info_full[buf]), static_cast<uint32_t>((it / kInfoBufs) & 1), abort_flag))) {
      fail = FMHA_I8_DEV_WAIT_INFO; fail_tile = it; break;
    }
    const UnitGeom geo = unit_geom(p, u);
    const UnitInfo* info = &ctl->info[buf];
    const int n_live = info->n_live;
    if (n_live > 0) {
      const uint32_t qb = qn % NQ;
      // the Q buffer is free once the last S = Q.K^T of the unit that used it NQ units ago has completed
      if (qn >= NQ && !__all_sync(0xFFFFFFFFu, mbar_wait_slow(smem_u32(&ctl->q_empty[qb]), ((qn / NQ) - 1) & 1u, abort_flag))) {
        fail = FMHA_I8_DEV_WAIT_K_FREE; fail_tile = it; break;
      }
      if (elect_one()) {
        const uint32_t bar_q = smem_u32(&ctl->q_full[qb]);
        mbar_arrive_expect_tx(bar_q, static_cast<uint32_t>(Cfg::kTileBytes));
        tma_load_3d(q_smem + qb * Cfg::kTileBytes, map_q, bar_q, 0, geo.q_row0, geo.bh_local);
      }
      ++qn;
      for (int j = 0; j < n_live; ++j, ++g) {
        const int t = info->live[j];
        const uint32_t sk = g % NK, rk = g / NK, sv = g % NV, rv = g / NV;
        if (rk > 0 && !__all_sync(0xFFFFFFFFu, mbar_wait_slow(smem_u32(&ctl->k_empty[sk]), (rk - 1) & 1u, abort_flag))) {
          fail = FMHA_I8_DEV_WAIT_K_FREE; fail_tile = g; break;
        }
        if (elect_one()) {
          mbar_arrive_expect_tx(smem_u32(&ctl->k_full[sk]), Cfg::kTileBytes);
          tma_load_3d(k_smem + sk * Cfg::kTileBytes, map_k, smem_u32(&ctl->k_full[sk]), 0, t * kTile, geo.bh_local);
        }
        if (rv > 0 && !__all_sync(0xFFFFFFFFu, mbar_wait_slow(smem_u32(&ctl->v_empty[sv]), (rv - 1) & 1u, abort_flag))) {
          fail = FMHA_I8_DEV_WAIT_V_FREE; fail_tile = g; break;
        }
        if (elect_one()) {
          mbar_arrive_expect_tx(smem_u32(&ctl->v_full[sv]), Cfg::kTileBytes);
          tma_load_3d(v_smem + sv * Cfg::kTileBytes, map_v, smem_u32(&ctl->v_full[sv]), 0, t * kTile, geo.bh_local);
        }
      }
    }
    __syncwarp();
    if (fail == 0u && elect_one()) mbar_arrive(smem_u32(&ctl->info_empty[buf]));
  }
  if (fail != 0u) {
    if (elect_one()) raise_status(abort_flag, p.status, fail, fail_tile);
    // unwinding: let copies that are still in flight land before the CTA may exit
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { /* about a millisecond */ }
  }
}

// ---------------------------------------------------------------------------------------------- MMA issuers
// Two warps issue tcgen05.mma: one the S = Q.K^T products, the other the P.V products.  Each runs warp-wide (every
// lane waits and counts, one elected lane issues) and walks the CTA's step sequence on its own; what orders them is the s_free barrier (S(g) may overwrite an accumulator only after
// the P.V that read the P bytes in it has completed) and, through the softmax warps, s_full -> p_ready.
// A wait that gives up only notes which one it was; the status is raised once, after the loop.
struct IssuerErr {
  uint32_t code = 0u, tile = 0u;
};
template <bool kSlow = false>
__device__ __forceinline__ bool issuer_wait(IssuerErr& e, uint32_t bar, uint32_t parity, uint32_t code, uint32_t tile, const volatile int* abort_flag) {
  if (__all_sync(0xFFFFFFFFu, kSlow ? mbar_wait_slow(bar, parity, abort_flag) : mbar_wait(bar, parity, abort_flag))) return true;
  e.code = code;
  e.tile = tile;
  return false;
}

template <int D>
__device__ __forceinline__ void s_issuer_role(const FwdParams& p, FwdCtl<FwdCfg<D>::kStagesK, FwdCfg<D>::kStagesV>* ctl, const uint32_t tmem_base,
                                              const uint32_t q_smem, const uint32_t k_smem, const uint32_t bias_a_smem, const uint32_t bias_b_smem,
                                              const int first_unit, const int unit_step) {
  using Cfg = FwdCfg<D>;
  constexpr uint32_t NK = Cfg::kStagesK, NQ = Cfg::kQBufs;
  volatile int* abort_flag = &ctl->abort;
  constexpr uint32_t idesc_s = make_idesc_i8(kTile, false);   // S = Q.K^T : N = 128 keys, both K-major
  constexpr uint32_t idesc_bias_s = make_idesc_f16(kTile);
  const uint64_t d_bias_a = make_smem_desc_noswizzle(bias_a_smem, 128, 256);
  const uint64_t d_bias_b = make_smem_desc_noswizzle(bias_b_smem, 128, 256);
  IssuerErr err;
  uint32_t g = 0, qn = 0;
  int it = 0;
  bool ok = true;
  for (int u = first_unit; u < p.n_units && ok; u += unit_step, ++it) {
    const int buf = it % kInfoBufs;
    if (!issuer_wait<true>(err, smem_u32(&ctl->info_full[buf]), static_cast<uint32_t>((it / kInfoBufs) & 1), FMHA_I8_DEV_WAIT_INFO, it, abort_flag)) break;
    const int n_live = ctl->info[buf].n_live;
    __syncwarp();
    if (elect_one()) mbar_arrive(smem_u32(&ctl->info_empty[buf]));            // only the tile count is needed here
    if (n_live == 0) continue;
    const uint32_t qb = qn % NQ;
    if (!issuer_wait<true>(err, smem_u32(&ctl->q_full[qb]), (qn / NQ) & 1u, FMHA_I8_DEV_WAIT_Q_LOAD, g, abort_flag)) break;
    const uint64_t dq = make_smem_desc(q_smem + qb * Cfg::kTileBytes, D);
    for (int j = 0; j < n_live; ++j, ++g) {
      const uint32_t sb = g % SBufs<D>::n, stage = g % NK;
      const uint64_t dk = make_smem_desc(k_smem + stage * Cfg::kTileBytes, D);
      const uint32_t tS = tmem_base + sb * kTile;
      // K first (it has normally been there for a while), then the accumulator: it still holds the partial output of
      // step g - n until the merge warps have drained it, and that hand-off is on the step-to-step critical path
      if (!issuer_wait<true>(err, smem_u32(&ctl->k_full[stage]), (g / NK) & 1u, FMHA_I8_DEV_WAIT_K_LOAD, g, abort_flag)) { ok = false; break; }
      if (g >= SBufs<D>::n && !issuer_wait(err, smem_u32(&ctl->s_free[sb]), ((g / SBufs<D>::n) - 1) & 1u, FMHA_I8_DEV_WAIT_O_FREE, g, abort_flag)) { ok = false; break; }
      FMHA_STAMP(15, g);
      tc_fence_after();
      if (elect_one()) {
        mma_f16_ss(tS, d_bias_a, d_bias_b, idesc_bias_s, 0u);      // accumulator := 0x4B400000
#pragma unroll
        for (int kk = 0; kk < D / 32; ++kk)
          mma_i8_ss(tS, desc_advance(dq, kk * 32), desc_advance(dk, kk * 32), idesc_s, 1u);
        mma_commit(smem_u32(&ctl->s_full[sb]));
        mma_commit(smem_u32(&ctl->k_empty[stage]));
        if (j == n_live - 1) mma_commit(smem_u32(&ctl->q_empty[qb]));                   // that was the unit's last use of its Q rows
      }
      FMHA_STAMP(12, g);
    }
    if (!ok) break;
    ++qn;
  }
  if (err.code != 0u && elect_one()) raise_status(abort_flag, p.status, err.code, err.tile);
}

template <int D>
__device__ __forceinline__ void o_issuer_role(const FwdParams& p, FwdCtl<FwdCfg<D>::kStagesK, FwdCfg<D>::kStagesV>* ctl, const uint32_t tmem_base,
                                              const uint32_t v_smem, const uint32_t bias_a_smem, const uint32_t bias_b_smem,
                                              const int first_unit, const int unit_step) {
  using Cfg = FwdCfg<D>;
  constexpr uint32_t NV = Cfg::kStagesV;
  volatile int* abort_flag = &ctl->abort;
  // O = P.V : V is an MN-major operand; one group of MMAs with N = head_dim output columns
  const uint32_t idesc_o = p.p_unsigned ? make_idesc_i8(D, true, true) : make_idesc_i8(D, true, false);
#if FMHA_PV_BIAS_MMA
  constexpr uint32_t idesc_bias = make_idesc_f16(D);
  const uint64_t d_bias_a = make_smem_desc_noswizzle(bias_a_smem, 128, 256);
  const uint64_t d_bias_b = make_smem_desc_noswizzle(bias_b_smem, 128, 256);
#endif
  IssuerErr err;
  uint32_t g = 0;
  int it = 0;
  bool ok = true;
  for (int u = first_unit; u < p.n_units && ok; u += unit_step, ++it) {
    const int buf = it % kInfoBufs;
    if (!issuer_wait<true>(err, smem_u32(&ctl->info_full[buf]), static_cast<uint32_t>((it / kInfoBufs) & 1), FMHA_I8_DEV_WAIT_INFO, it, abort_flag)) break;
    const int n_live = ctl->info[buf].n_live;
    __syncwarp();
    if (elect_one()) mbar_arrive(smem_u32(&ctl->info_empty[buf]));            // only the tile count is needed here
    for (int j = 0; j < n_live; ++j, ++g) {
      const uint32_t sb = g % SBufs<D>::n, stage = g % NV;
      const uint64_t dv = make_smem_desc(v_smem + stage * Cfg::kTileBytes, D);
      const uint32_t tS = tmem_base + sb * kTile;
      const uint32_t tP = PLayout<D>::kAnnex ? tmem_base + SBufs<D>::n * kTile + sb * PLayout<D>::kAnnexCols : tS;
      const uint32_t tO = tS + PLayout<D>::kOOff;
      // V first (loaded steps ago), then P: the MMAs go out as soon as the last softmax warp has arrived
      if (!issuer_wait<true>(err, smem_u32(&ctl->v_full[stage]), (g / NV) & 1u, FMHA_I8_DEV_WAIT_V_LOAD, g, abort_flag)) { ok = false; break; }
      if (!issuer_wait(err, smem_u32(&ctl->p_ready[g & 3u]), (g >> 2) & 1u, FMHA_I8_DEV_WAIT_P_READY, g, abort_flag)) { ok = false; break; }
      FMHA_STAMP(13, g);
      tc_fence_after();
      // The accumulator of this step is S(g)'s own buffer (free since the softmax threads have read S(g)), minus the
      // columns that hold P bytes at head_dim 64.
      if (elect_one()) {
#if FMHA_PV_BIAS_MMA
        mma_f16_ss(tO, d_bias_a, d_bias_b, idesc_bias, 0u);      // accumulator := 0x4B400000
#endif
#pragma unroll
        for (int kk = 0; kk < kTile / 32; ++kk)
          mma_i8_ts(tO, tP + PLayout<D>::p_col(kk), desc_advance(dv, kk * 32 * D), idesc_o, (FMHA_PV_BIAS_MMA || kk > 0) ? 1u : 0u);
        mma_commit(smem_u32(&ctl->o_full[sb]));
        mma_commit(smem_u32(&ctl->v_empty[stage]));
      }
      FMHA_STAMP(14, g);
    }
  }
  if (err.code != 0u && elect_one()) raise_status(abort_flag, p.status, err.code, err.tile);
}

// Persistent kernel: gridDim.x = min(units, SMs) CTAs; CTA b processes units b, b + gridDim.x, ...
// kPolicy: the launch that applies a whole-row P scaling policy from row statistics (see FwdParams::row_stats_in);
// the product default, and the statistics launch, are kPolicy = false.
template <int D, bool kPolicy>
__global__ void __launch_bounds__(kFwdThreads, 1)
fmha_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const FwdParams p) {
  using Cfg = FwdCfg<D>;
  constexpr int NK = Cfg::kStagesK, NV = Cfg::kStagesV, NQ = Cfg::kQBufs;
  using Ctl = FwdCtl<NK, NV>;
  extern __shared__ uint8_t smem_raw[];
  // tiles need 1024-byte alignment (swizzle atoms); the launch reserves the slack
  // (pointer arithmetic on the shared array, not a round trip through an integer: the compiler then knows that everything
  // derived from it is shared memory and uses 32-bit shared-space loads and stores instead of generic ones)
  uint8_t* tiles = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* bias_a = tiles + Cfg::kTilesBytesTotal;
  uint8_t* bias_b = bias_a + kBiasBytes;
  Ctl* ctl = reinterpret_cast<Ctl*>(bias_b + kBiasBytes);
  const uint32_t q_smem = smem_u32(tiles);
  const uint32_t k_smem = q_smem + NQ * Cfg::kTileBytes;
  const uint32_t v_smem = k_smem + NK * Cfg::kTileBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (p.S + kTile - 1) / kTile;
  const int first_unit = blockIdx.x, unit_step = gridDim.x;

  if (threadIdx.x == 0) {
    ctl->abort = 0;
    for (int w = 0; w < NQ; ++w) {
      mbar_init(smem_u32(&ctl->q_full[w]), 1);
      mbar_init(smem_u32(&ctl->q_empty[w]), 1);
    }
    for (int w = 0; w < 2; ++w)
      for (int q = 0; q < 4; ++q) mbar_init(smem_u32(&ctl->xch[w][q]), 64);
    for (int s = 0; s < SBufs<D>::n; ++s) {
      mbar_init(smem_u32(&ctl->s_full[s]), 1);
      mbar_init(smem_u32(&ctl->o_full[s]), 1);
      mbar_init(smem_u32(&ctl->s_free[s]), kMergeWarps * 32);
    }
    for (int s = 0; s < NK; ++s) {
      mbar_init(smem_u32(&ctl->k_full[s]), 1);
      mbar_init(smem_u32(&ctl->k_empty[s]), 1);
    }
    for (int s = 0; s < NV; ++s) {
      mbar_init(smem_u32(&ctl->v_full[s]), 1);
      mbar_init(smem_u32(&ctl->v_empty[s]), 1);
    }
    for (int s = 0; s < 4; ++s) mbar_init(smem_u32(&ctl->p_ready[s]), 8 * 32);
    for (int b = 0; b < kInfoBufs; ++b) {
      mbar_init(smem_u32(&ctl->info_full[b]), 1);
      mbar_init(smem_u32(&ctl->info_empty[b]), kInfoConsumers);
    }
    mbar_init_fence();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  fill_bias_operands(bias_a, bias_b);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);
  volatile int* abort_flag = &ctl->abort;

  // Every role walks the same unit sequence: `it` counts this CTA's units, info buffer = it % kInfoBufs,
  // phase of an info barrier = (it / kInfoBufs) & 1; `g` counts its steps (live key tiles) across units.
  if (warp >= kWarpSoftmax0) {
    setmaxnreg_dec<FwdRegs<D>::kSoftmax>();
    softmax_role<D, kPolicy>(p, ctl, tmem_base, first_unit, unit_step);
  } else if (warp >= kWarpMerge0) {
    setmaxnreg_inc<FwdRegs<D>::kMerge>();
    merge_role<D, kPolicy>(p, ctl, tmem_base, first_unit, unit_step);
  } else {
    if (FwdRegs<D>::kOther < kLaunchRegs) setmaxnreg_dec<FwdRegs<D>::kOther>();
    else if (FwdRegs<D>::kOther > kLaunchRegs) setmaxnreg_inc<FwdRegs<D>::kOther>();
    if (warp == kWarpLoad) {
      loader_role<D>(p, ctl, &map_q, &map_k, &map_v, q_smem, k_smem, v_smem, first_unit, unit_step);
    } else if (warp == kWarpMmaS) {
      s_issuer_role<D>(p, ctl, tmem_base, q_smem, k_smem, smem_u32(bias_a), smem_u32(bias_b), first_unit, unit_step);
    } else if (warp == kWarpMmaO) {
      o_issuer_role<D>(p, ctl, tmem_base, v_smem, smem_u32(bias_a), smem_u32(bias_b), first_unit, unit_step);
    } else if (warp == kWarpScan) {
      // ---------------------------------------------------------------- scanner: mask information, units ahead
      bool ok = true;
      int it = 0;
      for (int u = first_unit; u < p.n_units && ok; u += unit_step, ++it) {
        const int buf = it % kInfoBufs;
        // the buffer was used by unit it - kInfoBufs: wait until all its consumers have released it
        if (it >= kInfoBufs) {
          ok = __all_sync(0xFFFFFFFFu, mbar_wait_slow(smem_u32(&ctl->info_empty[buf]), static_cast<uint32_t>(((it / kInfoBufs) - 1) & 1), abort_flag));
          if (!ok) { if (lane == 0) raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_INFO, it); break; }
        }
        const UnitGeom geo = unit_geom(p, u);
        scan_mask_warp(&ctl->info[buf], p.mask + static_cast<int64_t>(geo.batch) * p.S, p.S, n_tiles);
        if (lane == 0) mbar_arrive(smem_u32(&ctl->info_full[buf]));
      }
    }
  }

  // every unit of this CTA has been computed and stored by the time the merge warps leave their loop
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace fmha
