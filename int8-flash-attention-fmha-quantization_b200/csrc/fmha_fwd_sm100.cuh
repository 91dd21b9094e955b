// The INT8 flash-attention forward kernel for sm_100a.
//
// Replaces the reference project's FMHAInferKernel (inc/fmha_i8.cuh:43-334).  Same arithmetic
// contract -- key tiles of 128 starting at key 0, P quantised to 8 bits against each tile's own row
// maximum, tiles merged in fp32 -- on a different machine model:
//
//   work unit  = (batch*head, pair of 128-row query tiles).  The kernel is persistent: min(units, SMs)
//                CTAs, one per SM, CTA c walks units c, c + grid, ...; barrier phases, the K/V ring and
//                tensor memory carry on from one unit to the next.
//   warp 8     = loader: TMA brings Q (once per unit) and a ring of K and V tiles into swizzled shared
//                memory, running ahead into the next unit
//   warp 9     = MMA issuer: one thread issues tcgen05.mma
//                  S_w   = bias + Q_w . K_j^T   (smem x smem  -> int32 in tensor memory)
//                  O~_w  = bias + P_w . V_j     (tmem x smem  -> int32 in tensor memory)
//   warp 10    = scanner: turns the next unit's padding-mask row into per-tile bit masks and the list
//                of key tiles that hold at least one unmasked key (double-buffered)
//   warps 0-3  = softmax group of query tile 0, warps 4-7 = of query tile 1: one thread owns one
//                query row, so row max / row sum need no shuffles.  Per key tile a thread reads its S
//                row from tensor memory twice (integer max, then exp + requantise), writes the 8-bit P
//                row back over the front of S, and after P.V drains the partial output into its fp32
//                running row.
//   warp 11    idle (it completes the third warpgroup so registers can be moved to the softmax groups
//                with setmaxnreg).
//
// The bias: every accumulator is first written by a one-step fp16 MMA whose operands hold 4096 and
// 3072, i.e. the fp32 value 1.5*2^23 (bits 0x4B400000); the int8 MMAs then add their integer result
// to that bit pattern.  Read back as a float the accumulator is exactly 1.5*2^23 + s, so the
// softmax threads never convert integers to floats: one fused multiply-add turns the raw
// accumulator into the exponent argument (or into the rescaled partial output).
//
// Tensor memory (512 columns x 128 lanes x 32 bit): S_0 [0,128) S_1 [128,256) O~_0 [256,256+D)
// O~_1 [256+D,256+2D).  P_w occupies the first 32 columns of S_w (four int8 per column).
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

namespace fmha {

// Optional timeline tracing for performance work: with -DFMHA_TRACE the first CTA records clock64()
// stamps of its phase boundaries.  Compiled out of the product build.
#ifndef FMHA_TRACE_Q
#define FMHA_TRACE_Q 0
#endif
#ifdef FMHA_TRACE
__device__ long long g_trace[16][512];
#define FMHA_STAMP(slot, idx) do { if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && (idx) < 512) g_trace[slot][idx] = clock64(); } while (0)
#else
#define FMHA_STAMP(slot, idx) do { } while (0)
#endif

constexpr int kTile = 128;           // query rows per tile == keys per tile
constexpr int kMaxSeq = 32768;
constexpr int kMaxTiles = kMaxSeq / kTile;
constexpr int kFwdThreads = 384;     // three warpgroups
constexpr int kWarpLoad = 8;
constexpr int kWarpMma = 9;
constexpr int kWarpScan = 10;         // prepares the next unit's mask information
// setmaxnreg moves registers inside the CTA's own launch allocation (registers per thread at launch x
// threads), not inside the SM's whole register file: a request that does not fit blocks forever.  With
// 384 threads the compiler's launch allocation is 168 registers per thread (the host checks this before
// the first launch and refuses otherwise).  head_dim 128: 8 warps x 208 + 4 warps x 88 = 12 x 168 (the
// softmax warps hold a 128-register output row; the MMA issuer needs more than the 56 a 224/56 split would
// leave it).  head_dim 64: nobody needs more than 168, so nothing is moved (measured: C5 +5 % against 208/88).
constexpr int kLaunchRegs = 168;
template <int D> struct FwdRegs {
  static constexpr int kSoftmax = (D == 128) ? 208 : kLaunchRegs;
  static constexpr int kOther = (D == 128) ? 88 : kLaunchRegs;
  static_assert(8 * kSoftmax + 4 * kOther <= (kFwdThreads / 32) * kLaunchRegs,
                "setmaxnreg targets exceed the CTA's register allocation: the kernel would hang");
  static_assert(kSoftmax >= kLaunchRegs && kOther <= kLaunchRegs, "softmax warps only gain, the others only give");
};
constexpr uint32_t kTmemCols = 512;
constexpr float kMagic = 12582912.0f;          // 1.5 * 2^23: float whose ulp is 1 over [2^23, 2^24)
constexpr uint32_t kMagicBits = 0x4B400000u;
constexpr int kBiasBytes = 4096;               // 128 rows x 16 fp16, unswizzled core-matrix layout

template <int D> struct FwdCfg {
  static_assert(D == 64 || D == 128, "head_dim must be 64 or 128");
  // Ring depth of K and of V.  Three stages are measured to be better than four, five or six: a deeper ring
  // buys nothing (the loader is tiles ahead anyway) and its shared memory comes out of the L1 that serves
  // the MMA issuer's and the softmax warps' few spilled registers.
  static constexpr int kStages = 3;
  static constexpr int kTileBytes = kTile * D;              // one 128-row tile of int8
  static constexpr int kTilesBytesTotal = (2 + 2 * kStages) * kTileBytes;
};

struct FwdParams {
  const int8_t* mask;   // [B,S] whole mask
  int8_t* o;            // first head of the slice
  int S;                // keys per head (seq_len; seq_len_k when queries and keys differ in number)
  int Sq;               // query rows per head (== S for self-attention)
  int H, bh_begin, bh_count, q_pairs;
  int n_units;          // bh_count * q_pairs work units, taken round-robin by the resident CTAs
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
};

// What every role needs to know about one work unit's padding mask.  Two of these live in shared
// memory: the scanner warp fills the one of the NEXT unit while the current unit is being processed.
struct UnitInfo {
  int n_live;                         // key tiles with at least one unmasked key
  uint32_t maskbits[kMaxTiles * 4];   // bit set = key masked (or beyond seq_len)
  uint16_t live[kMaxTiles];           // indices of the live key tiles, ascending
  uint8_t mixed[kMaxTiles];           // 1 = that live tile has masked keys too
};
constexpr int kInfoConsumers = 10;    // loader, MMA issuer and the eight softmax warps each release an info buffer once

template <int NS> struct FwdCtl {
  uint64_t q_full[2], q_empty[2];      // per query tile: its Q rows have landed / its last S = Q.K^T of the unit has completed
  uint64_t k_full[NS], k_empty[NS], v_full[NS], v_empty[NS];
  uint64_t s_full[2], p_ready[2], o_full[2], o_free[2];
  uint64_t info_full[2], info_empty[2];
  uint32_t tmem_base;
  int abort;
  UnitInfo info[2];
};

__device__ __noinline__ void raise_status(volatile int* abort_flag, unsigned* status, unsigned code, unsigned tile) {
  *abort_flag = 1;
  if (atomicCAS(&status[0], 0u, code) == 0u) {
    status[1] = blockIdx.x;
    status[2] = threadIdx.x >> 5;
    status[3] = tile;
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

struct TileStats {
  float m_tile;   // row maximum of the scaled scores of this tile (the reference's thread_max)
  float l_tile;   // row sum of exp(score - m_tile) (the reference's thread_sum)
};

// Row maximum over N raw accumulator words (biased integers compare like the integers themselves).
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

// N scores -> N probabilities (summed into four independent packed accumulators) -> N/4 words of
// packed signed bytes holding -rn(128 p).  x = raw accumulator read as float = kMagic + s.
template <bool kMixed, int N>
__device__ __forceinline__ void chunk_exp_pack(const uint32_t (&r)[N], uint32_t mw, const float2 c2, const float2 neg_hi,
                                               const float2 neg_128f, float2 (&sum)[4], uint32_t (&packed)[N / 4]) {
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
    const float2 p01 = make_float2(ex2_approx(a01.x), ex2_approx(a01.y));
    const float2 p23 = make_float2(ex2_approx(a23.x), ex2_approx(a23.y));
    sum[(2 * g) & 3] = __fadd2_rn(sum[(2 * g) & 3], p01);
    sum[(2 * g + 1) & 3] = __fadd2_rn(sum[(2 * g + 1) & 3], p23);
    const float2 y01 = __ffma2_rn(p01, neg_128f, magic2);      // low byte = two's complement of -P8
    const float2 y23 = __ffma2_rn(p23, neg_128f, magic2);
    packed[g] = __byte_perm(__byte_perm(__float_as_uint(y01.x), __float_as_uint(y01.y), 0x0040),
                            __byte_perm(__float_as_uint(y23.x), __float_as_uint(y23.y), 0x0040), 0x5410);
  }
}

// The same work split in two stages so that the exponentials of the next chunk (XU pipe, one warp
// instruction per 8 cycles) are interleaved IN PROGRAM ORDER with the packing of the current chunk
// (FMA/ALU pipes): a warp issues in order, so a run of back-to-back MUFUs would leave the other
// pipes idle.  chunk_exp alone is used for the first chunk, chunk_pack alone for the last.
template <int N>
__device__ __forceinline__ void chunk_exp(const uint32_t (&r)[N], const float2 c2, const float2 neg_hi, float2 (&pr)[N / 2]) {
#pragma unroll
  for (int i = 0; i < N / 2; ++i) {
    const float2 x = make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
    const float2 a = __ffma2_rn(x, c2, neg_hi);
    pr[i] = make_float2(ex2_approx(a.x), ex2_approx(a.y));
  }
}
__device__ __forceinline__ uint32_t pack_group(const float2 p01, const float2 p23, const float2 neg_128f, float2& sum_a, float2& sum_b) {
  const float2 magic2 = make_float2(kMagic, kMagic);
  sum_a = __fadd2_rn(sum_a, p01);
  sum_b = __fadd2_rn(sum_b, p23);
  const float2 y01 = __ffma2_rn(p01, neg_128f, magic2);      // low byte = two's complement of -P8
  const float2 y23 = __ffma2_rn(p23, neg_128f, magic2);
  return __byte_perm(__byte_perm(__float_as_uint(y01.x), __float_as_uint(y01.y), 0x0040),
                     __byte_perm(__float_as_uint(y23.x), __float_as_uint(y23.y), 0x0040), 0x5410);
}
template <int N>
__device__ __forceinline__ void chunk_pack(const float2 (&pr)[N / 2], const float2 neg_128f, float2 (&sum)[4], uint32_t (&packed)[N / 4]) {
#pragma unroll
  for (int g = 0; g < N / 4; ++g) packed[g] = pack_group(pr[2 * g], pr[2 * g + 1], neg_128f, sum[(2 * g) & 3], sum[(2 * g + 1) & 3]);
}
// exp of chunk `rn` (-> pn) interleaved with pack of chunk `pc` (-> packed), four elements at a time.
template <int N>
__device__ __forceinline__ void chunk_exp_and_pack(const uint32_t (&rn)[N], float2 (&pn)[N / 2], const float2 (&pc)[N / 2],
                                                   const float2 c2, const float2 neg_hi, const float2 neg_128f,
                                                   float2 (&sum)[4], uint32_t (&packed)[N / 4]) {
#pragma unroll
  for (int g = 0; g < N / 4; ++g) {
    const float2 x01 = make_float2(__uint_as_float(rn[4 * g]), __uint_as_float(rn[4 * g + 1]));
    const float2 x23 = make_float2(__uint_as_float(rn[4 * g + 2]), __uint_as_float(rn[4 * g + 3]));
    const float2 a01 = __ffma2_rn(x01, c2, neg_hi);
    const float2 a23 = __ffma2_rn(x23, c2, neg_hi);
    const float2 magic2 = make_float2(kMagic, kMagic);
    float2 n01, n23;
    n01.x = ex2_approx(a01.x);
    sum[(2 * g) & 3] = __fadd2_rn(sum[(2 * g) & 3], pc[2 * g]);
    sum[(2 * g + 1) & 3] = __fadd2_rn(sum[(2 * g + 1) & 3], pc[2 * g + 1]);
    n01.y = ex2_approx(a01.y);
    const float2 y01 = __ffma2_rn(pc[2 * g], neg_128f, magic2);
    const float2 y23 = __ffma2_rn(pc[2 * g + 1], neg_128f, magic2);
    n23.x = ex2_approx(a23.x);
    const uint32_t lo = __byte_perm(__float_as_uint(y01.x), __float_as_uint(y01.y), 0x0040);
    const uint32_t hi = __byte_perm(__float_as_uint(y23.x), __float_as_uint(y23.y), 0x0040);
    n23.y = ex2_approx(a23.y);
    packed[g] = __byte_perm(lo, hi, 0x5410);
    pn[2 * g] = n01;
    pn[2 * g + 1] = n23;
  }
}

// Constants of one row of one tile, derived from the biased integer row maximum.
struct RowConsts {
  float2 c2, neg_hi, neg_128f;
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
  k.neg_128f = make_float2(p_mul * k.f, p_mul * k.f);       // -128 f (or +255 f): quantisation multiplier
  // the value the reference computes for the maximal element (inc/fmha_i8.cuh:196)
  k.m_tile = (row_scale * static_cast<float>(imax - static_cast<int>(kMagicBits))) * scale_qk;
  return k;
}

// S row (tensor memory) -> statistics + quantised P row (tensor memory, over the front of S).
// Fast path: no masked key in the tile.  The eight 16-column chunks are double-buffered so that a
// tensor-memory load is always in flight while the previous chunk is processed.
__device__ __forceinline__ TileStats softmax_tile_fast(const uint32_t tS, const FwdParams& p, const int trace_slot = 0, const int trace_idx = 0) {
  uint32_t ra[16], rb[16];
  int max_a = INT_MIN, max_b = INT_MIN;
  {
    // pass 1 has almost no work per element, so it is bound by the tensor-memory round trip
    // (about 200 cycles): two wide loads instead of many narrow ones
    uint32_t wide[64];
    tmem_ld64_issue(tS, wide);
    tmem_ld_fence(wide);
    chunk_max<false, 64>(wide, 0u, max_a, max_b);
    tmem_ld64_issue(tS + 64, wide);
    tmem_ld_fence(wide);
    tmem_ld16_issue(tS, ra);                 // first chunk of pass 2, in flight during the second half of the max
    chunk_max<false, 64>(wide, 0u, max_a, max_b);
  }
  const RowConsts k = row_consts(max(max_a, max_b), p.c2, p.row_scale, p.scale_qk, p.p_mul);
  if ((threadIdx.x >> 5 & 3) == FMHA_TRACE_Q) FMHA_STAMP(trace_slot, trace_idx);
  float2 sum[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
  uint32_t packed[4];
  float2 pa[8], pb[8];
  // pass 2: software pipeline over eight 16-column chunks: the exponentials of chunk c+1 are issued
  // together with the packing of chunk c, and the load of chunk c+2 is in flight meanwhile
  tmem_ld_fence(ra); tmem_ld16_issue(tS + 16, rb);
  chunk_exp<16>(ra, k.c2, k.neg_hi, pa);
#pragma unroll
  for (int c = 0; c < 8; c += 2) {
    tmem_ld_fence(rb); if (c + 2 < 8) tmem_ld16_issue(tS + (c + 2) * 16, ra);
    chunk_exp_and_pack<16>(rb, pb, pa, k.c2, k.neg_hi, k.neg_128f, sum, packed); tmem_st4(tS + c * 4, packed);
    if (c + 2 < 8) {
      tmem_ld_fence(ra); tmem_ld16_issue(tS + (c + 3) * 16, rb);
      chunk_exp_and_pack<16>(ra, pa, pb, k.c2, k.neg_hi, k.neg_128f, sum, packed); tmem_st4(tS + (c + 1) * 4, packed);
    } else {
      chunk_pack<16>(pb, k.neg_128f, sum, packed); tmem_st4(tS + (c + 1) * 4, packed);
    }
  }
  TileStats st;
  st.m_tile = k.m_tile;
  st.l_tile = k.f * (((sum[0].x + sum[0].y) + (sum[1].x + sum[1].y)) + ((sum[2].x + sum[2].y) + (sum[3].x + sum[3].y)));
  return st;
}

// Per-key path for tiles that contain masked keys: compact (rolled) code, used at most once per row
// with valid-length padding.
__device__ __forceinline__ TileStats softmax_tile_mixed(const uint32_t tS, const float c2s, const float row_scale,
                                                        const float scale_qk, const float p_mul, const uint32_t* mask_words) {
  uint32_t r[32];
  int max_a = INT_MIN, max_b = INT_MIN;
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    tmem_ld32(tS + c * 32, r);
    chunk_max<true, 32>(r, mask_words[c], max_a, max_b);
  }
  const RowConsts k = row_consts(max(max_a, max_b), c2s, row_scale, scale_qk, p_mul);
  float2 sum[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    uint32_t packed[8];
    tmem_ld32(tS + c * 32, r);
    chunk_exp_pack<true, 32>(r, mask_words[c], k.c2, k.neg_hi, k.neg_128f, sum, packed);
    tmem_st8(tS + c * 8, packed);
  }
  TileStats st;
  st.m_tile = k.m_tile;
  st.l_tile = k.f * (((sum[0].x + sum[0].y) + (sum[1].x + sum[1].y)) + ((sum[2].x + sum[2].y) + (sum[3].x + sum[3].y)));
  return st;
}

// o2 (+)= e_cur * (P8 . V) for N output columns; x = raw accumulator read as float = kMagic + O~neg.
template <int N>
__device__ __forceinline__ void drain_chunk(const uint32_t (&r)[N], float2* o2, const float2 neg_ec, const float2 e_bias, const float2 e_old) {
#pragma unroll
  for (int i = 0; i < N / 2; ++i) {
    const float2 x = make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
    const float2 t = __ffma2_rn(x, neg_ec, e_bias);          // e_cur * (P8 . V), exact product before rounding
    o2[i] = __ffma2_rn(o2[i], e_old, t);
  }
}

// One softmax thread, one work unit: query row q_row of query tile w.  `tiles_done` counts the key tiles
// this query-tile slot has processed in earlier units of this CTA: the barriers shared with the MMA issuer
// keep flipping phase across units.  Returns false if a wait gave up.
template <int D>
__device__ __forceinline__ bool softmax_unit(const FwdParams& p, FwdCtl<FwdCfg<D>::kStages>* ctl, const UnitInfo* info, const int w,
                                             const uint32_t tmem_base, const int q_row, const int bh_local, const uint32_t tiles_done) {
  const int warp = threadIdx.x >> 5;
  const uint32_t lane_field = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const uint32_t tS = tmem_base + lane_field + static_cast<uint32_t>(w * kTile);
  const uint32_t tO = tmem_base + lane_field + static_cast<uint32_t>(2 * kTile + w * D);
  const uint32_t bar_s = smem_u32(&ctl->s_full[w]), bar_p = smem_u32(&ctl->p_ready[w]);
  const uint32_t bar_o = smem_u32(&ctl->o_full[w]), bar_f = smem_u32(&ctl->o_free[w]);
  const int n_live = info->n_live;
  volatile int* abort_flag = &ctl->abort;

  float2 o2[D / 2];
#pragma unroll
  for (int i = 0; i < D / 2; ++i) o2[i] = make_float2(0.f, 0.f);
  float m_run = -INFINITY, l_run = 0.f;
  bool ok = true;

#pragma unroll 1
  for (int j = 0; j < n_live; ++j) {
    const uint32_t ph = (tiles_done + static_cast<uint32_t>(j)) & 1u;
    ok = __all_sync(0xFFFFFFFFu, mbar_wait(bar_s, ph, abort_flag));
    if (!ok) { raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_S_READY, j); break; }
    tc_fence_after();
    if ((threadIdx.x >> 5 & 3) == FMHA_TRACE_Q) FMHA_STAMP(w * 4 + 0, j);

    TileStats st;
    if (info->mixed[j] != 0) st = softmax_tile_mixed(tS, p.c2, p.row_scale, p.scale_qk, p.p_mul, &info->maskbits[4 * info->live[j]]);
    else st = softmax_tile_fast(tS, p, 12 + w, j);
    tmem_wait_st();
    tc_fence_before();
    mbar_arrive(bar_p);
    if ((threadIdx.x >> 5 & 3) == FMHA_TRACE_Q) FMHA_STAMP(w * 4 + 1, j);

    // ---- merge of tile statistics (inc/fmha_i8.cuh:301-304)
    const float m_new = fmaxf(m_run, st.m_tile);
    const float e_old = __expf(m_run - m_new);                       // 0 on the first tile (m_run = -inf)
    const float e_cur = clear_low2(__expf(st.m_tile - m_new));       // 22 significant bits: kMagic*e_cur is exact
    l_run = fmaf(e_old, l_run, e_cur * st.l_tile);
    m_run = m_new;
    const float es = p.o_sign * e_cur;                               // the accumulator holds bias + o_sign * (P.V)
    const float2 neg_ec = make_float2(es, es), e_bias = make_float2(-es * kMagic, -es * kMagic);
    const float2 e_old2 = make_float2(e_old, e_old);

    // ---- drain O~ = bias -/+ (P8 . V) into the fp32 running row
    ok = __all_sync(0xFFFFFFFFu, mbar_wait(bar_o, ph, abort_flag));
    if (!ok) { raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_O_READY, j); break; }
    tc_fence_after();
    if ((threadIdx.x >> 5 & 3) == FMHA_TRACE_Q) FMHA_STAMP(w * 4 + 2, j);
    {
      uint32_t wide[64];
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tmem_ld64_issue(tO + c * 64, wide);
        tmem_ld_fence(wide);
        drain_chunk<64>(wide, o2 + c * 32, neg_ec, e_bias, e_old2);
      }
    }
    tc_fence_before();
    mbar_arrive(bar_f);
    if ((threadIdx.x >> 5 & 3) == FMHA_TRACE_Q) FMHA_STAMP(w * 4 + 3, j);
  }

  // ---- calibration mode: only the largest magnitude of the unquantised output is wanted (the reference
  //      takes o_amax from its fp32 CPU result, test_fmha_i8.cpp:161)
  if (p.amax_out != nullptr) {
    float mx = 0.f;
    if (ok && q_row < p.Sq && n_live > 0 && l_run > 0.f) {
      const float inv = 1.0f / l_run;
#pragma unroll
      for (int i = 0; i < D / 2; ++i) mx = fmaxf(mx, fmaxf(fabsf(o2[i].x * inv), fabsf(o2[i].y * inv)));
    }
    // non-negative floats order like their bit patterns
    const unsigned bits = __reduce_max_sync(0xFFFFFFFFu, __float_as_uint(mx * p.amax_scale));
    if ((threadIdx.x & 31) == 0 && bits != 0u) atomicMax(reinterpret_cast<unsigned*>(p.amax_out), bits);
    return ok;
  }

  // ---- epilogue (inc/fmha_i8.cuh:318-332): normalise, requantise, 16-byte stores
  if (ok && q_row < p.Sq) {
    const float inv = (n_live > 0 && l_run > 0.f) ? 1.0f / l_run : 0.f;
    int8_t* dst = p.o + (static_cast<int64_t>(bh_local) * p.Sq + q_row) * D;
    // rn(clamp(x)) through the magic-number addition (the low byte of clamp(x) + 1.5*2^23 is the two's-complement
    // integer), bytes gathered with PRMT: conversions and shifts would cost three times the issue cycles
    const float2 inv2 = make_float2(inv, inv), sc2 = make_float2(p.scale_v_out, p.scale_v_out);
    const float2 zero2 = make_float2(0.f, 0.f), magic2 = make_float2(kMagic, kMagic);
#pragma unroll
    for (int c = 0; c < D / 16; ++c) {
      uint32_t wds[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float2 a = __ffma2_rn(sc2, __ffma2_rn(o2[c * 8 + g * 2], inv2, zero2), zero2);        // scale_v_out * (o * inv), each product rounded
        float2 b = __ffma2_rn(sc2, __ffma2_rn(o2[c * 8 + g * 2 + 1], inv2, zero2), zero2);
        a.x = fminf(fmaxf(a.x, -127.f), 127.f); a.y = fminf(fmaxf(a.y, -127.f), 127.f);
        b.x = fminf(fmaxf(b.x, -127.f), 127.f); b.y = fminf(fmaxf(b.y, -127.f), 127.f);
        const float2 ya = __fadd2_rn(a, magic2), yb = __fadd2_rn(b, magic2);
        wds[g] = __byte_perm(__byte_perm(__float_as_uint(ya.x), __float_as_uint(ya.y), 0x0040),
                             __byte_perm(__float_as_uint(yb.x), __float_as_uint(yb.y), 0x0040), 0x5410);
      }
      *reinterpret_cast<uint4*>(dst + c * 16) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
    }
  }
  return ok;
}

// Geometry of work unit u.
struct UnitGeom {
  int bh_local, batch, q_row0, nq;
};
__device__ __forceinline__ UnitGeom unit_geom(const FwdParams& p, int u) {
  UnitGeom g;
  g.bh_local = u / p.q_pairs;
  const int pair = u - g.bh_local * p.q_pairs;
  g.batch = (p.bh_begin + g.bh_local) / p.H;
  g.q_row0 = pair * 2 * kTile;
  g.nq = (g.q_row0 + kTile < p.Sq) ? 2 : 1;
  return g;
}

// Persistent kernel: gridDim.x = min(units, SMs) CTAs; CTA b processes units b, b + gridDim.x, ...
// Tensor memory, barriers and the bias operands are set up once; the scanner warp prepares the next
// unit's mask information and the loader prefetches its tiles while the current unit is finishing, so a
// unit boundary costs about one MMA round trip instead of a CTA launch, a cold TMA load and a pipeline fill.
template <int D>
__global__ void __launch_bounds__(kFwdThreads, 1)
fmha_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const FwdParams p) {
  using Cfg = FwdCfg<D>;
  constexpr int NS = Cfg::kStages;
  using Ctl = FwdCtl<NS>;
  extern __shared__ uint8_t smem_raw[];
  // tiles need 1024-byte alignment (swizzle atoms); the launch reserves the slack
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* bias_a = tiles + Cfg::kTilesBytesTotal;
  uint8_t* bias_b = bias_a + kBiasBytes;
  Ctl* ctl = reinterpret_cast<Ctl*>(bias_b + kBiasBytes);
  const uint32_t q_smem = smem_u32(tiles);
  const uint32_t k_smem = q_smem + 2 * Cfg::kTileBytes;
  const uint32_t v_smem = k_smem + NS * Cfg::kTileBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (p.S + kTile - 1) / kTile;
  const int first_unit = blockIdx.x, unit_step = gridDim.x;

  // an earlier CTA already gave up: do not start (decided by one thread so the CTA stays uniform)
  __shared__ int s_go;
  if (threadIdx.x == 0) s_go = (*reinterpret_cast<volatile unsigned*>(p.status) == 0u) ? 1 : 0;
  __syncthreads();
  if (!s_go) return;

  if (threadIdx.x == 0) {
    ctl->abort = 0;
    for (int w = 0; w < 2; ++w) {
      mbar_init(smem_u32(&ctl->q_full[w]), 1);
      mbar_init(smem_u32(&ctl->q_empty[w]), 1);
    }
    for (int s = 0; s < NS; ++s) {
      mbar_init(smem_u32(&ctl->k_full[s]), 1);
      mbar_init(smem_u32(&ctl->k_empty[s]), 1);
      mbar_init(smem_u32(&ctl->v_full[s]), 1);
      mbar_init(smem_u32(&ctl->v_empty[s]), 1);
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(smem_u32(&ctl->s_full[w]), 1);
      mbar_init(smem_u32(&ctl->p_ready[w]), kTile);
      mbar_init(smem_u32(&ctl->o_full[w]), 1);
      mbar_init(smem_u32(&ctl->o_free[w]), kTile);
      mbar_init(smem_u32(&ctl->info_full[w]), 1);
      mbar_init(smem_u32(&ctl->info_empty[w]), kInfoConsumers);
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

  // Every role walks the same unit sequence; `it` counts this CTA's units, info buffer = it & 1, and the
  // phase of an info barrier for unit `it` is (it >> 1) & 1.
  if (warp < 8) {
    // ------------------------------------------------------------------ softmax groups
    setmaxnreg_inc<FwdRegs<D>::kSoftmax>();      // (a request equal to the launch allocation changes nothing)
    const int w = warp >> 2;
    const int row_in_tile = (warp & 3) * 32 + lane;
    uint32_t tiles_done = 0;
    int it = 0;
    for (int u = first_unit; u < p.n_units; u += unit_step, ++it) {
      const int buf = it & 1;
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&ctl->info_full[buf]), static_cast<uint32_t>((it >> 1) & 1), abort_flag))) {
        raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_INFO, it);
        break;
      }
      const UnitGeom g = unit_geom(p, u);
      const UnitInfo* info = &ctl->info[buf];
      bool ok = true;
      if (w < g.nq) {
        ok = softmax_unit<D>(p, ctl, info, w, tmem_base, g.q_row0 + w * kTile + row_in_tile, g.bh_local, tiles_done);
        tiles_done += static_cast<uint32_t>(info->n_live);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->info_empty[buf]));     // this warp is done with the unit's mask information
      if (!ok) break;
    }
  } else {
    setmaxnreg_dec<FwdRegs<D>::kOther>();
    if (warp == kWarpLoad) {
      // ---------------------------------------------------------------- loader
      if (lane == 0) {
        uint32_t kv_done = 0;      // key tiles loaded in earlier units: ring position and phase continue across units
        uint32_t q_loads[2] = {0u, 0u};   // Q tiles loaded so far per query-tile slot (phase of q_full[w] / q_empty[w])
        bool ok = true;
        int it = 0;
        for (int u = first_unit; u < p.n_units && ok; u += unit_step, ++it) {
          const int buf = it & 1;
          if (!mbar_wait(smem_u32(&ctl->info_full[buf]), static_cast<uint32_t>((it >> 1) & 1), abort_flag)) {
            raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_INFO, it); ok = false; break;
          }
          const UnitGeom g = unit_geom(p, u);
          const UnitInfo* info = &ctl->info[buf];
          const int n_live = info->n_live;
          if (n_live > 0) {
            // a slot's Q rows of the previous unit are free once that slot's last S = Q.K^T has completed
            for (int w = 0; w < g.nq && ok; ++w) {
              if (q_loads[w] > 0 && !mbar_wait(smem_u32(&ctl->q_empty[w]), (q_loads[w] - 1) & 1u, abort_flag)) {
                raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_K_FREE, it); ok = false; break;
              }
              const uint32_t bar_q = smem_u32(&ctl->q_full[w]);
              mbar_arrive_expect_tx(bar_q, static_cast<uint32_t>(Cfg::kTileBytes));
              tma_load_3d(q_smem + w * Cfg::kTileBytes, &map_q, bar_q, 0, g.q_row0 + w * kTile, g.bh_local);
              ++q_loads[w];
            }
            if (!ok) break;
            for (int j = 0; j < n_live; ++j) {
              const int t = info->live[j];
              const uint32_t gidx = kv_done + static_cast<uint32_t>(j);
              const uint32_t s = gidx % NS, round = gidx / NS;
              if (round > 0 && !mbar_wait(smem_u32(&ctl->k_empty[s]), (round - 1) & 1u, abort_flag)) {
                raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_K_FREE, j); ok = false; break;
              }
              mbar_arrive_expect_tx(smem_u32(&ctl->k_full[s]), Cfg::kTileBytes);
              tma_load_3d(k_smem + s * Cfg::kTileBytes, &map_k, smem_u32(&ctl->k_full[s]), 0, t * kTile, g.bh_local);
              if (round > 0 && !mbar_wait(smem_u32(&ctl->v_empty[s]), (round - 1) & 1u, abort_flag)) {
                raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_V_FREE, j); ok = false; break;
              }
              mbar_arrive_expect_tx(smem_u32(&ctl->v_full[s]), Cfg::kTileBytes);
              tma_load_3d(v_smem + s * Cfg::kTileBytes, &map_v, smem_u32(&ctl->v_full[s]), 0, t * kTile, g.bh_local);
            }
            kv_done += static_cast<uint32_t>(n_live);
          }
          mbar_arrive(smem_u32(&ctl->info_empty[buf]));
        }
        if (!ok) {
          // unwinding: let copies that are still in flight land before the CTA may exit
          const long long t0 = clock64();
          while (clock64() - t0 < 2000000LL) { /* about a millisecond */ }
        }
      }
    } else if (warp == kWarpMma) {
      // ---------------------------------------------------------------- MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc_s = make_idesc_i8(kTile, false);   // S = Q.K^T : N = 128 keys, both K-major
        const uint32_t idesc_o = p.p_unsigned ? make_idesc_i8(D, true, true) : make_idesc_i8(D, true, false);   // O = P.V : N = D, V is MN-major
        constexpr uint32_t idesc_bias_s = make_idesc_f16(kTile);
        constexpr uint32_t idesc_bias_o = make_idesc_f16(D);
        const uint64_t d_bias_a = make_smem_desc_noswizzle(smem_u32(bias_a), 128, 256);
        const uint64_t d_bias_b = make_smem_desc_noswizzle(smem_u32(bias_b), 128, 256);
        auto issue_s = [&](int w, uint32_t stage) {
          const uint64_t dq = make_smem_desc(q_smem + w * Cfg::kTileBytes, D);
          const uint64_t dk = make_smem_desc(k_smem + stage * Cfg::kTileBytes, D);
          mma_f16_ss(tmem_base + w * kTile, d_bias_a, d_bias_b, idesc_bias_s, 0u);      // accumulator := 0x4B400000
#pragma unroll
          for (int kk = 0; kk < D / 32; ++kk)
            mma_i8_ss(tmem_base + w * kTile, desc_advance(dq, kk * 32), desc_advance(dk, kk * 32), idesc_s, 1u);
          mma_commit(smem_u32(&ctl->s_full[w]));
        };
        auto issue_o = [&](int w, uint32_t stage) {
          const uint64_t dv = make_smem_desc(v_smem + stage * Cfg::kTileBytes, D);
          mma_f16_ss(tmem_base + 2 * kTile + w * D, d_bias_a, d_bias_b, idesc_bias_o, 0u);
#pragma unroll
          for (int kk = 0; kk < kTile / 32; ++kk)
            mma_i8_ts(tmem_base + 2 * kTile + w * D, tmem_base + w * kTile + kk * 8, desc_advance(dv, kk * 32 * D), idesc_o, 1u);
          mma_commit(smem_u32(&ctl->o_full[w]));
        };
        uint32_t kv_done = 0;              // key tiles consumed in earlier units (ring position / phase)
        uint32_t tiles_done[2] = {0u, 0u}; // key tiles each query-tile slot has processed in earlier units
        uint32_t q_waits[2] = {0u, 0u};    // Q tiles each slot has waited for so far (phase of q_full[w])
        bool pre[2] = {false, false};      // this unit's first S of slot w was already issued at the end of the previous unit
        int first_s_count = 0;             // how many slots have issued the current (or, when looking ahead, next) unit's first S
        bool ok = true;
        int it = 0;
        // A wait that gives up only notes which one it was; the status is raised once, after the loops, so that the
        // loops contain no calls (every call site would cost this register-starved thread spills around it).
        uint32_t err = 0u, err_tile = 0u;
        auto wait = [&](uint32_t bar, uint32_t parity, uint32_t code, uint32_t tile) -> bool {
          if (mbar_wait(bar, parity, abort_flag)) return true;
          err = code;
          err_tile = tile;
          return false;
        };
        // First S = Q.K^T of a unit for slot w: key-tile stage s0 of a unit with n_live_u live tiles and nq_u query tiles.
        auto first_s = [&](int w, uint32_t gidx0, int n_live_u, int nq_u) -> bool {
          const uint32_t s0 = gidx0 % NS;
          if (!wait(smem_u32(&ctl->q_full[w]), q_waits[w] & 1u, FMHA_I8_DEV_WAIT_Q_LOAD, w)) return false;
          ++q_waits[w];
          if (!wait(smem_u32(&ctl->k_full[s0]), (gidx0 / NS) & 1u, FMHA_I8_DEV_WAIT_K_LOAD, 0)) return false;
          tc_fence_after();
          issue_s(w, s0);
          if (n_live_u == 1) mma_commit(smem_u32(&ctl->q_empty[w]));      // the unit's only use of this slot's Q
          if (++first_s_count == nq_u) mma_commit(smem_u32(&ctl->k_empty[s0]));   // every slot has read this K stage
          return true;
        };
        for (int u = first_unit; u < p.n_units && ok; u += unit_step, ++it) {
          const int buf = it & 1;
          if (!wait(smem_u32(&ctl->info_full[buf]), static_cast<uint32_t>((it >> 1) & 1), FMHA_I8_DEV_WAIT_INFO, it)) { ok = false; break; }
          const UnitGeom g = unit_geom(p, u);
          const int n_live = ctl->info[buf].n_live;
          const int nq = g.nq;
          // what comes after this unit (looked at when a slot finishes its last tile here)
          const int u_next = u + unit_step;
          bool next_known = false;
          int n_live_next = 0, nq_next = 0;
          if (n_live > 0) {
            for (int w = 0; w < nq && ok; ++w)
              if (!pre[w]) ok = first_s(w, kv_done, n_live, nq);
            pre[0] = pre[1] = false;
            first_s_count = 0;
            for (int j = 0; j < n_live && ok; ++j) {
              const uint32_t gidx = kv_done + static_cast<uint32_t>(j);
              const uint32_t s = gidx % NS;
              if (!wait(smem_u32(&ctl->v_full[s]), (gidx / NS) & 1u, FMHA_I8_DEV_WAIT_V_LOAD, j)) { ok = false; break; }
              const uint32_t gn = gidx + 1, sn = gn % NS;
              for (int w = 0; w < nq; ++w) {
                const uint32_t tw = tiles_done[w] + static_cast<uint32_t>(j);     // this slot's cumulative tile index
                if (!wait(smem_u32(&ctl->p_ready[w]), tw & 1u, FMHA_I8_DEV_WAIT_P_READY, j)) { ok = false; break; }
                if (tw > 0 && !wait(smem_u32(&ctl->o_free[w]), (tw - 1) & 1u, FMHA_I8_DEV_WAIT_O_FREE, j)) { ok = false; break; }
                tc_fence_after();
                issue_o(w, s);
                if (w == nq - 1) mma_commit(smem_u32(&ctl->v_empty[s]));
                // ---- this slot's next S = Q.K^T: the next key tile of this unit, or -- after the unit's last tile --
                //      the first key tile of the NEXT unit, started now rather than when the other slot has finished
                //      too, so that the two slots keep their offset across unit boundaries
                bool cross = false, have_next = (j + 1 < n_live);
                uint32_t g_next = gidx + 1;
                if (!have_next && u_next < p.n_units) {
                  if (!next_known) {
                    if (!wait(smem_u32(&ctl->info_full[buf ^ 1]), static_cast<uint32_t>(((it + 1) >> 1) & 1), FMHA_I8_DEV_WAIT_INFO, it + 1)) { ok = false; break; }
                    n_live_next = ctl->info[buf ^ 1].n_live;
                    nq_next = unit_geom(p, u_next).nq;
                    next_known = true;
                  }
                  cross = have_next = (n_live_next > 0 && w < nq_next);
                }
                if (have_next) {
                  const uint32_t s_next = g_next % NS;
                  if (cross) {
                    if (!wait(smem_u32(&ctl->q_full[w]), q_waits[w] & 1u, FMHA_I8_DEV_WAIT_Q_LOAD, w)) { ok = false; break; }
                    ++q_waits[w];
                  }
                  if ((cross || w == 0) && !wait(smem_u32(&ctl->k_full[s_next]), (g_next / NS) & 1u, FMHA_I8_DEV_WAIT_K_LOAD, j + 1)) { ok = false; break; }
                  tc_fence_after();
                  // S_w / P_w columns are free again: the tensor pipe runs this thread's MMAs in order
                  issue_s(w, s_next);
                  // that was the unit's last use of this slot's Q rows?
                  if (cross ? (n_live_next == 1) : (j + 2 == n_live)) mma_commit(smem_u32(&ctl->q_empty[w]));
                  // has every slot read this K stage?
                  if (cross) {
                    pre[w] = true;
                    if (++first_s_count == nq_next) mma_commit(smem_u32(&ctl->k_empty[s_next]));
                  } else if (w == nq - 1) {
                    mma_commit(smem_u32(&ctl->k_empty[s_next]));
                  }
                }
              }
            }
            kv_done += static_cast<uint32_t>(n_live);
            for (int w = 0; w < nq; ++w) tiles_done[w] += static_cast<uint32_t>(n_live);
          }
          mbar_arrive(smem_u32(&ctl->info_empty[buf]));
        }
        if (err != 0u) raise_status(abort_flag, p.status, err, err_tile);
      }
    } else if (warp == kWarpScan) {
      // ---------------------------------------------------------------- scanner: mask information, one unit ahead
      bool ok = true;
      int it = 0;
      for (int u = first_unit; u < p.n_units && ok; u += unit_step, ++it) {
        const int buf = it & 1;
        // the buffer was used by unit it-2: wait until all ten consumer warps have released it
        if (it >= 2) {
          ok = __all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&ctl->info_empty[buf]), static_cast<uint32_t>(((it >> 1) - 1) & 1), abort_flag));
          if (!ok) { if (lane == 0) raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_INFO, it); break; }
        }
        const UnitGeom g = unit_geom(p, u);
        scan_mask_warp(&ctl->info[buf], p.mask + static_cast<int64_t>(g.batch) * p.S, p.S, n_tiles);
        if (lane == 0) mbar_arrive(smem_u32(&ctl->info_full[buf]));
      }
    }
  }

  // every unit of this CTA has been computed and stored by the time the softmax groups leave their loop
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace fmha
