// The INT8 flash-attention forward kernel for sm_100a.
//
// Replaces the reference project's FMHAInferKernel (inc/fmha_i8.cuh:43-334).  Same arithmetic
// contract -- key tiles of 128 starting at key 0, P quantised to 8 bits against each tile's own row
// maximum, tiles merged in fp32 -- on a different machine model:
//
//   work unit  = (batch*head, pair of 128-row query tiles); one CTA per unit, one CTA per SM
//   warp 8     = loader: TMA brings Q (once) and a ring of K and V tiles into swizzled shared memory
//   warp 9     = MMA issuer: one thread issues tcgen05.mma kind::i8
//                  S_w   = Q_w . K_j^T        (smem x smem  -> int32 in tensor memory)
//                  O~_w  = P_w . V_j          (tmem x smem  -> int32 in tensor memory)
//   warps 0-3  = softmax group of query tile 0, warps 4-7 = of query tile 1: one thread owns one
//                query row, so row max / row sum need no shuffles.  Per key tile a thread reads its S
//                row from tensor memory twice (integer max, then exp + requantise), writes the 8-bit P
//                row back over the front of S, and after P.V drains the int32 partial output into its
//                fp32 running row.
//
// Tensor memory (512 columns x 128 lanes x 32 bit): S_0 [0,128) S_1 [128,256) O~_0 [256,256+D)
// O~_1 [256+D,256+2D).  P_w occupies the first 32 columns of S_w (four int8 per column).
//
// Numerics kept equal to the reference kernel within the test tolerance: the running output is kept
// unnormalised (divided by the row sum once at the end) instead of renormalised after every tile,
// exp() is ex2.approx on an argument formed exactly in the integer domain, and masked keys
// contribute exactly zero (the reference adds a large negative number before scaling,
// inc/fmha_i8.cuh:191-193).  Key tiles with no unmasked key are skipped.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "ptx.cuh"
#include "../../include/fmha_i8_c.h"

namespace fmha {

constexpr int kTile = 128;           // query rows per tile == keys per tile
constexpr int kMaxSeq = 32768;
constexpr int kMaxTiles = kMaxSeq / kTile;
constexpr int kFwdThreads = 320;
constexpr int kWarpLoad = 8;
constexpr int kWarpMma = 9;
constexpr uint32_t kTmemCols = 512;
constexpr float kMagic = 12582912.0f;          // 1.5 * 2^23: float whose ulp is 1 over [2^23, 2^24)
constexpr uint32_t kMagicBits = 0x4B400000u;

template <int D> struct FwdCfg {
  static_assert(D == 64 || D == 128, "head_dim must be 64 or 128");
  static constexpr int kStages = (D == 128) ? 4 : 6;       // ring depth of K and of V
  static constexpr int kTileBytes = kTile * D;              // one 128-row tile of int8
  static constexpr int kTilesBytesTotal = (2 + 2 * kStages) * kTileBytes;
};

struct FwdParams {
  const int8_t* mask;   // [B,S] whole mask
  int8_t* o;            // first head of the slice
  int S, H, bh_begin, bh_count, q_pairs;
  float row_scale;      // 1/sqrt(D), the reference's constant (inc/fmha_i8.cuh:71)
  float scale_qk;       // q_amax*k_amax/127^2 (inc/fmha_i8.cuh:72)
  float scale_v_out;    // v_amax/(o_amax*128) (inc/fmha_i8.cuh:318)
  float c2;             // row_scale*scale_qk*log2(e) with the two lowest mantissa bits cleared
  float c2_bias;        // kMagic*c2, exact because c2 has 22 significant bits
  unsigned* status;     // eight device status words
};

template <int NS> struct FwdCtl {
  uint64_t q_full;
  uint64_t k_full[NS], k_empty[NS], v_full[NS], v_empty[NS];
  uint64_t s_full[2], p_ready[2], o_full[2], o_free[2];
  uint32_t tmem_base;
  int abort;
  int n_live;
  uint32_t maskbits[kMaxTiles * 4];   // bit set = key masked (or beyond seq_len)
  uint16_t live[kMaxTiles];           // indices of key tiles that have at least one unmasked key
  uint8_t mixed[kMaxTiles];           // 1 = that live tile has masked keys too
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

// Builds the per-CTA view of one batch's padding mask: 128-bit masks per key tile, the list of
// live tiles and whether each needs the per-key path.
template <class Ctl>
__device__ void scan_mask(Ctl* ctl, const int8_t* mask_row, int S, int n_tiles) {
  const uint32_t* words = reinterpret_cast<const uint32_t*>(mask_row);
  for (int g = threadIdx.x; g < n_tiles * 4; g += blockDim.x) {
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
    ctl->maskbits[g] = bits;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int n = 0;
    for (int t = 0; t < n_tiles; ++t) {
      const uint32_t a = ctl->maskbits[4 * t], b = ctl->maskbits[4 * t + 1], c = ctl->maskbits[4 * t + 2], d = ctl->maskbits[4 * t + 3];
      if ((a & b & c & d) != 0xFFFFFFFFu) {
        ctl->live[n] = static_cast<uint16_t>(t);
        ctl->mixed[n] = ((a | b | c | d) != 0u) ? 1 : 0;
        ++n;
      }
    }
    ctl->n_live = n;
  }
}

// One softmax thread: query row `row` of query tile w.  Returns false if a wait gave up.
template <int D, bool kDummy = false>
__device__ __forceinline__ void softmax_rows(const FwdParams& p, FwdCtl<FwdCfg<D>::kStages>* ctl, const int w,
                                             const uint32_t tmem_base, const int q_row, const int bh_local) {
  const int warp = threadIdx.x >> 5;
  const uint32_t lane_field = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const uint32_t tS = tmem_base + lane_field + static_cast<uint32_t>(w * kTile);
  const uint32_t tO = tmem_base + lane_field + static_cast<uint32_t>(2 * kTile + w * D);
  const uint32_t bar_s = smem_u32(&ctl->s_full[w]), bar_p = smem_u32(&ctl->p_ready[w]);
  const uint32_t bar_o = smem_u32(&ctl->o_full[w]), bar_f = smem_u32(&ctl->o_free[w]);
  const int n_live = ctl->n_live;
  volatile int* abort_flag = &ctl->abort;

  float o[D];
#pragma unroll
  for (int i = 0; i < D; ++i) o[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  bool ok = true;

  for (int j = 0; j < n_live; ++j) {
    const uint32_t ph = static_cast<uint32_t>(j & 1);
    ok = __all_sync(0xFFFFFFFFu, mbar_wait(bar_s, ph, abort_flag));
    if (!ok) { raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_S_READY, j); break; }
    tc_fence_after();

    const bool mixed = ctl->mixed[j] != 0;
    uint32_t mw[4] = {0u, 0u, 0u, 0u};
    if (mixed) {
      const int t = ctl->live[j];
#pragma unroll
      for (int c = 0; c < 4; ++c) mw[c] = ctl->maskbits[4 * t + c];
    }

    // ---- pass 1: row maximum of the unmasked keys, in the integer domain (the scale is positive)
    int imax = INT_MIN;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(tS + c * 32, r);
      if (mixed) {
#pragma unroll
        for (int i = 0; i < 32; ++i) imax = max(imax, ((mw[c] >> i) & 1u) ? INT_MIN : static_cast<int>(r[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) imax = max(imax, static_cast<int>(r[i]));
      }
    }
    // the value the reference computes for the maximal element (inc/fmha_i8.cuh:196)
    const float m_tile = (p.row_scale * static_cast<float>(imax)) * p.scale_qk;

    // ---- pass 2: p = 2^((s - smax) * c2), row sum, P8 = rn(-128 p) as signed bytes, written over S
    const uint32_t bias = kMagicBits - static_cast<uint32_t>(imax);   // float(bits) = kMagic + (s - smax), exact
    float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(tS + c * 32, r);
      uint32_t packed[8];
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        uint32_t y[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = 4 * g + e;
          float x = __uint_as_float(r[i] + bias);
          if (mixed && ((mw[c] >> i) & 1u)) x = -INFINITY;
          const float pe = ex2_approx(fmaf(x, p.c2, -p.c2_bias));
          if (e == 0) sum0 += pe; else if (e == 1) sum1 += pe; else if (e == 2) sum2 += pe; else sum3 += pe;
          y[e] = __float_as_uint(fmaf(pe, -128.f, kMagic));          // low byte = two's complement of -P8
        }
        packed[g] = __byte_perm(__byte_perm(y[0], y[1], 0x0040), __byte_perm(y[2], y[3], 0x0040), 0x5410);
      }
      tmem_st8(tS + c * 8, packed);
    }
    tmem_wait_st();
    tc_fence_before();
    mbar_arrive(bar_p);
    const float l_tile = (sum0 + sum1) + (sum2 + sum3);

    // ---- merge of tile statistics (inc/fmha_i8.cuh:301-304)
    const float m_new = fmaxf(m_run, m_tile);
    const float e_old = __expf(m_run - m_new);                       // 0 on the first tile (m_run = -inf)
    const float e_cur = clear_low2(__expf(m_tile - m_new));          // 22 significant bits: kMagic*e_cur is exact
    l_run = fmaf(e_old, l_run, e_cur * l_tile);
    m_run = m_new;
    const float e_bias = e_cur * kMagic;

    // ---- drain O~ = -(P8 . V) into the fp32 running row
    ok = __all_sync(0xFFFFFFFFu, mbar_wait(bar_o, ph, abort_flag));
    if (!ok) { raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_O_READY, j); break; }
    tc_fence_after();
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tO + c * 32, r);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float x = __uint_as_float(r[i] + kMagicBits);          // kMagic + O~neg, exact
        const float t = fmaf(x, -e_cur, e_bias);                     // e_cur * (P8 . V)
        o[c * 32 + i] = fmaf(o[c * 32 + i], e_old, t);
      }
    }
    tc_fence_before();
    mbar_arrive(bar_f);
  }

  // ---- epilogue (inc/fmha_i8.cuh:318-332): normalise, requantise, 16-byte stores
  if (ok && q_row < p.S) {
    const float inv = (n_live > 0 && l_run > 0.f) ? 1.0f / l_run : 0.f;
    int8_t* dst = p.o + (static_cast<int64_t>(bh_local) * p.S + q_row) * D;
#pragma unroll
    for (int c = 0; c < D / 16; ++c) {
      uint32_t wds[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint32_t b4 = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float f = p.scale_v_out * (o[c * 16 + g * 4 + e] * inv);
          const int q8 = __float2int_rn(fmaxf(fminf(f, 127.f), -127.f));
          b4 |= (static_cast<uint32_t>(q8) & 0xFFu) << (8 * e);
        }
        wds[g] = b4;
      }
      *reinterpret_cast<uint4*>(dst + c * 16) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
    }
  }
}

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
  Ctl* ctl = reinterpret_cast<Ctl*>(tiles + Cfg::kTilesBytesTotal);
  const uint32_t q_smem = smem_u32(tiles);
  const uint32_t k_smem = q_smem + 2 * Cfg::kTileBytes;
  const uint32_t v_smem = k_smem + NS * Cfg::kTileBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int unit = blockIdx.x;
  const int bh_local = unit / p.q_pairs;
  const int pair = unit - bh_local * p.q_pairs;
  const int batch = (p.bh_begin + bh_local) / p.H;
  const int q_row0 = pair * 2 * kTile;
  const int nq = (q_row0 + kTile < p.S) ? 2 : 1;
  const int n_tiles = (p.S + kTile - 1) / kTile;

  // an earlier CTA already gave up: do not start (decided by one thread so the CTA stays uniform)
  __shared__ int s_go;
  if (threadIdx.x == 0) s_go = (*reinterpret_cast<volatile unsigned*>(p.status) == 0u) ? 1 : 0;
  __syncthreads();
  if (!s_go) return;

  if (threadIdx.x == 0) {
    ctl->abort = 0;
    mbar_init(smem_u32(&ctl->q_full), 1);
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
  scan_mask(ctl, p.mask + static_cast<int64_t>(batch) * p.S, p.S, n_tiles);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);
  const int n_live = ctl->n_live;
  volatile int* abort_flag = &ctl->abort;

  if (warp < 8) {
    // ------------------------------------------------------------------ softmax groups
    const int w = warp >> 2;
    if (w < nq) {
      const int row_in_tile = (warp & 3) * 32 + lane;
      softmax_rows<D>(p, ctl, w, tmem_base, q_row0 + w * kTile + row_in_tile, bh_local);
    }
  } else if (warp == kWarpLoad) {
    // ------------------------------------------------------------------ loader
    if (lane == 0 && n_live > 0) {
      const uint32_t bar_q = smem_u32(&ctl->q_full);
      mbar_arrive_expect_tx(bar_q, static_cast<uint32_t>(nq * Cfg::kTileBytes));
      for (int w = 0; w < nq; ++w) tma_load_3d(q_smem + w * Cfg::kTileBytes, &map_q, bar_q, 0, q_row0 + w * kTile, bh_local);
      bool ok = true;
      for (int j = 0; j < n_live && ok; ++j) {
        const int t = ctl->live[j];
        const int s = j % NS, round = j / NS;
        if (round > 0 && !mbar_wait(smem_u32(&ctl->k_empty[s]), static_cast<uint32_t>((round - 1) & 1), abort_flag)) {
          raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_K_FREE, j); ok = false; break;
        }
        mbar_arrive_expect_tx(smem_u32(&ctl->k_full[s]), Cfg::kTileBytes);
        tma_load_3d(k_smem + s * Cfg::kTileBytes, &map_k, smem_u32(&ctl->k_full[s]), 0, t * kTile, bh_local);
        if (round > 0 && !mbar_wait(smem_u32(&ctl->v_empty[s]), static_cast<uint32_t>((round - 1) & 1), abort_flag)) {
          raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_V_FREE, j); ok = false; break;
        }
        mbar_arrive_expect_tx(smem_u32(&ctl->v_full[s]), Cfg::kTileBytes);
        tma_load_3d(v_smem + s * Cfg::kTileBytes, &map_v, smem_u32(&ctl->v_full[s]), 0, t * kTile, bh_local);
      }
      if (!ok) {
        // unwinding: let copies that are still in flight land before the CTA may exit
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { /* about a millisecond */ }
      }
    }
  } else {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_live > 0) {
      constexpr uint32_t idesc_s = make_idesc_i8(kTile, false);   // S = Q.K^T : N = 128 keys, both K-major
      constexpr uint32_t idesc_o = make_idesc_i8(D, true);        // O = P.V   : N = D, V is MN-major
      bool ok = true;
      auto issue_s = [&](int w, int stage) {
        const uint64_t dq = make_smem_desc(q_smem + w * Cfg::kTileBytes, D);
        const uint64_t dk = make_smem_desc(k_smem + stage * Cfg::kTileBytes, D);
#pragma unroll
        for (int kk = 0; kk < D / 32; ++kk)
          mma_i8_ss(tmem_base + w * kTile, desc_advance(dq, kk * 32), desc_advance(dk, kk * 32), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(smem_u32(&ctl->s_full[w]));
      };
      auto issue_o = [&](int w, int stage) {
        const uint64_t dv = make_smem_desc(v_smem + stage * Cfg::kTileBytes, D);
#pragma unroll
        for (int kk = 0; kk < kTile / 32; ++kk)
          mma_i8_ts(tmem_base + 2 * kTile + w * D, tmem_base + w * kTile + kk * 8, desc_advance(dv, kk * 32 * D), idesc_o,
                    kk > 0 ? 1u : 0u);
        mma_commit(smem_u32(&ctl->o_full[w]));
      };
      do {
        if (!mbar_wait(smem_u32(&ctl->q_full), 0u, abort_flag)) { raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_Q_LOAD, 0); ok = false; break; }
        if (!mbar_wait(smem_u32(&ctl->k_full[0]), 0u, abort_flag)) { raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_K_LOAD, 0); ok = false; break; }
        tc_fence_after();
        for (int w = 0; w < nq; ++w) issue_s(w, 0);
        mma_commit(smem_u32(&ctl->k_empty[0]));
        for (int j = 0; j < n_live && ok; ++j) {
          const int s = j % NS;
          const uint32_t ph = static_cast<uint32_t>(j & 1);
          if (!mbar_wait(smem_u32(&ctl->v_full[s]), static_cast<uint32_t>((j / NS) & 1), abort_flag)) {
            raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_V_LOAD, j); ok = false; break;
          }
          const int jn = j + 1, sn = jn % NS;
          for (int w = 0; w < nq; ++w) {
            if (!mbar_wait(smem_u32(&ctl->p_ready[w]), ph, abort_flag)) { raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_P_READY, j); ok = false; break; }
            if (j > 0 && !mbar_wait(smem_u32(&ctl->o_free[w]), ph ^ 1u, abort_flag)) { raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_O_FREE, j); ok = false; break; }
            tc_fence_after();
            issue_o(w, s);
            if (w == nq - 1) mma_commit(smem_u32(&ctl->v_empty[s]));
            if (jn < n_live) {
              if (w == 0 && !mbar_wait(smem_u32(&ctl->k_full[sn]), static_cast<uint32_t>((jn / NS) & 1), abort_flag)) {
                raise_status(abort_flag, p.status, FMHA_I8_DEV_WAIT_K_LOAD, jn); ok = false; break;
              }
              tc_fence_after();
              // S_w / P_w columns are free again: the tensor pipe runs this thread's MMAs in order
              issue_s(w, sn);
              if (w == nq - 1) mma_commit(smem_u32(&ctl->k_empty[sn]));
            }
          }
        }
      } while (false);
    }
  }

  // everything this CTA issued has been consumed by the time the softmax groups leave their loop
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace fmha
