// Debug kernels: each exercises one hardware-facing stage of the forward pass in isolation so that
// descriptor, swizzle and tensor-memory layout mistakes show up as a failed bit-exact comparison on
// the smallest possible surface, plus a CUDA-core restatement of the whole pass used as an
// on-device cross-check at sizes the CPU oracle can only sample.
#pragma once
#include "fmha_fwd_sm100.cuh"

namespace fmha {

struct DebugCtl {
  uint64_t full, done;
  uint32_t tmem_base;
  int abort;
};

// S_int32 tile (qt, kt) of head bh = Q tile . K tile^T  -- GEMM 1 of the forward pass
// (reference: inc/fmha_i8.cuh:120-172).  grid (key tiles, query tiles, heads), 128 threads.
template <int D>
__global__ void __launch_bounds__(128, 1)
debug_qk_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                int32_t* s_out, int S, unsigned* status) {
  constexpr int kTileBytes = kTile * D;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  DebugCtl* ctl = reinterpret_cast<DebugCtl*>(tiles + 2 * kTileBytes);
  const uint32_t q_smem = smem_u32(tiles), k_smem = q_smem + kTileBytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, qt = blockIdx.y, bh = blockIdx.z;
  volatile int* abort_flag = &ctl->abort;

  if (threadIdx.x == 0) {
    ctl->abort = 0;
    mbar_init(smem_u32(&ctl->full), 1);
    mbar_init(smem_u32(&ctl->done), 1);
    mbar_init_fence();
  }
  if (warp == 0) { __syncwarp(); tmem_alloc(smem_u32(&ctl->tmem_base), 128); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);

  if (threadIdx.x == 0) {
    const uint32_t bar = smem_u32(&ctl->full);
    mbar_arrive_expect_tx(bar, 2 * kTileBytes);
    tma_load_3d(q_smem, &map_q, bar, 0, qt * kTile, bh);
    tma_load_3d(k_smem, &map_k, bar, 0, kt * kTile, bh);
    if (mbar_wait(bar, 0u, abort_flag)) {
      tc_fence_after();
      const uint64_t dq = make_smem_desc(q_smem, D), dk = make_smem_desc(k_smem, D);
      constexpr uint32_t idesc = make_idesc_i8(kTile, false);
#pragma unroll
      for (int kk = 0; kk < D / 32; ++kk)
        mma_i8_ss(tmem_base, desc_advance(dq, kk * 32), desc_advance(dk, kk * 32), idesc, kk > 0 ? 1u : 0u);
      mma_commit(smem_u32(&ctl->done));
    } else {
      raise_status(abort_flag, status, FMHA_I8_DEV_WAIT_DEBUG, 0);
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000LL) { }
    }
  }
  const bool ok = __all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&ctl->done), 0u, abort_flag));
  if (ok) {
    tc_fence_after();
    const int row = qt * kTile + warp * 32 + lane;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + c * 32, r);
      if (row < S) {
        int32_t* dst = s_out + (static_cast<int64_t>(bh) * S + row) * S + kt * kTile + c * 32;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (kt * kTile + c * 32 + i < S) dst[i] = static_cast<int32_t>(r[i]);
      }
    }
  } else if (lane == 0) {
    raise_status(abort_flag, status, FMHA_I8_DEV_WAIT_DEBUG, 1);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem_base, 128); }
}

// O_int32 rows of query tile qt = sum over key tiles of P tile . V tile -- GEMM 2 of the forward
// pass (reference: inc/fmha_i8.cuh:255-296), accumulated in tensor memory across all key tiles.
// kFromTmem: P is written to tensor memory by its row's thread (the forward pass's way);
// otherwise P goes through a 128B-swizzled K-major shared-memory tile.
template <int D, bool kFromTmem>
__global__ void __launch_bounds__(128, 1)
debug_pv_kernel(const __grid_constant__ CUtensorMap map_v, const int8_t* p8, int32_t* o_out, int S, unsigned* status) {
  constexpr int kTileBytes = kTile * D;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* p_tile = tiles + kTileBytes;                       // 128 x 128 bytes
  DebugCtl* ctl = reinterpret_cast<DebugCtl*>(tiles + kTileBytes + kTile * kTile);
  const uint32_t v_smem = smem_u32(tiles), p_smem = smem_u32(p_tile);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, bh = blockIdx.y;
  const int row = qt * kTile + threadIdx.x;
  const int n_tiles = (S + kTile - 1) / kTile;
  volatile int* abort_flag = &ctl->abort;

  if (threadIdx.x == 0) {
    ctl->abort = 0;
    mbar_init(smem_u32(&ctl->full), 1);
    mbar_init(smem_u32(&ctl->done), 1);
    mbar_init_fence();
  }
  if (warp == 0) { __syncwarp(); tmem_alloc(smem_u32(&ctl->tmem_base), 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);
  const uint32_t lane_field = static_cast<uint32_t>(warp * 32) << 16;
  bool ok = true;

  for (int j = 0; j < n_tiles && ok; ++j) {
    if (threadIdx.x == 0) {
      mbar_arrive_expect_tx(smem_u32(&ctl->full), kTileBytes);
      tma_load_3d(v_smem, &map_v, smem_u32(&ctl->full), 0, j * kTile, bh);
    }
    // this thread's 128 P values for key tile j (zeros outside the matrix)
    uint4 pr[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      pr[c] = make_uint4(0u, 0u, 0u, 0u);
      if (row < S && j * kTile + c * 16 < S)
        pr[c] = *reinterpret_cast<const uint4*>(p8 + (static_cast<int64_t>(bh) * S + row) * S + j * kTile + c * 16);
    }
    if (kFromTmem) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t words[8] = {pr[2 * c].x, pr[2 * c].y, pr[2 * c].z, pr[2 * c].w,
                                   pr[2 * c + 1].x, pr[2 * c + 1].y, pr[2 * c + 1].z, pr[2 * c + 1].w};
        tmem_st8(tmem_base + lane_field + c * 8, words);
      }
      tmem_wait_st();
    } else {
      const int r = threadIdx.x;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(p_tile + r * 128 + ((c ^ (r & 7)) << 4)) = pr[c];
      fence_proxy_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) {
      if (mbar_wait(smem_u32(&ctl->full), static_cast<uint32_t>(j & 1), abort_flag)) {
        tc_fence_after();
        const uint64_t dv = make_smem_desc(v_smem, D);
        constexpr uint32_t idesc = make_idesc_i8(D, true);
#pragma unroll
        for (int kk = 0; kk < kTile / 32; ++kk) {
          const uint32_t acc = (j > 0 || kk > 0) ? 1u : 0u;
          if (kFromTmem) {
            mma_i8_ts(tmem_base + 128, tmem_base + kk * 8, desc_advance(dv, kk * 32 * D), idesc, acc);
          } else {
            const uint64_t dp = make_smem_desc(p_smem, 128);
            mma_i8_ss(tmem_base + 128, desc_advance(dp, kk * 32), desc_advance(dv, kk * 32 * D), idesc, acc);
          }
        }
        mma_commit(smem_u32(&ctl->done));
      } else {
        raise_status(abort_flag, status, FMHA_I8_DEV_WAIT_DEBUG, 2);
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
      }
    }
    ok = __all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&ctl->done), static_cast<uint32_t>(j & 1), abort_flag));
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    tc_fence_after();
  }
  if (ok) {
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tmem_base + lane_field + 128 + c * 32, r);
      if (row < S) {
        int32_t* dst = o_out + (static_cast<int64_t>(bh) * S + row) * D + c * 32;
#pragma unroll
        for (int i = 0; i < 32; ++i) dst[i] = static_cast<int32_t>(r[i]);
      }
    }
  } else if (threadIdx.x == 0) {
    raise_status(abort_flag, status, FMHA_I8_DEV_WAIT_DEBUG, 3);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

// Exercises the give-up path of the bounded waits without any fault: one warp waits, for at most
// `limit_cycles`, on a barrier that nothing will ever arrive on, records FMHA_I8_DEV_WAIT_DEBUG in the
// status words when the limit is reached and returns normally.  What a host sees afterwards is exactly
// what it would see if a wait of the forward kernel had run out.
__global__ void __launch_bounds__(32) wait_probe_kernel(unsigned* status, long long limit_cycles) {
  __shared__ uint64_t never;
  __shared__ int abort_word;
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(smem_u32(&never), 1);
    mbar_init_fence();
  }
  __syncwarp();
  const bool done = __all_sync(0xFFFFFFFFu, mbar_wait_limited(smem_u32(&never), 0u, &abort_word, limit_cycles));
  if (!done && threadIdx.x == 0) raise_status(&abort_word, status, FMHA_I8_DEV_WAIT_DEBUG, 4);
}

// The whole forward pass on CUDA cores, one thread per query row, in the operation order of the
// reference kernel's arithmetic (inc/fmha_i8.cuh:183-253,298-332): expf, per-tile renormalised
// running output, no fused multiply-add in the merge.  grid (query tiles, heads), 128 threads.
template <int D>
__global__ void __launch_bounds__(128)
simt_check_kernel(const int8_t* __restrict__ q, const int8_t* __restrict__ k, const int8_t* __restrict__ v,
                  const int8_t* __restrict__ mask, int8_t* __restrict__ o, int Sq, int S, int H, int bh_begin,
                  float row_scale, float scale_qk, float scale_v_out, float p_mul, float o_sign) {
  __shared__ __align__(16) int8_t ks[kTile * D];
  __shared__ __align__(16) int8_t vs[kTile * D];
  __shared__ int8_t ms[kTile];
  __shared__ int s_any;
  const int bh = blockIdx.y;
  const int row = blockIdx.x * kTile + threadIdx.x;
  const int batch = (bh_begin + bh) / H;
  const int64_t head_off = static_cast<int64_t>(bh) * S * D;       // keys and values: S rows per head
  const int64_t q_head_off = static_cast<int64_t>(bh) * Sq * D;    // queries and output: Sq rows per head

  int qreg[D / 4];
#pragma unroll
  for (int i = 0; i < D / 4; ++i)
    qreg[i] = (row < Sq) ? reinterpret_cast<const int*>(q + q_head_off + static_cast<int64_t>(row) * D)[i] : 0;

  float oacc[D];
#pragma unroll
  for (int i = 0; i < D; ++i) oacc[i] = 0.f;
  float m_run = -1e6f, l_run = 0.f;
  int s_loc[kTile];

  for (int j0 = 0; j0 < S; j0 += kTile) {
    const int width = min(kTile, S - j0);
    __syncthreads();
    if (threadIdx.x == 0) s_any = 0;
    for (int i = threadIdx.x; i < kTile * D / 16; i += blockDim.x) {
      const int r = (i * 16) / D;
      uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
      if (r < width) {
        kv = reinterpret_cast<const uint4*>(k + head_off + static_cast<int64_t>(j0) * D)[i];
        vv = reinterpret_cast<const uint4*>(v + head_off + static_cast<int64_t>(j0) * D)[i];
      }
      reinterpret_cast<uint4*>(ks)[i] = kv;
      reinterpret_cast<uint4*>(vs)[i] = vv;
    }
    __syncthreads();
    {
      const int c = threadIdx.x;
      const int8_t mv = (c < width) ? mask[static_cast<int64_t>(batch) * S + j0 + c] : static_cast<int8_t>(1);
      ms[c] = mv;
      if (mv == 0) s_any = 1;
    }
    __syncthreads();
    if (!s_any) continue;   // uniform: a key tile without any unmasked key contributes nothing

    float m_t = -INFINITY;
    for (int c = 0; c < kTile; ++c) {
      int acc = 0;
      const int* kr = reinterpret_cast<const int*>(ks + c * D);
#pragma unroll
      for (int i = 0; i < D / 4; ++i) acc = __dp4a(qreg[i], kr[i], acc);
      s_loc[c] = acc;
      const float sf = __fmul_rn(__fmul_rn(row_scale, static_cast<float>(acc)), scale_qk);
      if (ms[c] == 0) m_t = fmaxf(m_t, sf);
    }
    float l_t = 0.f;
    int ot[D];
#pragma unroll
    for (int i = 0; i < D; ++i) ot[i] = 0;
    for (int c = 0; c < kTile; ++c) {
      const float sf = __fmul_rn(__fmul_rn(row_scale, static_cast<float>(s_loc[c])), scale_qk);
      const float pe = (ms[c] != 0) ? 0.f : expf(__fsub_rn(sf, m_t));
      l_t = __fadd_rn(l_t, pe);
      const int p8 = __float2int_rn(fmaxf(fminf(__fmul_rn(p_mul, pe), fmaxf(p_mul, 0.f)), fminf(p_mul, 0.f)));   // -rn(128 p) or rn(255 p)
      if (p8 != 0) {
        const int8_t* vr = vs + c * D;
#pragma unroll
        for (int i = 0; i < D; ++i) ot[i] += p8 * static_cast<int>(vr[i]);
      }
    }
    const float m_new = fmaxf(m_run, m_t);
    const float e_old = expf(__fsub_rn(m_run, m_new));
    const float e_cur = expf(__fsub_rn(m_t, m_new));
    const float l_new = __fadd_rn(__fmul_rn(e_old, l_run), __fmul_rn(e_cur, l_t));
    const float rcp = __frcp_rn(l_new);
    const float a = __fmul_rn(l_run, e_old);
#pragma unroll
    for (int i = 0; i < D; ++i)
      oacc[i] = __fmul_rn(rcp, __fadd_rn(__fmul_rn(a, oacc[i]), __fmul_rn(e_cur, __fmul_rn(o_sign, static_cast<float>(ot[i])))));
    l_run = l_new;
    m_run = m_new;
  }
  if (row < Sq) {
    int8_t* dst = o + q_head_off + static_cast<int64_t>(row) * D;
#pragma unroll
    for (int i = 0; i < D; ++i)
      dst[i] = static_cast<int8_t>(__float2int_rn(fmaxf(fminf(__fmul_rn(scale_v_out, oacc[i]), 127.f), -127.f)));
  }
}

}  // namespace fmha
