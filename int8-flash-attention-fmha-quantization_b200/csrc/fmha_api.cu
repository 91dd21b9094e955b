// Host side of libfmha_i8_sm100.so: argument checks, tensor-map encoding, launches and the C ABI
// declared in include/fmha_i8_c.h.  Replaces the reference project's launcher
// (src/fmha_i8.cu:31-173): one runtime-shaped kernel instead of a table of compile-time shapes.
#include <cuda.h>
#include <cuda_runtime.h>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/fmha_i8_c.h"
#include "fmha_debug_sm100.cuh"
#include "fmha_fwd_sm100.cuh"
#include "fmha_quant_sm100.cuh"

namespace {

using namespace fmha;

__device__ unsigned g_status_words[8];

thread_local int t_last_status = FMHA_I8_OK;
std::atomic<unsigned long long> g_launch_count{0};

int finish(int status) {
  t_last_status = status;
  return status;
}

constexpr int kMaxDevices = 64;

struct DeviceInfo {
  int checked = 0;      // 0 = not yet, 1 = sm_100, -1 = something else
  unsigned* status = nullptr;
  // One word of mapped, pinned host memory per device.  A kernel whose bounded wait runs out writes 1 to
  // it (besides the device status words), so the next host call can see the failure without synchronising.
  volatile unsigned* host_flag = nullptr;
  int sm_count = 0;
  bool attr_set = false;
};
DeviceInfo g_dev[kMaxDevices];
std::mutex g_dev_mutex;

// Returns the per-device record of the current device (compute capability check, address of the
// status words, one-time kernel attributes), or nullptr with *err set.
DeviceInfo* current_device(int* err) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { *err = FMHA_I8_ERR_LAUNCH; return nullptr; }
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  DeviceInfo& d = g_dev[dev];
  if (d.checked == 0) {
    int major = 0, minor = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) {
      *err = FMHA_I8_ERR_LAUNCH;
      return nullptr;
    }
    d.checked = (major == 10 && minor == 0) ? 1 : -1;
    if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || d.sm_count < 1) d.sm_count = 1;
  }
  if (d.checked < 0) { *err = FMHA_I8_ERR_WRONG_ARCH; return nullptr; }
  if (!d.status) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_status_words) != cudaSuccess) { *err = FMHA_I8_ERR_LAUNCH; return nullptr; }
    // the host-visible failure word (set-up only: a few bytes of pinned host memory, nothing on the device)
    void* host_word = nullptr;
    void* dev_view = nullptr;
    if (cudaHostAlloc(&host_word, sizeof(unsigned), cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer(&dev_view, host_word, 0) != cudaSuccess) {
      cudaGetLastError();
      *err = FMHA_I8_ERR_LAUNCH;
      return nullptr;
    }
    *static_cast<volatile unsigned*>(host_word) = 0u;
    if (cudaMemcpyToSymbol(g_host_flag_ptr, &dev_view, sizeof(dev_view)) != cudaSuccess) {
      cudaGetLastError();
      *err = FMHA_I8_ERR_LAUNCH;
      return nullptr;
    }
    d.host_flag = static_cast<volatile unsigned*>(host_word);
    d.status = static_cast<unsigned*>(ptr);
  }
  return &d;
}

template <int D> size_t fwd_smem_bytes() {
  return 1024 + FwdCfg<D>::kTilesBytesTotal + 2 * kBiasBytes + sizeof(FwdCtl<FwdCfg<D>::kStagesK, FwdCfg<D>::kStagesV>);
}
template <int D> size_t qk_smem_bytes() { return 1024 + 2 * kTile * D + sizeof(DebugCtl); }
template <int D> size_t pv_smem_bytes() { return 1024 + kTile * D + kTile * kTile + sizeof(DebugCtl); }

int set_kernel_attributes(DeviceInfo* d) {
  if (d->attr_set) return FMHA_I8_OK;
  cudaError_t e = cudaSuccess;
  auto set = [&](const void* fn, size_t bytes) {
    if (e == cudaSuccess) e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
  };
  set(reinterpret_cast<const void*>(&fmha_fwd_kernel<64, false>), fwd_smem_bytes<64>());
  set(reinterpret_cast<const void*>(&fmha_fwd_kernel<128, false>), fwd_smem_bytes<128>());
  set(reinterpret_cast<const void*>(&fmha_fwd_kernel<64, true>), fwd_smem_bytes<64>());
  set(reinterpret_cast<const void*>(&fmha_fwd_kernel<128, true>), fwd_smem_bytes<128>());
  set(reinterpret_cast<const void*>(&debug_qk_kernel<64>), qk_smem_bytes<64>());
  set(reinterpret_cast<const void*>(&debug_qk_kernel<128>), qk_smem_bytes<128>());
  set(reinterpret_cast<const void*>(&debug_pv_kernel<64, true>), pv_smem_bytes<64>());
  set(reinterpret_cast<const void*>(&debug_pv_kernel<64, false>), pv_smem_bytes<64>());
  set(reinterpret_cast<const void*>(&debug_pv_kernel<128, true>), pv_smem_bytes<128>());
  set(reinterpret_cast<const void*>(&debug_pv_kernel<128, false>), pv_smem_bytes<128>());
  if (e != cudaSuccess) { cudaGetLastError(); return FMHA_I8_ERR_LAUNCH; }
  // The forward kernel redistributes registers with setmaxnreg; that only terminates if the launch
  // allocation is the one the targets were sized for.
  cudaFuncAttributes fa64{}, fa128{}, fp64{}, fp128{};
  if (cudaFuncGetAttributes(&fa64, reinterpret_cast<const void*>(&fmha_fwd_kernel<64, false>)) != cudaSuccess ||
      cudaFuncGetAttributes(&fa128, reinterpret_cast<const void*>(&fmha_fwd_kernel<128, false>)) != cudaSuccess ||
      cudaFuncGetAttributes(&fp64, reinterpret_cast<const void*>(&fmha_fwd_kernel<64, true>)) != cudaSuccess ||
      cudaFuncGetAttributes(&fp128, reinterpret_cast<const void*>(&fmha_fwd_kernel<128, true>)) != cudaSuccess ||
      fa64.numRegs != kLaunchRegs || fa128.numRegs != kLaunchRegs || fp64.numRegs != kLaunchRegs || fp128.numRegs != kLaunchRegs) {
    cudaGetLastError();
    std::fprintf(stderr, "fmha_i8_sm100: forward kernel built with %d/%d registers per thread, expected %d; refusing to launch\n",
                 fa64.numRegs, fa128.numRegs, kLaunchRegs);
    return FMHA_I8_ERR_LAUNCH;
  }
  d->attr_set = true;
  return FMHA_I8_OK;
}

// cuTensorMapEncodeTiled, fetched through the runtime so the library has no link-time libcuda dependency.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// int8 tensor [n_heads, S, D] seen as a 3-D map (D innermost) with boxes of 128 rows of one head.
// Rows past S are zero-filled by the copy engine instead of running into the next head.
int make_map(CUtensorMap* map, const void* base, int n_heads, int S, int D) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return FMHA_I8_ERR_DRIVER;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(n_heads)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(S) * D};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(D), static_cast<cuuint32_t>(kTile), 1u};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  const CUtensorMapSwizzle sw = (D == 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FMHA_I8_OK : FMHA_I8_ERR_DRIVER;
}

bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// Shape as the kernel sees it: Sq query rows and Sk keys per head (equal for the reference's self-attention).
struct Shape {
  int B, Sq, Sk, H, D;
};

int check_shape_x(const Shape& sh) {
  if (sh.B < 1 || sh.H < 1 || sh.Sk < 64 || sh.Sk > kMaxSeq || (sh.Sk % 64) != 0) return FMHA_I8_ERR_BAD_SHAPE;
  if (sh.Sq < 1 || sh.Sq > kMaxSeq) return FMHA_I8_ERR_BAD_SHAPE;
  if (sh.D != 64 && sh.D != 128) return FMHA_I8_ERR_BAD_SHAPE;
  if (static_cast<long long>(sh.B) * sh.H > 0x7FFFFFFFLL / 2) return FMHA_I8_ERR_BAD_SHAPE;
  return FMHA_I8_OK;
}

int check_shape(const int desc[4]) {
  const Shape sh{desc[0], desc[1], desc[1], desc[2], desc[3]};
  return check_shape_x(sh);
}

// The reference evaluates 1/sqrt(head_dim) with a Newton iteration carried in float
// (inc/fmha_i8.cuh:13-34,71); the same recurrence gives the same constant.
float reference_row_scale(int D) {
  const float x = static_cast<float>(D);
  float curr = x, prev = 0.f;
  while (curr != prev) {
    const float next = static_cast<float>(0.5 * (static_cast<double>(curr) + static_cast<double>(x / curr)));
    prev = curr;
    curr = next;
  }
  return 1.0f / curr;
}

int fill_params(FwdParams* p, const float amax[5], int D, unsigned flags = 0u) {
  for (int i = 0; i < 4; ++i)
    if (!(amax[i] > 0.f) || !std::isfinite(amax[i])) return FMHA_I8_ERR_BAD_AMAX;
  const bool up = (flags & FMHA_I8_FLAG_UINT8_P) != 0u;
  p->row_scale = reference_row_scale(D);
  p->scale_qk = amax[0] * amax[1] / (127.f * 127.f);
  p->scale_v_out = amax[2] * (1.0f / (amax[3] * (up ? 255.f : 128.f)));
  p->p_mul = up ? 255.f : -128.f;
  p->o_sign = up ? 1.f : -1.f;
  p->p_unsigned = up ? 1u : 0u;
  p->amax_out = nullptr;
  p->amax_scale = amax[2] / ((up ? 255.f : 128.f) * 127.f);   // O~/l counts P in 1/128 (1/255) and V in v_amax/127
  p->c2 = static_cast<float>(static_cast<double>(p->row_scale) * static_cast<double>(p->scale_qk) * 1.4426950408889634);
  if (!(p->c2 > 0.f) || !std::isfinite(p->c2 * kMagic)) return FMHA_I8_ERR_BAD_AMAX;
  return FMHA_I8_OK;
}

template <int D, bool kPolicy = false>
int launch_fwd(cudaStream_t stream, DeviceInfo* dev, FwdParams p, const void* q, const void* k, const void* v) {
  CUtensorMap mq, mk, mv;
  int st;
  if ((st = make_map(&mq, q, p.bh_count, p.Sq, D)) != FMHA_I8_OK) return st;
  if ((st = make_map(&mk, k, p.bh_count, p.S, D)) != FMHA_I8_OK) return st;
  if ((st = make_map(&mv, v, p.bh_count, p.S, D)) != FMHA_I8_OK) return st;
  // persistent CTAs: one per SM (tensor memory is allocated whole), each walking its share of the units
  const unsigned grid = static_cast<unsigned>(p.n_units < dev->sm_count ? p.n_units : dev->sm_count);
  fmha_fwd_kernel<D, kPolicy><<<grid, kFwdThreads, fwd_smem_bytes<D>(), stream>>>(mq, mk, mv, p);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? FMHA_I8_OK : FMHA_I8_ERR_LAUNCH;
}

// calib == nullptr: the forward pass into o.  calib != nullptr: calibration, o is not touched (may be null).
// Which of the three uses of the forward kernel a launch is.
struct LaunchMode {
  float* calib = nullptr;          // calibration: largest |output| to this device float, o untouched
  float2* stats_out = nullptr;     // statistics launch of a whole-row policy: {row max bits, exp-sum} per query row, o untouched
  const float2* stats_in = nullptr;  // policy launch: those statistics
  int policy = 0;                  // FMHA_I8_POLICY_* of a policy launch
};

int infer_x_impl(void* stream, const float amax[5], const Shape& sh, const void* q, const void* k,
                 const void* v, const void* mask, void* o, int bh_begin, int bh_count, unsigned flags,
                 float* calib = nullptr, const LaunchMode* mode = nullptr) {
  const bool no_output = calib || (mode && mode->stats_out);
  if (!amax || !q || !k || !v || !mask || (!o && !no_output)) return FMHA_I8_ERR_NULL_POINTER;
  if (!(flags & FMHA_I8_FLAG_USE_TCU)) return FMHA_I8_ERR_NO_CUDA_CORE_PATH;
  if (flags & ~(FMHA_I8_FLAG_USE_TCU | FMHA_I8_FLAG_UINT8_P)) return FMHA_I8_ERR_BAD_FLAGS;
  int st = check_shape_x(sh);
  if (st != FMHA_I8_OK) return st;
  const long long BH = static_cast<long long>(sh.B) * sh.H;
  if (bh_begin < 0 || bh_count < 1 || static_cast<long long>(bh_begin) + bh_count > BH) return FMHA_I8_ERR_BAD_SLICE;
  if (!aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16) || !aligned(o, 16) || !aligned(mask, 4) || !aligned(calib, 4))
    return FMHA_I8_ERR_MISALIGNED;
  FwdParams p{};
  if ((st = fill_params(&p, amax, sh.D, flags)) != FMHA_I8_OK) return st;
  p.amax_out = calib;
  const bool policy_launch = mode && mode->stats_in;
  if (mode) {
    p.row_stats_out = mode->stats_out;
    p.row_stats_in = mode->stats_in;
    if (policy_launch) {
      // fmha_i8_quant_deviation.py:7,38-43: 127 levels, unsigned, P8 = clip(rn(p * 127 / p_amax), 0, 127).
      // Per-row ("dynamic", :104-118): p_amax = the row's largest probability = 1/l, so P8 = rn(127 e) and the output
      // is (sum P8 v8) / (127 l) * v_amax/127.  Static (:82-98): p_amax = s_max for every row, so
      // P8 = min(rn(127 e / (l s_max)), 127) and the output is (sum P8 v8) * s_max/127 * v_amax/127.
      const float levels = 127.f;
      if (mode->policy == FMHA_I8_POLICY_STATIC && (!(amax[4] > 0.f) || !std::isfinite(amax[4]))) return FMHA_I8_ERR_BAD_AMAX;
      p.p_levels = levels;
      p.p_row_mul = levels;
      p.p_static_mul = (mode->policy == FMHA_I8_POLICY_STATIC) ? levels / amax[4] : 0.f;
      p.p_mul = levels;
      p.o_sign = 1.f;
      p.p_unsigned = 1u;
      p.scale_v_out = (mode->policy == FMHA_I8_POLICY_STATIC) ? amax[4] * amax[2] / (levels * amax[3]) : amax[2] / (levels * amax[3]);
    }
  }
  int err = FMHA_I8_OK;
  DeviceInfo* dev = current_device(&err);
  if (!dev) return err;
  if ((st = set_kernel_attributes(dev)) != FMHA_I8_OK) return st;
  // A kernel launched earlier gave up on a bounded wait (its output is invalid): say so ONCE, on the first call
  // that can see it, without launching; the details stay in the status words until fmha_i8_sm100_device_status().
  if (*dev->host_flag != 0u) {
    *dev->host_flag = 0u;
    return FMHA_I8_ERR_DEVICE;
  }
  p.mask = static_cast<const int8_t*>(mask);
  p.o = static_cast<int8_t*>(o);
  p.o_wide = aligned(o, 32) ? 1 : 0;
  p.S = sh.Sk;
  p.Sq = sh.Sq;
  p.H = sh.H;
  p.bh_begin = bh_begin;
  p.bh_count = bh_count;
  p.q_tiles = (p.Sq + kTile - 1) / kTile;
  {
    const long long units = static_cast<long long>(bh_count) * p.q_tiles;
    if (units > 0x7FFFFFFFLL) return FMHA_I8_ERR_BAD_SHAPE;
    p.n_units = static_cast<int>(units);
  }
  p.status = dev->status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (policy_launch) return sh.D == 128 ? launch_fwd<128, true>(s, dev, p, q, k, v) : launch_fwd<64, true>(s, dev, p, q, k, v);
  return sh.D == 128 ? launch_fwd<128>(s, dev, p, q, k, v) : launch_fwd<64>(s, dev, p, q, k, v);
}

int infer_slice_impl(void* stream, const float amax[5], const int desc[4], const void* q, const void* k,
                     const void* v, const void* mask, void* o, int bh_begin, int bh_count, unsigned flags) {
  if (!desc) return FMHA_I8_ERR_NULL_POINTER;
  const Shape sh{desc[0], desc[1], desc[1], desc[2], desc[3]};
  return infer_x_impl(stream, amax, sh, q, k, v, mask, o, bh_begin, bh_count, flags);
}

// Device staging buffers of fmha_i8_sm100_infer_host, one set per device, grown on demand, plus the
// three streams and the events of its copy/compute pipeline.
constexpr int kHostChunks = 8;
struct HostStaging {
  void* q = nullptr; void* k = nullptr; void* v = nullptr; void* o = nullptr; void* mask = nullptr;
  size_t tensor_cap = 0, mask_cap = 0;
  cudaStream_t s_in = nullptr, s_run = nullptr, s_out = nullptr;
  cudaEvent_t landed[kHostChunks] = {}, computed[kHostChunks] = {};
  bool ready = false;
};
HostStaging g_staging[kMaxDevices];
std::mutex g_staging_mutex[kMaxDevices];     // one lock per device: host threads that drive different GPUs do not wait for each other

// Scratch of fmha_i8_sm100_quantize_f32 (partial maxima), one buffer per device, grown on demand.
struct QuantScratch {
  float* partial = nullptr;
  long long capacity_chunks = 0;
};
QuantScratch g_quant_scratch[kMaxDevices];
std::mutex g_quant_mutex;

int check_quant_args(const float* x, long long n, const int8_t* out) {
  if (!x || !out) return FMHA_I8_ERR_NULL_POINTER;
  if (n < 1) return FMHA_I8_ERR_BAD_SHAPE;
  if (!aligned(x, 16) || !aligned(out, 16)) return FMHA_I8_ERR_MISALIGNED;
  return FMHA_I8_OK;
}

// Scratch of fmha_i8_sm100_quantize_f32_noalloc: the partial maxima live in the library's own device
// image instead of the heap.  Every GPU that loads the library carries these 16 KB until the process
// exits.  4096 chunks x 65536 elements = 268,435,456 elements (1 GiB of fp32) is the largest tensor
// the entry point accepts.
constexpr long long kNoAllocMaxChunks = 4096;
static __device__ __align__(256) float g_quant_partial_static[kNoAllocMaxChunks];
float* g_quant_static_ptr[kMaxDevices];      // device address of the array above, per device (0 = not looked up yet)
std::mutex g_quant_static_mutex;

int launch_quantize(cudaStream_t stream, const float* x, long long n, int8_t* out, float* amax_out, float* partial, long long n_chunks) {
  quant_absmax_kernel<<<static_cast<unsigned>(n_chunks), kQuantThreads, 0, stream>>>(x, n, partial);
  quant_apply_kernel<<<static_cast<unsigned>(n_chunks), kQuantThreads, 0, stream>>>(x, n, partial, static_cast<int>(n_chunks), out, amax_out);
  g_launch_count.fetch_add(2, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? FMHA_I8_OK : FMHA_I8_ERR_LAUNCH;
}

}  // namespace

extern "C" {

int fmha_i8_sm100_infer(void* stream, const float amax[5], const int desc[4], const void* q, const void* k,
                        const void* v, const void* mask, void* o, unsigned flags) {
  if (!desc) return finish(FMHA_I8_ERR_NULL_POINTER);
  const long long BH = static_cast<long long>(desc[0]) * desc[2];
  if (BH < 1 || BH > 0x7FFFFFFFLL) return finish(FMHA_I8_ERR_BAD_SHAPE);
  return finish(infer_slice_impl(stream, amax, desc, q, k, v, mask, o, 0, static_cast<int>(BH), flags));
}

int fmha_i8_sm100_infer_slice(void* stream, const float amax[5], const int desc[4], const void* q, const void* k,
                              const void* v, const void* mask, void* o, int bh_begin, int bh_count, unsigned flags) {
  return finish(infer_slice_impl(stream, amax, desc, q, k, v, mask, o, bh_begin, bh_count, flags));
}

int fmha_i8_sm100_infer_cross(void* stream, const float amax[5], const int desc5[5], const void* q, const void* k,
                              const void* v, const void* mask, void* o, int bh_begin, int bh_count, unsigned flags) {
  if (!desc5) return finish(FMHA_I8_ERR_NULL_POINTER);
  const Shape sh{desc5[0], desc5[1], desc5[2], desc5[3], desc5[4]};
  return finish(infer_x_impl(stream, amax, sh, q, k, v, mask, o, bh_begin, bh_count, flags));
}

int fmha_i8_sm100_infer_policy(void* stream, const float amax[5], const int desc5[5], const void* q, const void* k,
                               const void* v, const void* mask, void* o, int bh_begin, int bh_count, unsigned flags,
                               int policy, float* row_scratch) {
  if (!desc5) return finish(FMHA_I8_ERR_NULL_POINTER);
  const Shape sh{desc5[0], desc5[1], desc5[2], desc5[3], desc5[4]};
  if (policy == FMHA_I8_POLICY_TILE) return finish(infer_x_impl(stream, amax, sh, q, k, v, mask, o, bh_begin, bh_count, flags));
  if (policy != FMHA_I8_POLICY_ROW && policy != FMHA_I8_POLICY_STATIC) return finish(FMHA_I8_ERR_BAD_FLAGS);
  if (flags & FMHA_I8_FLAG_UINT8_P) return finish(FMHA_I8_ERR_BAD_FLAGS);       // the policies bring their own P format
  if (!row_scratch || !o) return finish(FMHA_I8_ERR_NULL_POINTER);
  if (!aligned(row_scratch, 8)) return finish(FMHA_I8_ERR_MISALIGNED);
  // launch 1: the forward pass with the reference's tile-local arithmetic, keeping only each row's maximum and exp-sum
  LaunchMode stats;
  stats.stats_out = reinterpret_cast<float2*>(row_scratch);
  int st = infer_x_impl(stream, amax, sh, q, k, v, mask, nullptr, bh_begin, bh_count, flags, nullptr, &stats);
  if (st != FMHA_I8_OK) return finish(st);
  // launch 2 (same stream, so ordered behind launch 1): every tile of a row quantised with the row's one scale
  LaunchMode apply;
  apply.stats_in = reinterpret_cast<const float2*>(row_scratch);
  apply.policy = policy;
  return finish(infer_x_impl(stream, amax, sh, q, k, v, mask, o, bh_begin, bh_count, flags, nullptr, &apply));
}

int fmha_i8_sm100_calibrate_o_amax(void* stream, const float amax[5], const int desc5[5], const void* q, const void* k,
                                   const void* v, const void* mask, float* o_amax_out, unsigned flags) {
  if (!desc5 || !amax || !o_amax_out) return finish(FMHA_I8_ERR_NULL_POINTER);
  const Shape sh{desc5[0], desc5[1], desc5[2], desc5[3], desc5[4]};
  const long long BH = static_cast<long long>(sh.B) * sh.H;
  if (BH < 1 || BH > 0x7FFFFFFFLL) return finish(FMHA_I8_ERR_BAD_SHAPE);
  // o_amax is what is being determined: any positive placeholder passes the argument check
  const float a[5] = {amax[0], amax[1], amax[2], 1.0f, 1.0f};
  if (cudaMemsetAsync(o_amax_out, 0, sizeof(float), static_cast<cudaStream_t>(stream)) != cudaSuccess) {
    cudaGetLastError();
    return finish(FMHA_I8_ERR_LAUNCH);
  }
  return finish(infer_x_impl(stream, a, sh, q, k, v, mask, nullptr, 0, static_cast<int>(BH), flags, o_amax_out));
}

// Host buffers in, host buffer out, for heads [bh_begin, bh_begin + bh_count): host_q/k/v/o point at the first head
// of the slice, host_mask is the whole [B,S] mask.
static int infer_host_slice_impl(const float amax[5], const int desc[4], const void* host_q, const void* host_k,
                                 const void* host_v, const void* host_mask, void* host_o, int bh_begin, int bh_count, unsigned flags) {
  if (!amax || !desc || !host_q || !host_k || !host_v || !host_mask || !host_o) return FMHA_I8_ERR_NULL_POINTER;
  int st = check_shape(desc);
  if (st != FMHA_I8_OK) return st;
  const long long BH_all = static_cast<long long>(desc[0]) * desc[2];
  if (bh_begin < 0 || bh_count < 1 || static_cast<long long>(bh_begin) + bh_count > BH_all) return FMHA_I8_ERR_BAD_SLICE;
  int dev_id = 0;
  if (cudaGetDevice(&dev_id) != cudaSuccess || dev_id < 0 || dev_id >= kMaxDevices) return FMHA_I8_ERR_LAUNCH;
  const size_t head_bytes = static_cast<size_t>(desc[1]) * desc[3];
  const size_t tensor_bytes = static_cast<size_t>(bh_count) * head_bytes;
  const size_t mask_bytes = static_cast<size_t>(desc[0]) * desc[1];
  std::lock_guard<std::mutex> lock(g_staging_mutex[dev_id]);
  HostStaging& s = g_staging[dev_id];
  if (!s.ready) {
    bool good = cudaStreamCreateWithFlags(&s.s_in, cudaStreamNonBlocking) == cudaSuccess &&
                cudaStreamCreateWithFlags(&s.s_run, cudaStreamNonBlocking) == cudaSuccess &&
                cudaStreamCreateWithFlags(&s.s_out, cudaStreamNonBlocking) == cudaSuccess;
    for (int i = 0; i < kHostChunks && good; ++i)
      good = cudaEventCreateWithFlags(&s.landed[i], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&s.computed[i], cudaEventDisableTiming) == cudaSuccess;
    if (!good) { cudaGetLastError(); return FMHA_I8_ERR_LAUNCH; }
    s.ready = true;
  }
  if (s.tensor_cap < tensor_bytes) {
    cudaFree(s.q); cudaFree(s.k); cudaFree(s.v); cudaFree(s.o);
    s.q = s.k = s.v = s.o = nullptr;
    s.tensor_cap = 0;
    if (cudaMalloc(&s.q, tensor_bytes) != cudaSuccess || cudaMalloc(&s.k, tensor_bytes) != cudaSuccess ||
        cudaMalloc(&s.v, tensor_bytes) != cudaSuccess || cudaMalloc(&s.o, tensor_bytes) != cudaSuccess) {
      cudaGetLastError();
      return FMHA_I8_ERR_LAUNCH;
    }
    s.tensor_cap = tensor_bytes;
  }
  if (s.mask_cap < mask_bytes) {
    cudaFree(s.mask);
    s.mask = nullptr;
    s.mask_cap = 0;
    if (cudaMalloc(&s.mask, mask_bytes) != cudaSuccess) { cudaGetLastError(); return FMHA_I8_ERR_LAUNCH; }
    s.mask_cap = mask_bytes;
  }
  // Pipeline over contiguous ranges of heads: while chunk i is computed, chunk i+1 is on its way in and
  // chunk i-1 on its way out (the bus is full duplex).  Each chunk is one forward launch on a sub-slice.
  const int BH = bh_count;
  const int n_chunks = BH < kHostChunks ? BH : kHostChunks;
  // The inbound copies are the bottleneck, so what follows the last of them -- the last chunk's kernel and its
  // outbound copy -- is exposed: with enough heads the last chunk is made small (1/24 of the heads) and the
  // others share the rest equally.
  int bounds[kHostChunks + 1];
  {
    const int tail = (BH >= 8 * kHostChunks) ? (BH / 24 > 0 ? BH / 24 : 1) : 0;      // 0: equal chunks
    const int body = BH - tail, n_body = tail ? n_chunks - 1 : n_chunks;
    for (int i = 0; i <= n_body; ++i) bounds[i] = static_cast<int>(static_cast<long long>(body) * i / n_body);
    if (tail) bounds[n_chunks] = BH;
  }
  cudaError_t e = cudaMemcpyAsync(s.mask, host_mask, mask_bytes, cudaMemcpyHostToDevice, s.s_in);
  for (int i = 0; i < n_chunks && e == cudaSuccess; ++i) {
    const int begin = bounds[i];
    const int end = bounds[i + 1];
    const size_t off = begin * head_bytes, bytes = (end - begin) * head_bytes;
    const char* hq = static_cast<const char*>(host_q) + off;
    const char* hk = static_cast<const char*>(host_k) + off;
    const char* hv = static_cast<const char*>(host_v) + off;
    char* dq = static_cast<char*>(s.q) + off;
    char* dk = static_cast<char*>(s.k) + off;
    char* dv = static_cast<char*>(s.v) + off;
    char* dout = static_cast<char*>(s.o) + off;
    e = cudaMemcpyAsync(dq, hq, bytes, cudaMemcpyHostToDevice, s.s_in);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dk, hk, bytes, cudaMemcpyHostToDevice, s.s_in);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dv, hv, bytes, cudaMemcpyHostToDevice, s.s_in);
    if (e == cudaSuccess) e = cudaEventRecord(s.landed[i], s.s_in);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(s.s_run, s.landed[i], 0);
    if (e != cudaSuccess) break;
    st = infer_slice_impl(s.s_run, amax, desc, dq, dk, dv, s.mask, dout, bh_begin + begin, end - begin, flags);
    if (st != FMHA_I8_OK) break;
    e = cudaEventRecord(s.computed[i], s.s_run);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(s.s_out, s.computed[i], 0);
    if (e == cudaSuccess) e = cudaMemcpyAsync(static_cast<char*>(host_o) + off, dout, bytes, cudaMemcpyDeviceToHost, s.s_out);
  }
  // drain all three streams whatever happened, so the staging buffers are idle when the lock is released
  const cudaError_t e1 = cudaStreamSynchronize(s.s_in), e2 = cudaStreamSynchronize(s.s_run), e3 = cudaStreamSynchronize(s.s_out);
  if (st != FMHA_I8_OK) return st;
  if (e != cudaSuccess || e1 != cudaSuccess || e2 != cudaSuccess || e3 != cudaSuccess) { cudaGetLastError(); return FMHA_I8_ERR_LAUNCH; }
  return FMHA_I8_OK;
}

int fmha_i8_sm100_infer_host(const float amax[5], const int desc[4], const void* host_q, const void* host_k,
                             const void* host_v, const void* host_mask, void* host_o, unsigned flags) {
  if (!desc) return finish(FMHA_I8_ERR_NULL_POINTER);
  const long long BH = static_cast<long long>(desc[0]) * desc[2];
  if (BH < 1 || BH > 0x7FFFFFFFLL) return finish(FMHA_I8_ERR_BAD_SHAPE);
  return finish(infer_host_slice_impl(amax, desc, host_q, host_k, host_v, host_mask, host_o, 0, static_cast<int>(BH), flags));
}

int fmha_i8_sm100_infer_host_slice(const float amax[5], const int desc[4], const void* host_q, const void* host_k,
                                   const void* host_v, const void* host_mask, void* host_o, int bh_begin, int bh_count,
                                   unsigned flags) {
  return finish(infer_host_slice_impl(amax, desc, host_q, host_k, host_v, host_mask, host_o, bh_begin, bh_count, flags));
}

int fmha_i8_sm100_debug_qk(void* stream, const int desc[4], const void* q, const void* k, int32_t* s_out) {
  if (!desc || !q || !k || !s_out) return finish(FMHA_I8_ERR_NULL_POINTER);
  int st = check_shape(desc);
  if (st != FMHA_I8_OK) return finish(st);
  if (!aligned(q, 16) || !aligned(k, 16) || !aligned(s_out, 4)) return finish(FMHA_I8_ERR_MISALIGNED);
  int err = FMHA_I8_OK;
  DeviceInfo* dev = current_device(&err);
  if (!dev) return finish(err);
  if ((st = set_kernel_attributes(dev)) != FMHA_I8_OK) return finish(st);
  const int BH = desc[0] * desc[2], S = desc[1], D = desc[3];
  if (BH > 65535) return finish(FMHA_I8_ERR_TOO_LARGE);
  CUtensorMap mq, mk;
  if ((st = make_map(&mq, q, BH, S, D)) != FMHA_I8_OK) return finish(st);
  if ((st = make_map(&mk, k, BH, S, D)) != FMHA_I8_OK) return finish(st);
  const int nt = (S + kTile - 1) / kTile;
  const dim3 grid(nt, nt, BH);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (D == 128) debug_qk_kernel<128><<<grid, 128, qk_smem_bytes<128>(), s>>>(mq, mk, s_out, S, dev->status);
  else debug_qk_kernel<64><<<grid, 128, qk_smem_bytes<64>(), s>>>(mq, mk, s_out, S, dev->status);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return finish(cudaGetLastError() == cudaSuccess ? FMHA_I8_OK : FMHA_I8_ERR_LAUNCH);
}

int fmha_i8_sm100_debug_pv(void* stream, const int desc[4], const void* p, const void* v, int32_t* o_out,
                           unsigned variant) {
  if (!desc || !p || !v || !o_out) return finish(FMHA_I8_ERR_NULL_POINTER);
  int st = check_shape(desc);
  if (st != FMHA_I8_OK) return finish(st);
  if (!aligned(p, 16) || !aligned(v, 16) || !aligned(o_out, 4)) return finish(FMHA_I8_ERR_MISALIGNED);
  if (variant > 1) return finish(FMHA_I8_ERR_BAD_SHAPE);
  int err = FMHA_I8_OK;
  DeviceInfo* dev = current_device(&err);
  if (!dev) return finish(err);
  if ((st = set_kernel_attributes(dev)) != FMHA_I8_OK) return finish(st);
  const int BH = desc[0] * desc[2], S = desc[1], D = desc[3];
  if (BH > 65535) return finish(FMHA_I8_ERR_TOO_LARGE);
  CUtensorMap mv;
  if ((st = make_map(&mv, v, BH, S, D)) != FMHA_I8_OK) return finish(st);
  const dim3 grid((S + kTile - 1) / kTile, BH);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int8_t* p8 = static_cast<const int8_t*>(p);
  if (D == 128) {
    if (variant == 0) debug_pv_kernel<128, true><<<grid, 128, pv_smem_bytes<128>(), s>>>(mv, p8, o_out, S, dev->status);
    else debug_pv_kernel<128, false><<<grid, 128, pv_smem_bytes<128>(), s>>>(mv, p8, o_out, S, dev->status);
  } else {
    if (variant == 0) debug_pv_kernel<64, true><<<grid, 128, pv_smem_bytes<64>(), s>>>(mv, p8, o_out, S, dev->status);
    else debug_pv_kernel<64, false><<<grid, 128, pv_smem_bytes<64>(), s>>>(mv, p8, o_out, S, dev->status);
  }
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return finish(cudaGetLastError() == cudaSuccess ? FMHA_I8_OK : FMHA_I8_ERR_LAUNCH);
}

int fmha_i8_sm100_debug_simt_x(void* stream, const float amax[5], const int desc5[5], const void* q, const void* k,
                               const void* v, const void* mask, void* o, unsigned flags) {
  if (!amax || !desc5 || !q || !k || !v || !mask || !o) return finish(FMHA_I8_ERR_NULL_POINTER);
  const Shape sh{desc5[0], desc5[1], desc5[2], desc5[3], desc5[4]};
  int st = check_shape_x(sh);
  if (st != FMHA_I8_OK) return finish(st);
  if (!aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16) || !aligned(o, 16)) return finish(FMHA_I8_ERR_MISALIGNED);
  FwdParams p{};
  if ((st = fill_params(&p, amax, sh.D, flags)) != FMHA_I8_OK) return finish(st);
  int err = FMHA_I8_OK;
  if (!current_device(&err)) return finish(err);
  const long long BH = static_cast<long long>(sh.B) * sh.H;
  if (BH > 65535) return finish(FMHA_I8_ERR_TOO_LARGE);
  const dim3 grid((sh.Sq + kTile - 1) / kTile, static_cast<unsigned>(BH));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int8_t* q8 = static_cast<const int8_t*>(q);
  const int8_t* k8 = static_cast<const int8_t*>(k);
  const int8_t* v8 = static_cast<const int8_t*>(v);
  const int8_t* m8 = static_cast<const int8_t*>(mask);
  int8_t* o8 = static_cast<int8_t*>(o);
  if (sh.D == 128)
    simt_check_kernel<128><<<grid, 128, 0, s>>>(q8, k8, v8, m8, o8, sh.Sq, sh.Sk, sh.H, 0, p.row_scale, p.scale_qk, p.scale_v_out, p.p_mul, p.o_sign);
  else
    simt_check_kernel<64><<<grid, 128, 0, s>>>(q8, k8, v8, m8, o8, sh.Sq, sh.Sk, sh.H, 0, p.row_scale, p.scale_qk, p.scale_v_out, p.p_mul, p.o_sign);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return finish(cudaGetLastError() == cudaSuccess ? FMHA_I8_OK : FMHA_I8_ERR_LAUNCH);
}

int fmha_i8_sm100_debug_simt(void* stream, const float amax[5], const int desc[4], const void* q, const void* k,
                             const void* v, const void* mask, void* o) {
  if (!desc) return finish(FMHA_I8_ERR_NULL_POINTER);
  const int desc5[5] = {desc[0], desc[1], desc[1], desc[2], desc[3]};
  return fmha_i8_sm100_debug_simt_x(stream, amax, desc5, q, k, v, mask, o, 0u);
}

int fmha_i8_sm100_debug_wait_probe(void* stream, long long limit_cycles) {
  if (limit_cycles < 1000 || limit_cycles > kWaitLimitCycles) return finish(FMHA_I8_ERR_TOO_LARGE);
  int err = FMHA_I8_OK;
  DeviceInfo* dev = current_device(&err);
  if (!dev) return finish(err);
  wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(dev->status, limit_cycles);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return finish(cudaGetLastError() == cudaSuccess ? FMHA_I8_OK : FMHA_I8_ERR_LAUNCH);
}

int fmha_i8_sm100_quantize_f32(void* stream, const float* x, long long n, int8_t* out, float* amax_out) {
  int st = check_quant_args(x, n, out);
  if (st != FMHA_I8_OK) return finish(st);
  int err = FMHA_I8_OK;
  if (!current_device(&err)) return finish(err);
  int dev_id = 0;
  cudaGetDevice(&dev_id);
  const long long n_chunks = (n + kQuantChunk - 1) / kQuantChunk;
  if (n_chunks > 0x7FFFFFFFLL) return finish(FMHA_I8_ERR_TOO_LARGE);
  // The lock is held until the kernels are enqueued: another host thread that has to grow the scratch
  // synchronises the device before it frees the old buffer, and that only covers work already enqueued.
  std::lock_guard<std::mutex> lock(g_quant_mutex);
  QuantScratch& q = g_quant_scratch[dev_id];
  if (q.capacity_chunks < n_chunks) {
    // growing frees the old buffer: wait for work that may still read it
    if (q.partial) { cudaDeviceSynchronize(); cudaFree(q.partial); q.partial = nullptr; q.capacity_chunks = 0; }
    const long long cap = n_chunks < 4096 ? 4096 : n_chunks;
    if (cudaMalloc(&q.partial, sizeof(float) * cap) != cudaSuccess) { cudaGetLastError(); return finish(FMHA_I8_ERR_LAUNCH); }
    q.capacity_chunks = cap;
  }
  return finish(launch_quantize(static_cast<cudaStream_t>(stream), x, n, out, amax_out, q.partial, n_chunks));
}

int fmha_i8_sm100_quantize_f32_noalloc(void* stream, const float* x, long long n, int8_t* out, float* amax_out) {
  int st = check_quant_args(x, n, out);
  if (st != FMHA_I8_OK) return finish(st);
  const long long n_chunks = (n + kQuantChunk - 1) / kQuantChunk;
  if (n_chunks > kNoAllocMaxChunks) {
    std::fprintf(stderr, "fmha_i8_sm100_quantize_f32_noalloc: %lld elements exceed the built-in scratch (at most %lld)\n", n,
                 kNoAllocMaxChunks * kQuantChunk);
    return finish(FMHA_I8_ERR_TOO_LARGE);
  }
  int err = FMHA_I8_OK;
  if (!current_device(&err)) return finish(err);
  int dev_id = 0;
  if (cudaGetDevice(&dev_id) != cudaSuccess || dev_id < 0 || dev_id >= kMaxDevices) return finish(FMHA_I8_ERR_LAUNCH);
  float* partial = nullptr;
  {
    // One-time set-up per device, done by the first call on that device with the device current:
    // in host code the array's name is only a handle, the kernels need its device address.
    std::lock_guard<std::mutex> lock(g_quant_static_mutex);
    if (!g_quant_static_ptr[dev_id]) {
      float* ptr = nullptr;
      if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_quant_partial_static) != cudaSuccess || !ptr) {
        cudaGetLastError();
        return finish(FMHA_I8_ERR_LAUNCH);
      }
      g_quant_static_ptr[dev_id] = ptr;
    }
    partial = g_quant_static_ptr[dev_id];
  }
  // Nothing in the scratch has to start at zero: pass 1 overwrites every slot that pass 2 reads
  // (slots [0, n_chunks)); what an earlier, larger call left beyond them is never looked at.
  return finish(launch_quantize(static_cast<cudaStream_t>(stream), x, n, out, amax_out, partial, n_chunks));
}

int fmha_i8_sm100_device_status(unsigned words[8]) {
  if (!words) return finish(FMHA_I8_ERR_NULL_POINTER);
  if (cudaDeviceSynchronize() != cudaSuccess) { return finish(FMHA_I8_ERR_LAUNCH); }
  if (cudaMemcpyFromSymbol(words, g_status_words, sizeof(unsigned) * 8) != cudaSuccess) return finish(FMHA_I8_ERR_LAUNCH);
  const unsigned zeros[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (cudaMemcpyToSymbol(g_status_words, zeros, sizeof zeros) != cudaSuccess) return finish(FMHA_I8_ERR_LAUNCH);
  {
    int dev_id = 0;
    if (cudaGetDevice(&dev_id) == cudaSuccess && dev_id >= 0 && dev_id < kMaxDevices) {
      std::lock_guard<std::mutex> lock(g_dev_mutex);
      if (g_dev[dev_id].host_flag) *g_dev[dev_id].host_flag = 0u;
    }
  }
  return finish(words[0] == 0u ? FMHA_I8_OK : FMHA_I8_ERR_DEVICE);
}

int fmha_i8_sm100_last_status(void) { return t_last_status; }

const char* fmha_i8_sm100_status_string(int status) {
  switch (status) {
    case FMHA_I8_OK: return "ok";
    case FMHA_I8_ERR_NULL_POINTER: return "a required pointer is NULL";
    case FMHA_I8_ERR_BAD_SHAPE: return "unsupported shape (head_dim must be 64 or 128, seq_len a multiple of 64 up to 32768)";
    case FMHA_I8_ERR_MISALIGNED: return "q/k/v/o must be 16-byte aligned and the mask 4-byte aligned";
    case FMHA_I8_ERR_NO_CUDA_CORE_PATH: return "use_tcu == false is not supported (the reference's CUDA-core kernel is an empty stub)";
    case FMHA_I8_ERR_WRONG_ARCH: return "the current device is not compute capability 10.0 (B200)";
    case FMHA_I8_ERR_LAUNCH: return "the CUDA runtime reported an error";
    case FMHA_I8_ERR_DRIVER: return "tensor-map encoding failed";
    case FMHA_I8_ERR_BAD_SLICE: return "bh_begin/bh_count outside the batch*head range";
    case FMHA_I8_ERR_BAD_AMAX: return "amax values must be finite and positive";
    case FMHA_I8_ERR_TOO_LARGE: return "size beyond the maximum of this entry point";
    case FMHA_I8_ERR_DEVICE: return "a device-side bounded wait ran out (see fmha_i8_sm100_device_status)";
    case FMHA_I8_ERR_BAD_FLAGS: return "an undefined flag bit is set";
    default: return "unknown status";
  }
}

unsigned long long fmha_i8_sm100_launch_count(void) { return g_launch_count.load(std::memory_order_relaxed); }

int fmha_i8_sm100_version(void) { return 100; }

#ifdef FMHA_TRACE
// Performance-work builds only: copies out the timeline stamps of the first CTA.
int fmha_i8_sm100_read_trace(long long* out) {
  if (cudaDeviceSynchronize() != cudaSuccess) return FMHA_I8_ERR_LAUNCH;
  return cudaMemcpyFromSymbol(out, fmha::g_trace, sizeof(long long) * 48 * 512) == cudaSuccess ? FMHA_I8_OK : FMHA_I8_ERR_LAUNCH;
}
#endif

}  // extern "C"

// The reference project's C++ entry point (inc/fmha_i8.h:5-17), kept symbol-for-symbol.
#include "../../include/fmha_i8.h"
namespace gpuImpl {
void FMHAInferI8(cudaStream_t stream, FMHAParamI8 fmha_param, AttnDataDescriptor attn_desc, const void* q,
                 const void* k, const void* v, const void* padding_mask, void* o, const bool use_tcu) {
  const float amax[5] = {fmha_param.q_amax, fmha_param.k_amax, fmha_param.v_amax, fmha_param.o_amax, fmha_param.s_max};
  const int desc[4] = {attn_desc.batch_num, attn_desc.seq_len, attn_desc.head_num, attn_desc.head_dim};
  const int st = fmha_i8_sm100_infer(stream, amax, desc, q, k, v, padding_mask, o, use_tcu ? FMHA_I8_FLAG_USE_TCU : 0u);
  if (st != FMHA_I8_OK) std::fprintf(stderr, "gpuImpl::FMHAInferI8: %s (status %d)\n", fmha_i8_sm100_status_string(st), st);
}
}  // namespace gpuImpl
