/* C ABI of libfmha_i8_sm100.so: the INT8 flash-attention forward pass for NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only, so the library can be bound from any language.  The C++ symbol
 * gpuImpl::FMHAInferI8 (include/fmha_i8.h) is a thin shim over fmha_i8_sm100_infer.
 *
 * Conventions shared by every entry point
 *   amax[5] = {q_amax, k_amax, v_amax, o_amax, s_max}   -- FMHAParamI8, inc/fmha_param_i8.h:10-17
 *   desc[4] = {batch_num, seq_len, head_num, head_dim}  -- AttnDataDescriptor, inc/fmha_param_i8.h:3-8
 *   q,k,v,o : int8 [B,H,S,D] contiguous, 16-byte aligned (an o that is 32-byte aligned, as every cudaMalloc'ed
 *             buffer is, lets the kernel use wider stores: same bytes, about 1 % faster);  mask : int8 [B,S], 4-byte aligned,
 *             non-zero byte = key masked out (inc/cpuSoftmax.hpp:24, inc/fmha_i8.cuh:189-192)
 *   stream  : a cudaStream_t passed as void* (NULL = default stream)
 *   return  : FMHA_I8_OK or a negative FMHA_I8_ERR_* decided on the host before anything is
 *             launched.  Device-side trouble (a bounded wait that ran out in a kernel launched
 *             earlier) is reported in two ways: the details through fmha_i8_sm100_device_status(),
 *             and -- for callers of the void C++ entry point, who never ask -- ONCE as
 *             FMHA_I8_ERR_DEVICE by the first forward call made after the failing kernel has
 *             finished; that call launches nothing, the next one runs again.  The kernels
 *             themselves never look at the status words: one failure does not switch the
 *             library off.
 * All device-pointer entry points enqueue on the stream and return without synchronising.
 */
#ifndef FMHA_I8_C_H_
#define FMHA_I8_C_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  FMHA_I8_OK = 0,
  FMHA_I8_ERR_NULL_POINTER = -1,   /* a required pointer is NULL */
  FMHA_I8_ERR_BAD_SHAPE = -2,      /* head_dim not in {64,128}, seq_len not a multiple of 64 or > 32768, B/H < 1 */
  FMHA_I8_ERR_MISALIGNED = -3,     /* q/k/v/o not 16-byte aligned or mask not 4-byte aligned */
  FMHA_I8_ERR_NO_CUDA_CORE_PATH = -4, /* use_tcu == false: the reference's CUDA-core kernel is an empty stub */
  FMHA_I8_ERR_WRONG_ARCH = -5,     /* current device is not compute capability 10.0 */
  FMHA_I8_ERR_LAUNCH = -6,         /* the CUDA runtime rejected the launch or a copy */
  FMHA_I8_ERR_DRIVER = -7,         /* tensor-map encoding failed or the driver entry point is missing */
  FMHA_I8_ERR_BAD_SLICE = -8,      /* bh_begin/bh_count outside [0, B*H] */
  FMHA_I8_ERR_BAD_AMAX = -9,       /* an amax is not a finite positive number */
  FMHA_I8_ERR_TOO_LARGE = -10,     /* size beyond a stated maximum of the entry point */
  FMHA_I8_ERR_DEVICE = -11,        /* the device status words are non-zero (see device_status) */
  FMHA_I8_ERR_BAD_FLAGS = -12      /* a flag bit this library does not define is set */
};

/* words[0] of fmha_i8_sm100_device_status(): the bounded wait that ran out first. */
enum {
  FMHA_I8_DEV_OK = 0,
  FMHA_I8_DEV_WAIT_Q_LOAD = 1,     /* MMA issuer waiting for the Q tiles */
  FMHA_I8_DEV_WAIT_K_LOAD = 2,     /* MMA issuer waiting for a K stage */
  FMHA_I8_DEV_WAIT_V_LOAD = 3,     /* MMA issuer waiting for a V stage */
  FMHA_I8_DEV_WAIT_K_FREE = 4,     /* loader waiting for a K stage to be released */
  FMHA_I8_DEV_WAIT_V_FREE = 5,     /* loader waiting for a V stage to be released */
  FMHA_I8_DEV_WAIT_S_READY = 6,    /* softmax waiting for S = Q.K^T */
  FMHA_I8_DEV_WAIT_P_READY = 7,    /* MMA issuer waiting for the quantised P */
  FMHA_I8_DEV_WAIT_O_READY = 8,    /* softmax waiting for P.V */
  FMHA_I8_DEV_WAIT_O_FREE = 9,     /* MMA issuer waiting for the previous P.V to be drained */
  FMHA_I8_DEV_WAIT_DEBUG = 10,     /* a wait inside a debug kernel */
  FMHA_I8_DEV_WAIT_INFO = 11       /* a role waiting for (or the scanner waiting to reuse) a unit's mask information */
};

#define FMHA_I8_FLAG_USE_TCU 1u    /* mirrors the reference's use_tcu argument; must be set */
/* P quantised as UNSIGNED 8 bit with 255 levels, P8 = rn(255 p), final scale v_amax/(255 o_amax): the
 * UINT8 x INT8 variant the reference's README lists as planned (README.md:15,137-143,186) and its kernel
 * does not have.  Off by default: without it P8 = -rn(128 p) as in inc/fmha_i8.cuh:241-250. */
#define FMHA_I8_FLAG_UINT8_P 2u

/* Replaces gpuImpl::FMHAInferI8 / LaunchFMHAInfer_TCU / FMHAInferKernel
 * (src/fmha_i8.cu:157-173, :31-155, inc/fmha_i8.cuh:43-334): the whole forward pass
 * O8 = requant(softmax_tile128(Q8 K8^T * q_amax k_amax / (127^2 sqrt(D))) V8). */
int fmha_i8_sm100_infer(void* stream, const float amax[5], const int desc[4],
                        const void* q, const void* k, const void* v, const void* mask, void* o,
                        unsigned flags);

/* The same computation for heads [bh_begin, bh_begin + bh_count) of the flattened batch*head
 * axis, for partitioning one problem over several GPUs.  q,k,v,o point at the FIRST head of the
 * slice (each GPU holds only its slice); mask is the whole [B,S] mask and desc the whole shape.
 * The reference has no counterpart: its grid is (batch, head) on one GPU (src/fmha_i8.cu:43). */
int fmha_i8_sm100_infer_slice(void* stream, const float amax[5], const int desc[4],
                              const void* q, const void* k, const void* v, const void* mask, void* o,
                              int bh_begin, int bh_count, unsigned flags);

/* Attention with a different number of query rows and keys (cross-attention, decoding against a cache):
 * desc5 = {batch_num, seq_len_q, seq_len_k, head_num, head_dim}; q and o are int8 [B,H,seq_len_q,D],
 * k and v int8 [B,H,seq_len_k,D], mask int8 [B,seq_len_k].  seq_len_q is any number from 1 to 32768,
 * seq_len_k a multiple of 64 up to 32768.  bh_begin/bh_count select heads as in
 * fmha_i8_sm100_infer_slice (0 and B*H for the whole problem).  The reference lists this shape as
 * planned (README.md:13) and has no entry point for it; its CPU softmax already takes both lengths
 * (inc/cpuSoftmax.hpp:12), which is what the test oracle is pinned to. */
int fmha_i8_sm100_infer_cross(void* stream, const float amax[5], const int desc5[5],
                              const void* q, const void* k, const void* v, const void* mask, void* o,
                              int bh_begin, int bh_count, unsigned flags);

/* Whole-row scaling policies for the 8-bit P, the subject of the reference's accuracy study
 * (fmha_i8_quant_deviation.py:57-121, fmha_i8_quant_error_seqlen.py, README.md:192-222) and absent from its kernel,
 * which quantises P against the maximum of each 128-key tile.
 *   FMHA_I8_POLICY_TILE    the reference kernel's arithmetic: identical to fmha_i8_sm100_infer_cross
 *   FMHA_I8_POLICY_ROW     "dynamic quantization": P8 = rn(127 p / p_amax_row), p_amax_row = the row's largest
 *                          probability (fmha_i8_quant_deviation.py:104-121)
 *   FMHA_I8_POLICY_STATIC  "static quantization": P8 = min(rn(127 p / s_max), 127) with ONE calibrated scale for
 *                          every row: amax[4] = s_max, the FMHAParamI8 field the reference fills
 *                          (test_fmha_i8.cpp:152) and never reads (README.md:27; :82-102 of the script)
 * P is unsigned with 127 levels as in the study.  A row's scale is only known when all its keys have been seen, so
 * the call makes two launches on `stream`: the first computes every row's maximum and exp-sum, the second
 * quantises and multiplies.  row_scratch: caller-owned device memory, 2 floats per query row of the slice
 * (8 * bh_count * seq_len_q bytes, 8-byte aligned); nothing is allocated.  Other arguments as in
 * fmha_i8_sm100_infer_cross; FMHA_I8_FLAG_UINT8_P is not accepted. */
#define FMHA_I8_POLICY_TILE 0
#define FMHA_I8_POLICY_ROW 1
#define FMHA_I8_POLICY_STATIC 2
int fmha_i8_sm100_infer_policy(void* stream, const float amax[5], const int desc5[5],
                               const void* q, const void* k, const void* v, const void* mask, void* o,
                               int bh_begin, int bh_count, unsigned flags, int policy, float* row_scratch);

/* Calibration of o_amax on the device.  The reference takes o_amax = max|O| from its fp32 CPU attention
 * (test_fmha_i8.cpp:161) before it can call the int8 kernel at all; this runs the same int8 pipeline
 * (same kernel, same tiles) but instead of storing O8 it writes the largest magnitude of the unquantised
 * output, in real units, to the device float *o_amax_out (zeroed first, on the same stream).  amax[0..2]
 * = q, k, v ranges; amax[3], amax[4] are ignored.  desc5 and flags as in fmha_i8_sm100_infer_cross; o is
 * not needed.  Feeding the result back as o_amax makes the largest output element quantise to +-127. */
int fmha_i8_sm100_calibrate_o_amax(void* stream, const float amax[5], const int desc5[5],
                                   const void* q, const void* k, const void* v, const void* mask,
                                   float* o_amax_out, unsigned flags);

/* End-to-end form of the caller in test_fmha_i8.cpp:165-178,204,236: HOST buffers in, HOST
 * buffer out.  Copies q,k,v,mask to device staging buffers owned by the library (grown on demand,
 * kept for reuse), runs the forward pass, copies o back and synchronises.  The work is pipelined
 * over up to eight ranges of heads on three internal streams, so with pinned host memory the
 * inbound copies, the kernels and the outbound copies overlap; pageable memory works too. */
int fmha_i8_sm100_infer_host(const float amax[5], const int desc[4],
                             const void* host_q, const void* host_k, const void* host_v,
                             const void* host_mask, void* host_o, unsigned flags);

/* The same for heads [bh_begin, bh_begin + bh_count) of the flattened batch*head axis: host_q/k/v/o point at
 * the FIRST head of the slice (each process holds only its slice), host_mask is the whole [B,S] mask and desc
 * the whole shape.  This is what one rank of a multi-GPU job calls when its inputs live in host memory.  The
 * reference has no counterpart (one GPU, grid = (batch, head), src/fmha_i8.cu:43). */
int fmha_i8_sm100_infer_host_slice(const float amax[5], const int desc[4],
                                   const void* host_q, const void* host_k, const void* host_v,
                                   const void* host_mask, void* host_o, int bh_begin, int bh_count,
                                   unsigned flags);

/* Debug: S_int32[bh, i, j] = sum_d q[bh,i,d] k[bh,j,d] written as int32 [B*H, S, S] through the
 * same TMA + tensor-core stage the forward pass uses (GEMM 1, inc/fmha_i8.cuh:120-172).  For
 * bit-exact checks against cpuGEMM<int32_t,int32_t,int8_t,int32_t>; small shapes only. */
int fmha_i8_sm100_debug_qk(void* stream, const int desc[4], const void* q, const void* k, int32_t* s_out);

/* Debug: O_int32[bh, i, d] = sum_j p[bh,i,j] v[bh,j,d] as int32 [B*H, S, D] with p int8 [B*H,S,S],
 * through the P.V stage of the forward pass (GEMM 2, inc/fmha_i8.cuh:255-296).
 * variant 0: P handed to the tensor core from tensor memory; variant 1: from shared memory. */
int fmha_i8_sm100_debug_pv(void* stream, const int desc[4], const void* p, const void* v,
                           int32_t* o_out, unsigned variant);

/* Debug: the forward pass on CUDA cores (dp4a), one thread per query row, with the operation
 * order of the quantised CPU oracle.  An on-device cross-check for full-size shapes, never
 * selected by the product entry points.  Same arguments as fmha_i8_sm100_infer. */
int fmha_i8_sm100_debug_simt(void* stream, const float amax[5], const int desc[4],
                             const void* q, const void* k, const void* v, const void* mask, void* o);

/* The same cross-check for the extended shapes and flags of fmha_i8_sm100_infer_cross
 * (desc5 = {batch_num, seq_len_q, seq_len_k, head_num, head_dim}; flags: FMHA_I8_FLAG_UINT8_P or 0). */
int fmha_i8_sm100_debug_simt_x(void* stream, const float amax[5], const int desc5[5],
                               const void* q, const void* k, const void* v, const void* mask, void* o,
                               unsigned flags);

/* Debug: shows what a host sees when a device-side wait gives up, without faulting anything.  One warp
 * waits for at most limit_cycles (1000 ... 2e9 SM cycles) on a barrier that never completes, records
 * FMHA_I8_DEV_WAIT_DEBUG in the status words and returns normally; the context stays usable.  The first
 * forward call the host makes after that kernel has finished returns FMHA_I8_ERR_DEVICE once (nothing
 * is launched); fmha_i8_sm100_device_status() reports the words and clears them.  No counterpart in the
 * reference, which checks nothing. */
int fmha_i8_sm100_debug_wait_probe(void* stream, long long limit_cycles);

/* Per-tensor symmetric quantisation on the device, the producer step in front of the attention call:
 * amax = max|x| (abs_max, inc/utils.hpp:31-39) and q[i] = clamp(floor(x[i]*127/amax + 0.5), -127, 127)
 * (float_quant2_int8, inc/utils.hpp:23-29; the reference does both on the host, test_fmha_i8.cpp:95-110).
 * x: n floats (device, 16-byte aligned), out: n int8 (device, 16-byte aligned), amax_out: one float on
 * the device (may be NULL).  Two kernels on `stream`, no synchronisation.  Uses a scratch buffer of
 * partial maxima that the library allocates per device and keeps (calls on different streams of one
 * device that overlap in time would share it: serialise them). */
int fmha_i8_sm100_quantize_f32(void* stream, const float* x, long long n, int8_t* out, float* amax_out);

/* The same quantisation for callers that must not allocate device memory.  (No counterpart in the
 * reference project.)  Some hosts of this library hand every byte of the GPU to their own memory pool
 * when they start, so a cudaMalloc made later by a library either fails or escapes the pool's
 * accounting; others run a latency-critical loop and cannot afford the device-wide synchronisation that
 * cudaMalloc and cudaFree imply.  For them the partial maxima are kept in a 16 KB array that is part of
 * the library's device image: this entry point calls no cudaMalloc, no cudaFree and nothing else that
 * allocates.
 *   - Limit: n <= 268,435,456 elements (4096 chunks of 65536); larger tensors are refused with
 *     FMHA_I8_ERR_TOO_LARGE and one line on stderr.
 *   - The first call on each device looks up the device address of that array (with that device
 *     current); make that first call before any stream capture begins.
 *   - All calls on one device share the one array.  Nothing in it has to be cleared between calls (each
 *     call overwrites every slot it later reads), but two calls whose kernels overlap on the GPU --
 *     different streams without an ordering between them -- race on it: keep them ordered.
 * Arguments and results are those of fmha_i8_sm100_quantize_f32. */
int fmha_i8_sm100_quantize_f32_noalloc(void* stream, const float* x, long long n, int8_t* out, float* amax_out);

/* Synchronises the current device, copies out and clears the eight device status words.
 * words[0] == 0 means no kernel of this library gave up on a bounded wait since the last call.
 * Otherwise words[0] = which wait gave up (FMHA_I8_DEV_*), words[1] = block index, words[2] = warp,
 * words[3] = key-tile counter of the first failure.
 * Returns FMHA_I8_OK, FMHA_I8_ERR_DEVICE when words[0] != 0, or FMHA_I8_ERR_LAUNCH. */
int fmha_i8_sm100_device_status(unsigned words[8]);

/* Status of the most recent call on this host thread (what the void C++ shim could not return). */
int fmha_i8_sm100_last_status(void);
const char* fmha_i8_sm100_status_string(int status);

/* Number of kernels this library has launched in this process (all entry points). */
unsigned long long fmha_i8_sm100_launch_count(void);

int fmha_i8_sm100_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FMHA_I8_C_H_ */
