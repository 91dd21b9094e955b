"""B200-native INT8 flash-attention forward pass behind the host API of
jundaf2/INT8-Flash-Attention-FMHA-Quantization.

This module is the Python mirror of the reference's C++ host interface (inc/fmha_i8.h:5-17,
inc/fmha_param_i8.h:3-17): the same names (`FMHAInferI8`, `FMHAParamI8`, `AttnDataDescriptor`), the
same argument order and meaning.  It binds the C ABI of libfmha_i8_sm100.so (include/fmha_i8_c.h)
with ctypes; there is no other implementation behind it: if the library is missing the import
fails, and every call needs a B200.
"""
import ctypes
import os
from dataclasses import dataclass

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libfmha_i8_sm100.so")

OK = 0
ERR_NULL_POINTER = -1
ERR_BAD_SHAPE = -2
ERR_MISALIGNED = -3
ERR_NO_CUDA_CORE_PATH = -4
ERR_WRONG_ARCH = -5
ERR_LAUNCH = -6
ERR_DRIVER = -7
ERR_BAD_SLICE = -8
ERR_BAD_AMAX = -9
ERR_TOO_LARGE = -10
ERR_DEVICE = -11
ERR_BAD_FLAGS = -12
FLAG_USE_TCU = 1
FLAG_UINT8_P = 2     # P quantised as unsigned 8 bit, 255 levels (the reference README's planned variant)

EXPORTS = (
    "fmha_i8_sm100_infer", "fmha_i8_sm100_infer_slice", "fmha_i8_sm100_infer_cross", "fmha_i8_sm100_calibrate_o_amax", "fmha_i8_sm100_infer_host",
    "fmha_i8_sm100_infer_host_slice", "fmha_i8_sm100_infer_policy",
    "fmha_i8_sm100_debug_qk", "fmha_i8_sm100_debug_pv", "fmha_i8_sm100_debug_simt", "fmha_i8_sm100_debug_simt_x", "fmha_i8_sm100_debug_wait_probe",
    "fmha_i8_sm100_quantize_f32", "fmha_i8_sm100_quantize_f32_noalloc", "fmha_i8_sm100_device_status", "fmha_i8_sm100_last_status", "fmha_i8_sm100_status_string",
    "fmha_i8_sm100_launch_count", "fmha_i8_sm100_version",
)


class FmhaError(RuntimeError):
    def __init__(self, status, where):
        self.status = status
        super().__init__(f"{where}: {status_string(status)} (status {status})")


@dataclass
class AttnDataDescriptor:
    """Shape of the problem; field order as in the reference (seq_len before head_num)."""
    batch_num: int = 1
    seq_len: int = 64
    head_num: int = 4
    head_dim: int = 64

    def as_c(self):
        return (ctypes.c_int * 4)(self.batch_num, self.seq_len, self.head_num, self.head_dim)


@dataclass
class AttnDataDescriptorX:
    """Shape with separate query and key lengths (the reference lists this as planned, README.md:13)."""
    batch_num: int = 1
    seq_len_q: int = 64
    seq_len_k: int = 64
    head_num: int = 4
    head_dim: int = 64

    def as_c(self):
        return (ctypes.c_int * 5)(self.batch_num, self.seq_len_q, self.seq_len_k, self.head_num, self.head_dim)


@dataclass
class FMHAParamI8:
    """Per-tensor symmetric quantisation ranges (real = int8 * amax / 127)."""
    q_amax: float = 0.0
    k_amax: float = 0.0
    v_amax: float = 0.0
    o_amax: float = 1.0
    s_max: float = 1.0

    def as_c(self):
        return (ctypes.c_float * 5)(self.q_amax, self.k_amax, self.v_amax, self.o_amax, self.s_max)


_lib = None


def lib():
    """The loaded shared library.  Raises if it has not been built (python build.py)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python {os.path.join(HERE, 'build.py')}`; "
                              "there is no fallback implementation")
        L = ctypes.CDLL(LIB_PATH)
        vp, fp, ip, u = ctypes.c_void_p, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_int), ctypes.c_uint
        L.fmha_i8_sm100_infer.argtypes = [vp, fp, ip, vp, vp, vp, vp, vp, u]
        L.fmha_i8_sm100_infer_slice.argtypes = [vp, fp, ip, vp, vp, vp, vp, vp, ctypes.c_int, ctypes.c_int, u]
        L.fmha_i8_sm100_infer_cross.argtypes = [vp, fp, ip, vp, vp, vp, vp, vp, ctypes.c_int, ctypes.c_int, u]
        L.fmha_i8_sm100_calibrate_o_amax.argtypes = [vp, fp, ip, vp, vp, vp, vp, vp, u]
        L.fmha_i8_sm100_infer_policy.argtypes = [vp, fp, ip, vp, vp, vp, vp, vp, ctypes.c_int, ctypes.c_int, u, ctypes.c_int, vp]
        L.fmha_i8_sm100_infer_host.argtypes = [fp, ip, vp, vp, vp, vp, vp, u]
        L.fmha_i8_sm100_infer_host_slice.argtypes = [fp, ip, vp, vp, vp, vp, vp, ctypes.c_int, ctypes.c_int, u]
        L.fmha_i8_sm100_debug_qk.argtypes = [vp, ip, vp, vp, vp]
        L.fmha_i8_sm100_debug_pv.argtypes = [vp, ip, vp, vp, vp, u]
        L.fmha_i8_sm100_debug_simt.argtypes = [vp, fp, ip, vp, vp, vp, vp, vp]
        L.fmha_i8_sm100_debug_simt_x.argtypes = [vp, fp, ip, vp, vp, vp, vp, vp, u]
        L.fmha_i8_sm100_debug_wait_probe.argtypes = [vp, ctypes.c_longlong]
        L.fmha_i8_sm100_quantize_f32.argtypes = [vp, vp, ctypes.c_longlong, vp, vp]
        L.fmha_i8_sm100_quantize_f32_noalloc.argtypes = [vp, vp, ctypes.c_longlong, vp, vp]
        L.fmha_i8_sm100_device_status.argtypes = [ctypes.POINTER(ctypes.c_uint)]
        L.fmha_i8_sm100_status_string.restype = ctypes.c_char_p
        L.fmha_i8_sm100_status_string.argtypes = [ctypes.c_int]
        L.fmha_i8_sm100_launch_count.restype = ctypes.c_ulonglong
        for name in EXPORTS:
            getattr(L, name)
        _lib = L
    return _lib


def status_string(status):
    return lib().fmha_i8_sm100_status_string(int(status)).decode()


def _ptr(x):
    """Device or host address of a torch tensor / numpy array / raw int."""
    if x is None:
        return None
    if isinstance(x, int):
        return ctypes.c_void_p(x)
    if hasattr(x, "data_ptr"):
        return ctypes.c_void_p(x.data_ptr())
    if hasattr(x, "ctypes"):
        return ctypes.c_void_p(x.ctypes.data)
    raise TypeError(f"cannot take the address of {type(x)}")


def _stream_handle(stream):
    if stream is None:
        import torch
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if isinstance(stream, int):
        return ctypes.c_void_p(stream)
    return ctypes.c_void_p(stream.cuda_stream)


def _flags(use_tcu=True, uint8_p=False):
    return (FLAG_USE_TCU if use_tcu else 0) | (FLAG_UINT8_P if uint8_p else 0)


def FMHAInferI8(stream, fmha_param, attn_desc, q, k, v, padding_mask, o, use_tcu=True, check=True, uint8_p=False):
    """Mirror of gpuImpl::FMHAInferI8 (reference inc/fmha_i8.h:7-15).

    q, k, v, o: int8 [B,H,S,D] device tensors; padding_mask: int8 [B,S], non-zero = key masked.
    Enqueues on `stream` (None = torch's current stream) and returns the status without
    synchronising.  With check=True a non-zero status raises FmhaError (the reference returns void
    and silently does nothing on unsupported input)."""
    st = lib().fmha_i8_sm100_infer(_stream_handle(stream), fmha_param.as_c(), attn_desc.as_c(), _ptr(q), _ptr(k),
                                   _ptr(v), _ptr(padding_mask), _ptr(o), _flags(use_tcu, uint8_p))
    if check and st != OK:
        raise FmhaError(st, "FMHAInferI8")
    return st


def FMHAInferI8Cross(stream, fmha_param, attn_desc_x, q, k, v, padding_mask, o, bh_begin=0, bh_count=None,
                     use_tcu=True, check=True, uint8_p=False):
    """Query rows and keys differ in number: q, o int8 [B,H,Sq,D]; k, v int8 [B,H,Sk,D]; padding_mask int8
    [B,Sk].  attn_desc_x is an AttnDataDescriptorX.  bh_begin/bh_count select heads as in FMHAInferI8Slice."""
    if bh_count is None:
        bh_count = attn_desc_x.batch_num * attn_desc_x.head_num - bh_begin
    st = lib().fmha_i8_sm100_infer_cross(_stream_handle(stream), fmha_param.as_c(), attn_desc_x.as_c(), _ptr(q), _ptr(k),
                                         _ptr(v), _ptr(padding_mask), _ptr(o), int(bh_begin), int(bh_count),
                                         _flags(use_tcu, uint8_p))
    if check and st != OK:
        raise FmhaError(st, "FMHAInferI8Cross")
    return st


POLICY_TILE, POLICY_ROW, POLICY_STATIC = 0, 1, 2


def FMHAInferI8Policy(stream, fmha_param, attn_desc_x, q, k, v, padding_mask, o, policy, row_scratch, bh_begin=0, bh_count=None,
                      check=True):
    """Whole-row scaling policies for the 8-bit P (reference fmha_i8_quant_deviation.py:57-121): POLICY_ROW = per-row
    ("dynamic") scale, POLICY_STATIC = one calibrated scale fmha_param.s_max for all rows, POLICY_TILE = the reference
    kernel's tile-local scale.  row_scratch: float32 device tensor with 2 elements per query row of the slice."""
    if bh_count is None:
        bh_count = attn_desc_x.batch_num * attn_desc_x.head_num - bh_begin
    st = lib().fmha_i8_sm100_infer_policy(_stream_handle(stream), fmha_param.as_c(), attn_desc_x.as_c(), _ptr(q), _ptr(k), _ptr(v),
                                          _ptr(padding_mask), _ptr(o), int(bh_begin), int(bh_count), _flags(True, False),
                                          int(policy), _ptr(row_scratch))
    if check and st != OK:
        raise FmhaError(st, "FMHAInferI8Policy")
    return st


def calibrate_o_amax(stream, fmha_param, attn_desc_x, q, k, v, padding_mask, o_amax_out, uint8_p=False):
    """Largest |output| of the int8 pipeline in real units, written to the one-element float32 device tensor
    `o_amax_out` (the reference takes this number from its fp32 CPU attention, test_fmha_i8.cpp:161).
    Only q_amax, k_amax, v_amax of `fmha_param` are used.  Enqueues on `stream`, no synchronisation."""
    st = lib().fmha_i8_sm100_calibrate_o_amax(_stream_handle(stream), fmha_param.as_c(), attn_desc_x.as_c(), _ptr(q), _ptr(k),
                                              _ptr(v), _ptr(padding_mask), _ptr(o_amax_out), _flags(True, uint8_p))
    if st != OK:
        raise FmhaError(st, "calibrate_o_amax")


def FMHAInferI8Slice(stream, fmha_param, attn_desc, q, k, v, padding_mask, o, bh_begin, bh_count, check=True, uint8_p=False):
    """Heads [bh_begin, bh_begin+bh_count) of the flattened batch*head axis; q,k,v,o hold only the slice."""
    st = lib().fmha_i8_sm100_infer_slice(_stream_handle(stream), fmha_param.as_c(), attn_desc.as_c(), _ptr(q), _ptr(k),
                                         _ptr(v), _ptr(padding_mask), _ptr(o), int(bh_begin), int(bh_count), _flags(True, uint8_p))
    if check and st != OK:
        raise FmhaError(st, "FMHAInferI8Slice")
    return st


def FMHAInferI8Host(fmha_param, attn_desc, host_q, host_k, host_v, host_mask, host_o, check=True, uint8_p=False):
    """Host buffers in, host buffer out (copies inside); synchronous."""
    st = lib().fmha_i8_sm100_infer_host(fmha_param.as_c(), attn_desc.as_c(), _ptr(host_q), _ptr(host_k), _ptr(host_v),
                                        _ptr(host_mask), _ptr(host_o), _flags(True, uint8_p))
    if check and st != OK:
        raise FmhaError(st, "FMHAInferI8Host")
    return st


def FMHAInferI8HostSlice(fmha_param, attn_desc, host_q, host_k, host_v, host_mask, host_o, bh_begin, bh_count,
                         check=True, uint8_p=False):
    """Host buffers of heads [bh_begin, bh_begin+bh_count) in, host buffer of those heads out; the mask is whole."""
    st = lib().fmha_i8_sm100_infer_host_slice(fmha_param.as_c(), attn_desc.as_c(), _ptr(host_q), _ptr(host_k), _ptr(host_v),
                                              _ptr(host_mask), _ptr(host_o), int(bh_begin), int(bh_count), _flags(True, uint8_p))
    if check and st != OK:
        raise FmhaError(st, "FMHAInferI8HostSlice")
    return st


def debug_qk(stream, attn_desc, q, k, s_out):
    st = lib().fmha_i8_sm100_debug_qk(_stream_handle(stream), attn_desc.as_c(), _ptr(q), _ptr(k), _ptr(s_out))
    if st != OK:
        raise FmhaError(st, "debug_qk")


def debug_pv(stream, attn_desc, p, v, o_out, variant=0):
    st = lib().fmha_i8_sm100_debug_pv(_stream_handle(stream), attn_desc.as_c(), _ptr(p), _ptr(v), _ptr(o_out), variant)
    if st != OK:
        raise FmhaError(st, "debug_pv")


def debug_simt(stream, fmha_param, attn_desc, q, k, v, padding_mask, o):
    st = lib().fmha_i8_sm100_debug_simt(_stream_handle(stream), fmha_param.as_c(), attn_desc.as_c(), _ptr(q), _ptr(k),
                                        _ptr(v), _ptr(padding_mask), _ptr(o))
    if st != OK:
        raise FmhaError(st, "debug_simt")


def debug_simt_x(stream, fmha_param, attn_desc_x, q, k, v, padding_mask, o, uint8_p=False):
    st = lib().fmha_i8_sm100_debug_simt_x(_stream_handle(stream), fmha_param.as_c(), attn_desc_x.as_c(), _ptr(q), _ptr(k),
                                          _ptr(v), _ptr(padding_mask), _ptr(o), FLAG_UINT8_P if uint8_p else 0)
    if st != OK:
        raise FmhaError(st, "debug_simt_x")


def debug_wait_probe(stream, limit_cycles):
    """Launches the one-warp kernel whose bounded wait runs out on purpose (no fault; see the C header)."""
    st = lib().fmha_i8_sm100_debug_wait_probe(_stream_handle(stream), int(limit_cycles))
    if st != OK:
        raise FmhaError(st, "debug_wait_probe")


def quantize_f32(stream, x, out, amax_out=None, n=None, entry="fmha_i8_sm100_quantize_f32"):
    """Device-side abs_max + float_quant2_int8 (reference inc/utils.hpp:23-39): x float32 -> out int8,
    amax written to the one-element device tensor `amax_out`.  Enqueues on `stream`, no synchronisation.
    entry="fmha_i8_sm100_quantize_f32_noalloc" selects the variant that never allocates device memory
    (built-in scratch, at most 268,435,456 elements, calls on one device must not overlap)."""
    count = int(n if n is not None else x.numel())
    st = getattr(lib(), entry)(_stream_handle(stream), _ptr(x), count, _ptr(out), _ptr(amax_out))
    if st != OK:
        raise FmhaError(st, entry)


def device_status():
    """Synchronises, returns (status, [8 words]) and clears the words."""
    words = (ctypes.c_uint * 8)()
    st = lib().fmha_i8_sm100_device_status(words)
    return st, list(words)


def launch_count():
    return int(lib().fmha_i8_sm100_launch_count())
