"""ctypes binding of liblthn_cuda.so (the C ABI in include/lthn_cuda.h).

This module is the Python face of the shared library that tests and bench.py use;
it adds nothing to the compute path. Importing it never needs a GPU; calling a
compute function without the library built, or without a device, raises."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("LTHN_CUDA_LIB") or os.path.join(os.path.dirname(_HERE), "liblthn_cuda.so")

OK = 0
F32, BF16 = 0, 1


class LthnError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"lthn error {code}: {msg}")
        self.code = code
        self.msg = msg


class DeviceInfo(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("architecture", C.c_char * 16), ("memory_size", C.c_uint64),
                ("max_buffer_length", C.c_uint64), ("max_recommended_working_set", C.c_uint64),
                ("sm_count", C.c_int32), ("compute_major", C.c_int32), ("compute_minor", C.c_int32)]


class LoadOptions(C.Structure):
    _fields_ = [("max_len", C.c_int32), ("max_lanes", C.c_int32), ("tp_rank", C.c_int32), ("tp_size", C.c_int32),
                ("comm", C.c_void_p), ("uniform_attention", C.c_int32)]


class SampleParams(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float), ("min_p", C.c_float),
                ("repeat_penalty", C.c_float), ("min_tokens_before_stop", C.c_int32), ("suppress", C.POINTER(C.c_int32)),
                ("n_suppress", C.c_int32)]


def sample_params(temperature=0.0, top_k=0, top_p=0.0, min_p=0.0, repeat_penalty=0.0, min_tokens_before_stop=0, suppress=()):
    sup = np.ascontiguousarray(suppress, dtype=np.int32)
    p = SampleParams(temperature, top_k, top_p, min_p, repeat_penalty, min_tokens_before_stop,
                     sup.ctypes.data_as(C.POINTER(C.c_int32)) if sup.size else None, sup.size)
    p._keep = sup   # the struct borrows the array
    return p


class Sampler:
    """model.Sampler: a reproducible splitmix64 stream plus the sampling arithmetic (lthn_sampler_*)."""

    def __init__(self, seed: int):
        h = C.c_void_p()
        check(lib().lthn_sampler_create(seed, C.byref(h)))
        self.h = h

    def draw(self) -> float:
        return float(lib().lthn_sampler_draw(self.h))

    def sample(self, logits_bf16: np.ndarray, params: SampleParams, ids=None) -> int:
        a = np.ascontiguousarray(logits_bf16, dtype=np.uint16)
        tok = C.c_int32()
        if ids is None:
            check(lib().lthn_sampler_sample(self.h, a.ctypes.data, a.size, C.byref(params), C.byref(tok)))
        else:
            i = np.ascontiguousarray(ids, dtype=np.int32)
            check(lib().lthn_sampler_sample_candidates(self.h, a.ctypes.data, i.ctypes.data, a.size, C.byref(params), C.byref(tok)))
        return int(tok.value)

    def close(self):
        if self.h:
            lib().lthn_sampler_destroy(self.h)
            self.h = None


class _PhaseShare(C.Structure):
    _fields_ = [("name", C.c_char * 48), ("per_token_us", C.c_double), ("gpu", C.c_int32)]


class DecodePhaseBudget(C.Structure):
    """inference.DecodePhaseBudget."""
    _fields_ = [("tokens", C.c_int32), ("total_per_token_us", C.c_double), ("gpu_per_token_us", C.c_double),
                ("n_phases", C.c_int32), ("phases", _PhaseShare * 8)]

    def shares(self):
        return [(self.phases[i].name.decode(), float(self.phases[i].per_token_us), bool(self.phases[i].gpu)) for i in range(self.n_phases)]


class ModelConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("layers", "hidden", "q_heads", "kv_heads", "head_dim", "ffn", "vocab",
                                         "group_size", "bits", "max_len", "max_lanes")] + \
               [(n, C.c_float) for n in ("eps", "rope_base", "attn_scale", "embed_scale")] + \
               [("tp_rank", C.c_int32), ("tp_size", C.c_int32), ("sliding_window", C.c_int32), ("sliding_pattern", C.c_int32),
                ("rope_local_base", C.c_float)]


_lib = None


def lib() -> C.CDLL:
    """Loads the shared library; fails loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LthnError(3, f"{LIB_PATH} is missing: run `python go-inference_b200/build.py`")
        _lib = C.CDLL(LIB_PATH)
        _lib.lthn_last_error.restype = C.c_char_p
        for name in dir(_Sig):
            if name.startswith("lthn_"):
                try:
                    fn = getattr(_lib, name)
                except AttributeError:
                    if name.startswith("lthn_debug_"):
                        continue   # only the test-hook build (liblthn_cuda_hooks.so) has these
                    raise
                fn.restype, fn.argtypes = getattr(_Sig, name)
    return _lib


vp, i32, i64, u64, f32, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_float, C.c_size_t
pvp = C.POINTER(C.c_void_p)


class _Sig:
    lthn_cuda_available = (i32, [])
    lthn_cuda_device_count = (i32, [])
    lthn_cuda_set_device = (i32, [i32])
    lthn_cuda_device_info = (i32, [i32, C.POINTER(DeviceInfo)])
    lthn_cuda_mem_info = (i32, [C.POINTER(u64), C.POINTER(u64)])
    lthn_device_status = (i32, [vp, C.POINTER(C.c_uint32)])
    lthn_malloc = (i32, [pvp, sz])
    lthn_free = (i32, [vp])
    lthn_host_alloc = (i32, [pvp, sz])
    lthn_host_free = (i32, [vp])
    lthn_memcpy_h2d = (i32, [vp, vp, sz, vp])
    lthn_memcpy_d2h = (i32, [vp, vp, sz, vp])
    lthn_memcpy_d2d = (i32, [vp, vp, sz, vp])
    lthn_memset = (i32, [vp, i32, sz, vp])
    lthn_stream_create = (i32, [pvp])
    lthn_stream_destroy = (i32, [vp])
    lthn_stream_sync = (i32, [vp])
    lthn_device_sync = (i32, [])
    lthn_event_create = (i32, [pvp])
    lthn_event_destroy = (i32, [vp])
    lthn_event_record = (i32, [vp, vp])
    lthn_event_elapsed_ms = (i32, [vp, vp, C.POINTER(f32)])
    lthn_graph_begin = (i32, [vp])
    lthn_graph_end = (i32, [vp, pvp])
    lthn_graph_launch = (i32, [vp, vp])
    lthn_graph_destroy = (i32, [vp])
    lthn_affine_quantize = (i32, [vp, vp, i64, i64, i32, i32, i32, vp, vp, vp])
    lthn_affine_dequantize = (i32, [vp, vp, vp, vp, i64, i64, i32, i32, vp])
    lthn_affine_dequantize_bf16 = (i32, [vp, vp, vp, vp, i64, i64, i32, i32, vp])
    lthn_synth_normal_fill = (i32, [vp, u64, u64, i64, f32, vp])
    lthn_synth_affine_weight = (i32, [vp, u64, f32, i64, i64, i32, i32, i32, vp, vp, vp])
    lthn_affine_qmv = (i32, [vp, vp, i32, i32, vp, vp, vp, i64, i64, i32, i32, vp, i32])
    lthn_affine_qmv_host = (i32, [vp, sz, vp, sz, vp, sz, vp, sz, i64, i64, i32, i32, vp, sz])
    lthn_affine_qmv_noalloc = (i32, [vp, vp, i32, vp, vp, vp, i64, i64, vp])
    lthn_affine_qmv_geglu = (i32, [vp, vp, i32, i32, vp, vp, vp, vp, vp, vp, i64, i64, vp, i32])
    lthn_affine_qmv_normed = (i32, [vp, vp, vp, vp, vp, vp, f32, i32, vp, vp, vp, vp, vp, vp, i64, i64, vp, i32])
    lthn_affine_qmv_geglu_bits = (i32, [vp, vp, i32, i32, vp, vp, vp, vp, vp, vp, i64, i64, i32, vp, i32])
    lthn_affine_qmv_normed_bits = (i32, [vp, vp, vp, vp, vp, vp, f32, i32, vp, vp, vp, vp, vp, vp, i64, i64, i32, vp, i32])
    lthn_rmsnorm = (i32, [vp, vp, vp, vp, i32, i32, f32])
    lthn_rmsnorm_residual = (i32, [vp, vp, vp, vp, vp, vp, i32, i32, f32])
    lthn_debug_rmsnorm_gather_local = (i32, [vp, vp, i32, vp, vp, vp, vp, vp, i32, i32, f32, i32, C.c_uint32])
    lthn_rmsnorm_rope = (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, f32, f32, i32])
    lthn_sdpa_decode = (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i64, f32, i32])
    lthn_argmax = (i32, [vp, vp, i32, i32, vp])
    lthn_model_create = (i32, [C.POINTER(ModelConfig), pvp])
    lthn_model_load_dir = (i32, [C.c_char_p, C.POINTER(LoadOptions), pvp])
    lthn_checkpoint_inspect = (i32, [C.c_char_p, C.c_char_p, sz])
    lthn_model_upload_linear = (i32, [vp, i32, i32, vp, vp, vp, i64, i64])
    lthn_model_upload_linear_bits = (i32, [vp, i32, i32, vp, vp, vp, i64, i64, i32])
    lthn_model_upload_norm = (i32, [vp, i32, i32, vp, i64])
    lthn_model_synthesize = (i32, [vp, u64, f32])
    lthn_model_finalize = (i32, [vp])
    lthn_model_weight_bytes = (i32, [vp, C.POINTER(u64)])
    lthn_model_tp_exchange = (i32, [vp, C.POINTER(i32)])
    lthn_model_graph_state = (i32, [vp, C.POINTER(i32)])
    lthn_model_decode_kernel = (i32, [vp, C.POINTER(i32)])
    lthn_model_destroy = (i32, [vp])
    lthn_tp_unique_id = (i32, [vp])
    lthn_tp_init = (i32, [i32, i32, vp, pvp])
    lthn_tp_destroy = (i32, [vp])
    lthn_model_set_comm = (i32, [vp, vp])
    lthn_session_open = (i32, [vp, pvp])
    lthn_session_prefill = (i32, [vp, vp, i32])
    lthn_session_append = (i32, [vp, vp, i32])
    lthn_session_pos = (i32, [vp])
    lthn_session_decode_greedy = (i32, [vp, i32, i32, vp, C.POINTER(i32)])
    lthn_session_logits = (i32, [vp, vp, i64])
    lthn_session_trace_begin = (i32, [vp])
    lthn_session_trace_end = (i32, [vp, C.POINTER(DecodePhaseBudget)])
    lthn_session_decode_sampled = (i32, [vp, vp, C.POINTER(SampleParams), i32, vp, i32, vp, C.POINTER(i32)])
    lthn_sampler_create = (i32, [u64, pvp])
    lthn_sampler_destroy = (i32, [vp])
    lthn_sampler_draw = (f32, [vp])
    lthn_sampler_sample = (i32, [vp, vp, i32, C.POINTER(SampleParams), C.POINTER(i32)])
    lthn_sampler_sample_candidates = (i32, [vp, vp, vp, i32, C.POINTER(SampleParams), C.POINTER(i32)])
    lthn_topk_candidates = (i32, [vp, vp, i32, i32, i32, vp, vp, vp])
    lthn_laneset_prepare_sampled = (i32, [vp, vp, i32, i32, vp, i32, C.POINTER(SampleParams), u64, C.POINTER(i32)])
    lthn_session_kv_export = (i32, [vp, i32, i32, vp, sz])
    lthn_session_kv_import = (i32, [vp, i32, i32, vp, i32])
    lthn_session_kv_export_range = (i32, [vp, i32, i32, i32, i32, vp, C.c_size_t])
    lthn_session_kv_import_range = (i32, [vp, i32, i32, i32, vp, i32])
    lthn_session_kv_gather_range = (i32, [vp, i32, i32, i32, i32, vp, C.c_size_t])
    lthn_session_fork = (i32, [vp, pvp])
    lthn_session_reset = (i32, [vp])
    lthn_session_set_state = (i32, [vp, i32, i32])
    lthn_session_close = (i32, [vp])
    lthn_laneset_open = (i32, [vp, i32, pvp])
    lthn_laneset_prepare = (i32, [vp, vp, i32, i32, vp, i32, C.POINTER(i32)])
    lthn_laneset_step = (i32, [vp, vp, vp, vp, C.POINTER(i32)])
    lthn_laneset_retire = (i32, [vp, i32])
    lthn_laneset_active = (i32, [vp])
    lthn_laneset_batch_forward_count = (u64, [vp])
    lthn_laneset_close = (i32, [vp])
    lthn_affine_qmm = (i32, [vp, vp, i32, vp, vp, vp, i64, i64, i32, i32, vp])
    lthn_affine_qmm_geglu = (i32, [vp, vp, i32, vp, vp, vp, vp, vp, vp, i64, i64, vp])
    lthn_affine_qmm_geglu_bits = (i32, [vp, vp, i32, vp, vp, vp, vp, vp, vp, i64, i64, i32, vp])
    lthn_prefill_attention = (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, f32])
    lthn_debug_qmm_force_tile = (None, [i32])
    lthn_debug_i8_plan = (i32, [i64, i64, i32, i32, i32, i32, i32, vp])
    lthn_debug_qmv_force_config = (None, [i32, i32])
    lthn_debug_qmv_force_kernel = (None, [i32])


def check(rc: int):
    if rc != OK:
        raise LthnError(rc, lib().lthn_last_error().decode(errors="replace"))


def device_count() -> int:
    try:
        return int(lib().lthn_cuda_device_count())
    except (OSError, LthnError):
        return 0


def available() -> bool:
    try:
        return bool(lib().lthn_cuda_available())
    except (OSError, LthnError):
        return False


def set_device(i: int):
    check(lib().lthn_cuda_set_device(i))


def device_info(i: int = 0) -> DeviceInfo:
    info = DeviceInfo()
    check(lib().lthn_cuda_device_info(i, C.byref(info)))
    return info


def sync():
    check(lib().lthn_device_sync())


def mem_info():
    """(free, total) bytes of the current device."""
    f, t = C.c_uint64(), C.c_uint64()
    check(lib().lthn_cuda_mem_info(C.byref(f), C.byref(t)))
    return int(f.value), int(t.value)


def device_status(stream=None) -> int:
    """Reads and clears the sticky device status words; raises LthnError (code 5) when a bounded
    device-side wait ran out since the last read, else returns 0."""
    bits = C.c_uint32()
    check(lib().lthn_device_status(stream.h if stream else None, C.byref(bits)))
    return int(bits.value)


class Stream:
    def __init__(self):
        h = C.c_void_p()
        check(lib().lthn_stream_create(C.byref(h)))
        self.h = h

    def sync(self):
        check(lib().lthn_stream_sync(self.h))

    def close(self):
        if self.h:
            lib().lthn_stream_destroy(self.h)
            self.h = None


class Event:
    def __init__(self):
        h = C.c_void_p()
        check(lib().lthn_event_create(C.byref(h)))
        self.h = h

    def record(self, stream=None):
        check(lib().lthn_event_record(self.h, stream.h if stream else None))

    def elapsed_ms(self, stop: "Event") -> float:
        ms = C.c_float()
        check(lib().lthn_event_elapsed_ms(self.h, stop.h, C.byref(ms)))
        return float(ms.value)


class Graph:
    """Captures the calls issued on `stream` inside the `with` block into a CUDA graph."""

    def __init__(self, stream: Stream):
        self.stream = stream
        self.h = None

    def __enter__(self):
        check(lib().lthn_graph_begin(self.stream.h))
        return self

    def __exit__(self, et, ev, tb):
        h = C.c_void_p()
        rc = lib().lthn_graph_end(self.stream.h, C.byref(h))
        if et is None:
            check(rc)
            self.h = h
        return False

    def launch(self, stream=None):
        check(lib().lthn_graph_launch(self.h, (stream or self.stream).h))

    def destroy(self):
        if self.h:
            lib().lthn_graph_destroy(self.h)
            self.h = None


class Buf:
    """A device allocation with NumPy upload / download helpers."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        check(lib().lthn_malloc(C.byref(p), max(self.nbytes, 1)))
        self.ptr = p.value

    @classmethod
    def from_array(cls, a: np.ndarray, stream=None) -> "Buf":
        a = np.ascontiguousarray(a)
        b = cls(a.nbytes)
        b.upload(a, stream)
        return b

    def upload(self, a: np.ndarray, stream=None):
        a = np.ascontiguousarray(a)
        assert a.nbytes <= self.nbytes
        check(lib().lthn_memcpy_h2d(self.ptr, a.ctypes.data, a.nbytes, stream.h if stream else None))
        check(lib().lthn_stream_sync(stream.h if stream else None))

    def download(self, dtype, shape, stream=None) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        assert out.nbytes <= self.nbytes
        check(lib().lthn_memcpy_d2h(out.ctypes.data, self.ptr, out.nbytes, stream.h if stream else None))
        return out

    def zero(self, stream=None):
        check(lib().lthn_memset(self.ptr, 0, self.nbytes, stream.h if stream else None))

    def free(self):
        if self.ptr:
            lib().lthn_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class PinnedArray:
    """NumPy view over pinned host memory (for full-rate host<->device copies)."""

    def __init__(self, shape, dtype):
        self.dtype = np.dtype(dtype)
        self.shape = tuple(shape) if not np.isscalar(shape) else (int(shape),)
        n = int(np.prod(self.shape)) * self.dtype.itemsize
        p = C.c_void_p()
        check(lib().lthn_host_alloc(C.byref(p), max(n, 1)))
        self.ptr = p.value
        self.nbytes = n
        self.array = np.frombuffer((C.c_char * max(n, 1)).from_address(self.ptr), dtype=self.dtype,
                                   count=int(np.prod(self.shape))).reshape(self.shape)

    def free(self):
        if self.ptr:
            self.array = None
            lib().lthn_host_free(self.ptr)
            self.ptr = None


def _s(stream):
    return stream.h if stream else None


class QuantWeight:
    """Device-resident MLX-affine weight: packed u32 [N,K*bits/32], bf16 scales/biases [N,K/gs]."""

    def __init__(self, N, K, bits=4, gs=64):
        self.N, self.K, self.bits, self.gs = int(N), int(K), int(bits), int(gs)
        self.packed = Buf(self.N * self.K * bits // 8)
        self.scales = Buf(self.N * (self.K // gs) * 2)
        self.biases = Buf(self.N * (self.K // gs) * 2)

    @classmethod
    def from_host(cls, packed, scales, biases, bits=4, gs=64):
        packed = np.ascontiguousarray(packed, dtype=np.uint32)
        N, K = packed.shape[0], packed.shape[1] * 32 // bits
        w = cls(N, K, bits, gs)
        w.packed.upload(packed)
        w.scales.upload(np.ascontiguousarray(scales, dtype=np.uint16))
        w.biases.upload(np.ascontiguousarray(biases, dtype=np.uint16))
        return w

    @classmethod
    def synth(cls, seed, sigma, N, K, bits=4, gs=64, variant=0, stream=None):
        w = cls(N, K, bits, gs)
        check(lib().lthn_synth_affine_weight(_s(stream), seed, sigma, N, K, bits, gs, variant, w.packed.ptr,
                                             w.scales.ptr, w.biases.ptr))
        return w

    @property
    def stream_bytes(self):
        return self.packed.nbytes + self.scales.nbytes + self.biases.nbytes

    def to_host(self):
        return (self.packed.download(np.uint32, (self.N, self.K * self.bits // 32)),
                self.scales.download(np.uint16, (self.N, self.K // self.gs)),
                self.biases.download(np.uint16, (self.N, self.K // self.gs)))

    def free(self):
        for b in (self.packed, self.scales, self.biases):
            b.free()


def quantize(w_dev: Buf, N, K, bits=4, gs=64, variant=0, stream=None) -> QuantWeight:
    q = QuantWeight(N, K, bits, gs)
    check(lib().lthn_affine_quantize(_s(stream), w_dev.ptr, N, K, bits, gs, variant, q.packed.ptr, q.scales.ptr,
                                     q.biases.ptr))
    return q


def dequantize(q: QuantWeight, out: Buf, bf16=False, stream=None):
    fn = lib().lthn_affine_dequantize_bf16 if bf16 else lib().lthn_affine_dequantize
    check(fn(_s(stream), q.packed.ptr, q.scales.ptr, q.biases.ptr, q.N, q.K, q.bits, q.gs, out.ptr))


def qmv(x: Buf, x_dtype, M, q: QuantWeight, y: Buf, y_dtype, stream=None):
    check(lib().lthn_affine_qmv(_s(stream), x.ptr, x_dtype, M, q.packed.ptr, q.scales.ptr, q.biases.ptr, q.N, q.K,
                                q.gs, q.bits, y.ptr, y_dtype))


def qmv_noalloc(x_f32: Buf, M, q: QuantWeight, y_f32: Buf, stream=None):
    """Allocation-free affine_qmv (f32 in, f32 out, 4 bit / group 64; see the header for its size limit)."""
    check(lib().lthn_affine_qmv_noalloc(_s(stream), x_f32.ptr, M, q.packed.ptr, q.scales.ptr, q.biases.ptr, q.N, q.K,
                                        y_f32.ptr))


def qmm(x: Buf, M, q: QuantWeight, y: Buf, stream=None):
    check(lib().lthn_affine_qmm(_s(stream), x.ptr, M, q.packed.ptr, q.scales.ptr, q.biases.ptr, q.N, q.K, q.gs, q.bits,
                                y.ptr))


def qmm_geglu(x: Buf, M, gate: QuantWeight, up: QuantWeight, y: Buf, stream=None):
    if gate.bits != 4:
        check(lib().lthn_affine_qmm_geglu_bits(_s(stream), x.ptr, M, gate.packed.ptr, gate.scales.ptr, gate.biases.ptr,
                                               up.packed.ptr, up.scales.ptr, up.biases.ptr, gate.N, gate.K, gate.bits, y.ptr))
        return
    check(lib().lthn_affine_qmm_geglu(_s(stream), x.ptr, M, gate.packed.ptr, gate.scales.ptr, gate.biases.ptr,
                                      up.packed.ptr, up.scales.ptr, up.biases.ptr, gate.N, gate.K, y.ptr))


def prefill_attention(q: Buf, kcache: Buf, vcache: Buf, out: Buf, rows, pos0, q_heads, kv_heads, head_dim, scale=0.0,
                      stream=None):
    check(lib().lthn_prefill_attention(_s(stream), q.ptr, kcache.ptr, vcache.ptr, out.ptr, rows, pos0, q_heads,
                                       kv_heads, head_dim, scale))


def topk_candidates(logits_f32: Buf, rows, vocab, k, scratch_bf16: Buf, out_ids: Buf, out_bf16: Buf, stream=None):
    """k best entries of each row after bf16 rounding, at out_ids / out_bf16 + row*256 (unordered within the k)."""
    check(lib().lthn_topk_candidates(_s(stream), logits_f32.ptr, rows, vocab, k, scratch_bf16.ptr, out_ids.ptr, out_bf16.ptr))


def qmv_geglu(x: Buf, x_dtype, M, gate: QuantWeight, up: QuantWeight, y: Buf, y_dtype, stream=None):
    if gate.bits != 4:
        check(lib().lthn_affine_qmv_geglu_bits(_s(stream), x.ptr, x_dtype, M, gate.packed.ptr, gate.scales.ptr, gate.biases.ptr,
                                               up.packed.ptr, up.scales.ptr, up.biases.ptr, gate.N, gate.K, gate.bits, y.ptr, y_dtype))
        return
    check(lib().lthn_affine_qmv_geglu(_s(stream), x.ptr, x_dtype, M, gate.packed.ptr, gate.scales.ptr, gate.biases.ptr,
                                      up.packed.ptr, up.scales.ptr, up.biases.ptr, gate.N, gate.K, y.ptr, y_dtype))


def qmv_host(x_bf16: np.ndarray, packed: np.ndarray, scales: np.ndarray, biases: np.ndarray, out_dim, in_dim, gs,
             bits) -> np.ndarray:
    """model.QuantMatVec.MatVec over host byte buffers (bf16 in, bf16 out)."""
    xb = np.ascontiguousarray(x_bf16).view(np.uint8).reshape(-1)
    pb = np.ascontiguousarray(packed).view(np.uint8).reshape(-1)
    sb = np.ascontiguousarray(scales).view(np.uint8).reshape(-1)
    bb = np.ascontiguousarray(biases).view(np.uint8).reshape(-1)
    y = np.zeros(max(int(out_dim), 0), dtype=np.uint16)
    check(lib().lthn_affine_qmv_host(xb.ctypes.data, xb.size, pb.ctypes.data, pb.size, sb.ctypes.data, sb.size,
                                     bb.ctypes.data, bb.size, out_dim, in_dim, gs, bits, y.ctypes.data, y.nbytes))
    return y


# ------------------------------------------------------------------ engine ----

ROLE = dict(q=0, k=1, v=2, o=3, gate=4, up=5, down=6)
NORM = dict(input=0, post_attn=1, pre_ff=2, post_ff=3, q_norm=4, k_norm=5)


def make_config(layers, hidden, q_heads, kv_heads, head_dim, ffn, vocab, max_len, max_lanes=1, eps=1e-6,
                rope_base=10000.0, tp_rank=0, tp_size=1, sliding_window=0, sliding_pattern=0, rope_local_base=0.0) -> ModelConfig:
    return ModelConfig(layers=layers, hidden=hidden, q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim, ffn=ffn,
                       vocab=vocab, group_size=64, bits=4, max_len=max_len, max_lanes=max_lanes, eps=eps,
                       rope_base=rope_base, attn_scale=0.0, embed_scale=0.0, tp_rank=tp_rank, tp_size=tp_size,
                       sliding_window=sliding_window, sliding_pattern=sliding_pattern, rope_local_base=rope_local_base)


def checkpoint_inspect(path: str) -> dict:
    """Host-side summary of a checkpoint directory (config.json + safetensors headers)."""
    import json
    buf = C.create_string_buffer(4096)
    check(lib().lthn_checkpoint_inspect(os.fsencode(path), buf, len(buf)))
    return json.loads(buf.value.decode())


class Model:
    """engine.TokenModel: resident weights + KV lanes (lthn_model_*)."""

    def __init__(self, cfg: ModelConfig):
        self.cfg = cfg
        h = C.c_void_p()
        check(lib().lthn_model_create(C.byref(cfg), C.byref(h)))
        self.h = h

    @classmethod
    def load_dir(cls, path: str, max_len=0, max_lanes=1, tp_rank=0, tp_size=1, comm=None, uniform_attention=False) -> "Model":
        """Backend.LoadModel for a checkpoint directory (lthn_model_load_dir)."""
        info = checkpoint_inspect(path)
        opts = LoadOptions(max_len=max_len, max_lanes=max_lanes, tp_rank=tp_rank, tp_size=tp_size, comm=comm,
                           uniform_attention=int(uniform_attention))
        h = C.c_void_p()
        check(lib().lthn_model_load_dir(os.fsencode(path), C.byref(opts), C.byref(h)))
        m = cls.__new__(cls)
        m.h = h
        m.cfg = make_config(info["layers"], info["hidden"], info["q_heads"], info["kv_heads"], info["head_dim"], info["ffn"],
                            info["vocab"], max_len, max_lanes, tp_rank=tp_rank, tp_size=tp_size)
        return m

    def upload_linear(self, layer, role, packed, scales, biases, bits=4):
        """bits=8: an MLP projection of a mixed-precision pack (one code per byte, group 64)."""
        pk = np.ascontiguousarray(packed, dtype=np.uint32)
        sc = np.ascontiguousarray(scales, dtype=np.uint16)
        bi = np.ascontiguousarray(biases, dtype=np.uint16)
        r = ROLE[role] if isinstance(role, str) else role
        if bits == 4:
            check(lib().lthn_model_upload_linear(self.h, layer, r, pk.ctypes.data, sc.ctypes.data, bi.ctypes.data,
                                                 pk.shape[0], pk.shape[1] * 8))
        else:
            check(lib().lthn_model_upload_linear_bits(self.h, layer, r, pk.ctypes.data, sc.ctypes.data, bi.ctypes.data,
                                                      pk.shape[0], pk.shape[1] * 32 // bits, bits))

    def upload_norm(self, layer, role, w):
        a = np.ascontiguousarray(w, dtype=np.float32)
        r = NORM[role] if isinstance(role, str) else role
        check(lib().lthn_model_upload_norm(self.h, layer, r, a.ctypes.data, a.size))

    def synthesize(self, seed, sigma=0.02):
        check(lib().lthn_model_synthesize(self.h, seed, sigma))

    def set_comm(self, comm):
        check(lib().lthn_model_set_comm(self.h, comm))

    def finalize(self):
        check(lib().lthn_model_finalize(self.h))

    @property
    def weight_bytes(self):
        v = C.c_uint64()
        check(lib().lthn_model_weight_bytes(self.h, C.byref(v)))
        return int(v.value)

    @property
    def tp_exchange(self):
        """0 single device, 1 NCCL all-reduce, 2 peer-memory exchange fused into the residual norm."""
        v = C.c_int32()
        check(lib().lthn_model_tp_exchange(self.h, C.byref(v)))
        return int(v.value)

    @property
    def decode_kernel(self):
        """0: per-op kernel chain, 1: one cooperative kernel per token (one row, one GPU)."""
        v = C.c_int32()
        check(lib().lthn_model_decode_kernel(self.h, C.byref(v)))
        return int(v.value)

    @property
    def graph_state(self):
        """0 decode steps not captured yet, 1 replaying a CUDA graph, 2 capture impossible (eager)."""
        v = C.c_int32()
        check(lib().lthn_model_graph_state(self.h, C.byref(v)))
        return int(v.value)

    def open_session(self) -> "Session":
        return Session(self)

    def open_lane_set(self, max_lanes=0) -> "LaneSet":
        return LaneSet(self, max_lanes)

    def close(self):
        if self.h:
            lib().lthn_model_destroy(self.h)
            self.h = None


class Session:
    """engine.Session over one KV lane."""

    def __init__(self, model: Model):
        self.model = model
        h = C.c_void_p()
        check(lib().lthn_session_open(model.h, C.byref(h)))
        self.h = h

    def prefill(self, ids):
        a = np.ascontiguousarray(ids, dtype=np.int32)
        check(lib().lthn_session_prefill(self.h, a.ctypes.data, a.size))

    def append(self, ids):
        a = np.ascontiguousarray(ids, dtype=np.int32)
        check(lib().lthn_session_append(self.h, a.ctypes.data, a.size))

    @property
    def pos(self):
        return int(lib().lthn_session_pos(self.h))

    def decode_greedy(self, max_new, eos_id=-1):
        out = np.empty(max(max_new, 1), dtype=np.int32)
        n = C.c_int32()
        check(lib().lthn_session_decode_greedy(self.h, max_new, eos_id, out.ctypes.data, C.byref(n)))
        return out[:n.value].copy()

    def decode_sampled(self, sampler: "Sampler", params: SampleParams, max_new, stop=()):
        out = np.empty(max(max_new, 1), dtype=np.int32)
        st = np.ascontiguousarray(stop, dtype=np.int32)
        n = C.c_int32()
        check(lib().lthn_session_decode_sampled(self.h, sampler.h, C.byref(params), max_new, st.ctypes.data if st.size else None,
                                                st.size, out.ctypes.data, C.byref(n)))
        return out[:n.value].copy()

    def trace_begin(self):
        """engine.DecodePhaseTracer.BeginDecodePhaseTrace; trace_end() is the stop function."""
        check(lib().lthn_session_trace_begin(self.h))

    def trace_end(self) -> DecodePhaseBudget:
        out = DecodePhaseBudget()
        check(lib().lthn_session_trace_end(self.h, C.byref(out)))
        return out

    def logits(self):
        n = self.model.cfg.vocab // max(1, self.model.cfg.tp_size)
        out = np.empty(n, dtype=np.float32)
        check(lib().lthn_session_logits(self.h, out.ctypes.data, n))
        return out

    def kv_export(self, layer, which):
        kr = self.model.cfg.kv_heads // max(1, self.model.cfg.tp_size) * self.model.cfg.head_dim
        out = np.empty((self.pos, kr), dtype=np.uint16)
        check(lib().lthn_session_kv_export(self.h, layer, which, out.ctypes.data, out.nbytes))
        return out

    def kv_import(self, layer, which, data):
        a = np.ascontiguousarray(data, dtype=np.uint16)
        check(lib().lthn_session_kv_import(self.h, layer, which, a.ctypes.data, a.shape[0]))

    def _kr(self, gathered=False):
        c = self.model.cfg
        return (c.kv_heads if gathered else c.kv_heads // max(1, c.tp_size)) * c.head_dim

    def kv_export_range(self, layer, which, token0, ntokens, gathered=False):
        out = np.empty((ntokens, self._kr(gathered)), dtype=np.uint16)
        fn = lib().lthn_session_kv_gather_range if gathered else lib().lthn_session_kv_export_range
        check(fn(self.h, layer, which, token0, ntokens, out.ctypes.data, out.nbytes))
        return out

    def kv_import_range(self, layer, which, token0, data):
        a = np.ascontiguousarray(data, dtype=np.uint16)
        check(lib().lthn_session_kv_import_range(self.h, layer, which, token0, a.ctypes.data, a.shape[0]))

    def range_kv_blocks(self, block_size, block_start_token=0):
        """Session.RangeKVBlocks: yields (index, token_start, token_count, {(layer, which): rows}) for the
        blocks that end after block_start_token (kv.CaptureOptions.BlockStartToken)."""
        pos, layers = self.pos, self.model.cfg.layers
        for index, t0 in enumerate(range(0, pos, block_size)):
            n = min(block_size, pos - t0)
            if t0 + n <= block_start_token:
                continue
            yield index, t0, n, {(li, w): self.kv_export_range(li, w, t0, n) for li in range(layers) for w in (0, 1)}

    def fork(self) -> "Session":
        f = Session.__new__(Session)
        f.model = self.model
        h = C.c_void_p()
        check(lib().lthn_session_fork(self.h, C.byref(h)))
        f.h = h
        return f

    def reset(self):
        check(lib().lthn_session_reset(self.h))

    def set_state(self, pos, pending):
        check(lib().lthn_session_set_state(self.h, pos, pending))

    def close(self):
        if self.h:
            lib().lthn_session_close(self.h)
            self.h = None


class LaneSet:
    """inference.LaneSet: K lanes advanced by one batched forward per step."""

    def __init__(self, model: Model, max_lanes=0):
        self.model = model
        h = C.c_void_p()
        check(lib().lthn_laneset_open(model.h, max_lanes, C.byref(h)))
        self.h = h

    def prepare(self, ids, max_new=0, stop=()):
        a = np.ascontiguousarray(ids, dtype=np.int32)
        st = np.ascontiguousarray(stop, dtype=np.int32)
        lane = C.c_int32()
        check(lib().lthn_laneset_prepare(self.h, a.ctypes.data, a.size, max_new, st.ctypes.data if st.size else None,
                                         st.size, C.byref(lane)))
        return int(lane.value)

    def prepare_sampled(self, ids, params: SampleParams, seed: int, max_new=0, stop=()):
        a = np.ascontiguousarray(ids, dtype=np.int32)
        st = np.ascontiguousarray(stop, dtype=np.int32)
        lane = C.c_int32()
        check(lib().lthn_laneset_prepare_sampled(self.h, a.ctypes.data, a.size, max_new, st.ctypes.data if st.size else None,
                                                 st.size, C.byref(params), seed, C.byref(lane)))
        return int(lane.value)

    def step(self):
        lanes = np.empty(32, dtype=np.int32)
        toks = np.empty(32, dtype=np.int32)
        flags = np.empty(32, dtype=np.int32)
        n = C.c_int32()
        check(lib().lthn_laneset_step(self.h, lanes.ctypes.data, toks.ctypes.data, flags.ctypes.data, C.byref(n)))
        return [(int(lanes[i]), int(toks[i]), bool(flags[i] & 1), bool(flags[i] & 2)) for i in range(n.value)]

    def retire(self, lane):
        check(lib().lthn_laneset_retire(self.h, lane))

    @property
    def active(self):
        return int(lib().lthn_laneset_active(self.h))

    @property
    def batch_forward_count(self):
        return int(lib().lthn_laneset_batch_forward_count(self.h))

    def close(self):
        if self.h:
            lib().lthn_laneset_close(self.h)
            self.h = None


def tensor_seed(seed, layer, role):
    """Seed of the synthetic tensor lthn_model_synthesize draws for (layer, role); layer -1 = embedding."""
    return (seed * 1000003 + (layer + 1) * 16 + role) & 0xFFFFFFFFFFFFFFFF
