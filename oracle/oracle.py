"""ctypes loader for the CPU oracle (oracle/liblthn_oracle.so) plus a second,
independent NumPy restatement of the MLX-affine codec.

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's CPU-baseline legs as the checker / timed baseline. The shipped library
never imports or calls anything here.

The NumPy functions follow go/model/quant/mlxaffine/mlxaffine.go:80-241 (quantise,
dequantise, bf16 RNE) and the array formulation of tools/mlxaffine_dequant.py:47-60;
they exist so the C restatement can be checked against a differently-written one.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liblthn_oracle.so")


def build(force: bool = False) -> str:
    """Compile the C oracle with the committed Makefile (gcc, OpenMP)."""
    srcs = [os.path.join(_HERE, f) for f in ("lthn_oracle.c", "lthn_oracle_decoder.c", "Makefile")]
    stale = (not os.path.exists(_LIB_PATH)) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in srcs)
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-B"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _declare(_lib)
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


class DecoderConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("layers", "hidden", "q_heads", "kv_heads", "head_dim", "ffn", "vocab", "gs", "bits", "max_len")] + \
               [(n, C.c_float) for n in ("eps", "rope_base", "attn_scale", "embed_scale")] + \
               [("kv_bf16", C.c_int32), ("prefill_bf16", C.c_int32), ("sliding_window", C.c_int32), ("sliding_pattern", C.c_int32),
                ("rope_local_base", C.c_float)]


def _declare(l):
    vp, i32, i64, f32, f64, u64 = C.c_void_p, C.c_int, C.c_long, C.c_float, C.c_double, C.c_uint64
    l.lthn_o_f32_to_bf16.restype = C.c_uint16
    l.lthn_o_f32_to_bf16.argtypes = [f32]
    l.lthn_o_bf16_to_f32.restype = f32
    l.lthn_o_bf16_to_f32.argtypes = [C.c_uint16]
    l.lthn_o_num_threads.restype = i32
    l.lthn_o_quantize.argtypes = [vp, i64, i64, i32, i32, i32, vp, vp, vp]
    l.lthn_o_dequantize.argtypes = [vp, vp, vp, i64, i64, i32, i32, vp]
    l.lthn_o_affine_set_code.argtypes = [vp, i64, i32, C.c_uint32]
    l.lthn_o_affine_extract_code.restype = C.c_uint32
    l.lthn_o_affine_extract_code.argtypes = [vp, i64, i32]
    l.lthn_o_ref_affine_matvec.argtypes = [vp, i64, vp, i64, vp, i64, vp, i64, i64, i64, i32, i32, vp]
    l.lthn_o_hip_affine_projection.argtypes = [vp, vp, vp, vp, i64, i64, i32, i32, vp]
    l.lthn_o_hip_affine_projection_rows.argtypes = [vp, i64, vp, vp, vp, i64, i64, i32, i32, vp]
    l.lthn_o_matnt_quant_host.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i32, i32, i32]
    l.lthn_o_matnt.argtypes = [vp, vp, i64, i64, i64, vp]
    l.lthn_o_qmm_bf16.argtypes = [vp, vp, vp, vp, i64, i64, i64, i32, i32, vp]
    l.lthn_o_proj_bf16_contract.argtypes = [vp, i64, vp, vp, vp, i64, i64, i32, i32, vp]
    l.lthn_o_rmsnorm.argtypes = [vp, vp, i64, f32, vp]
    l.lthn_o_rope_neox.argtypes = [vp, i64, i64, f64, i64, i64, f64, vp]
    l.lthn_o_rope_interleaved.argtypes = [vp, i64, i64, f64, i64, f64, vp]
    l.lthn_o_qknorm_rope_bf16.argtypes = [vp, vp, i64, i64, i64, f32, f32, i64, f32, vp]
    l.lthn_o_attention_single_head.argtypes = [vp, vp, vp, i64, i64, i64, f32, vp, vp]
    l.lthn_o_kv_head_for_query.restype = i64
    l.lthn_o_kv_head_for_query.argtypes = [i64, i64, i64]
    l.lthn_o_gelu_tanh.argtypes = [vp, i64, vp]
    l.lthn_o_greedy_f32.restype = i64
    l.lthn_o_greedy_f32.argtypes = [vp, i64]
    l.lthn_o_greedy_bf16.restype = i64
    l.lthn_o_greedy_bf16.argtypes = [vp, i64]
    l.lthn_o_affine_embedding_row.argtypes = [vp, vp, vp, i64, i64, i32, i32, i64, vp]
    l.lthn_o_fold_norm_bias_one_f32.argtypes = [vp, i64, vp]
    l.lthn_o_fold_norm_bias_one_bf16.argtypes = [vp, i64, vp]
    l.lthn_o_synth_normal.restype = f32
    l.lthn_o_synth_normal.argtypes = [u64, u64, f32]
    l.lthn_o_synth_normal_fill.argtypes = [u64, u64, i64, f32, vp]
    l.lthn_o_round_bf16_inplace.argtypes = [vp, i64]
    l.lthn_o_decoder_create.restype = vp
    l.lthn_o_decoder_create.argtypes = [C.POINTER(DecoderConfig)]
    l.lthn_o_decoder_destroy.argtypes = [vp]
    l.lthn_o_decoder_set_linear.argtypes = [vp, i32, i32, vp, vp, vp, i64, i64]
    l.lthn_o_decoder_set_linear_bits.argtypes = [vp, i32, i32, i32]
    l.lthn_o_decoder_set_norm.argtypes = [vp, i32, i32, vp]
    l.lthn_o_decoder_pos.restype = i64
    l.lthn_o_decoder_pos.argtypes = [vp]
    l.lthn_o_decoder_reset.argtypes = [vp]
    l.lthn_o_decoder_set_tap.argtypes = [vp, i32, i32, vp]
    l.lthn_o_decoder_forward.argtypes = [vp, vp, i64, vp, vp]
    l.lthn_o_decoder_generate.argtypes = [vp, vp, i64, vp, vp]
    l.lthn_o_decoder_read_kv.argtypes = [vp, i32, i32, vp]


class OracleError(ValueError):
    """The oracle rejected its arguments (the reference returns an error here)."""


def _check(rc, what):
    if rc != 0:
        raise OracleError(f"{what}: rejected (rc={rc})")


# ----------------------------------------------------------------- codec ----

def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    """RNE f32 -> bf16 bit patterns (mlxaffine.go:229-236), vectorised."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)
    return np.where(nan, ((u >> 16) | 0x40).astype(np.uint16), r)


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def quantize(w: np.ndarray, bits: int = 4, gs: int = 64, variant: int = 0):
    """QuantizeTensor (mlxaffine.go:80-129). Returns (packed u32 [N,K*bits/32],
    scales u16 [N,K/gs], biases u16 [N,K/gs]). variant 1 = literal min/max rule."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    if w.ndim != 2:
        raise OracleError("quantize: want a 2-D weight")
    n, k = w.shape
    if bits not in (1, 2, 4, 8) or n <= 0 or k <= 0 or gs <= 0 or k % gs or gs % (32 // bits):
        raise OracleError("quantize: unsupported bits/shape/group")
    packed = np.zeros((n, k * bits // 32), dtype=np.uint32)
    scales = np.zeros((n, k // gs), dtype=np.uint16)
    biases = np.zeros((n, k // gs), dtype=np.uint16)
    _check(lib().lthn_o_quantize(_p(w), n, k, bits, gs, variant, _p(packed), _p(scales), _p(biases)), "quantize")
    return packed, scales, biases


def dequantize(packed, scales, biases, bits: int = 4, gs: int = 64) -> np.ndarray:
    """DequantizeTensor (mlxaffine.go:178-208) -> f32 [N,K]."""
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.uint16)
    biases = np.ascontiguousarray(biases, dtype=np.uint16)
    n = packed.shape[0]
    k = packed.shape[1] * 32 // bits
    if scales.shape != (n, k // gs) or biases.shape != scales.shape:
        raise OracleError("dequantize: scales/biases do not match [N, K/gs]")
    out = np.empty((n, k), dtype=np.float32)
    _check(lib().lthn_o_dequantize(_p(packed), _p(scales), _p(biases), n, k, bits, gs, _p(out)), "dequantize")
    return out


def np_dequantize(packed, scales, biases, bits: int = 4, gs: int = 64) -> np.ndarray:
    """Independent array-style dequantiser (formulation of tools/mlxaffine_dequant.py:47-60)."""
    words = np.ascontiguousarray(packed, dtype=np.uint32)
    n = words.shape[0]
    per_word = 32 // bits
    shifts = (np.arange(per_word, dtype=np.uint32) * bits).astype(np.uint32)
    codes = ((words[..., None] >> shifts) & np.uint32((1 << bits) - 1)).reshape(n, -1)
    s = np.repeat(bf16_to_f32(scales), gs, axis=1)
    b = np.repeat(bf16_to_f32(biases), gs, axis=1)
    return (codes.astype(np.float32) * s + b).astype(np.float32)


def np_quantize(w: np.ndarray, bits: int = 4, gs: int = 64, variant: int = 0):
    """Independent vectorised QuantizeTensor (mlxaffine.go:80-173) in f32 NumPy."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    g = w.reshape(n, k // gs, gs)
    nb = np.float32((1 << bits) - 1)
    wmin = g.min(axis=2)
    wmax = g.max(axis=2)
    scale = ((wmax - wmin) / nb).astype(np.float32)
    scale = np.maximum(scale, np.float32(1e-7))
    if variant == 1:
        bias = wmin
    else:
        min_dom = np.abs(wmin) > np.abs(wmax)
        edge = np.where(min_dom, wmin, wmax).astype(np.float32)
        scale = np.where(min_dom, scale, -scale).astype(np.float32)
        with np.errstate(divide="ignore", invalid="ignore"):
            q0 = _round_half_away((edge / scale).astype(np.float32))
            scale = np.where(q0 == 0, scale, (edge / np.where(q0 == 0, np.float32(1), q0)).astype(np.float32))
        bias = np.where(q0 == 0, np.float32(0), edge).astype(np.float32)
    q = _round_half_away(((g - bias[..., None]) / scale[..., None]).astype(np.float32))
    q = np.clip(q, 0, nb).astype(np.uint32).reshape(n, k)
    per_word = 32 // bits
    shifts = (np.arange(per_word, dtype=np.uint32) * bits).astype(np.uint32)
    packed = (q.reshape(n, k // per_word, per_word) << shifts).sum(axis=2, dtype=np.uint64).astype(np.uint32)
    return packed, f32_to_bf16(scale.astype(np.float32)), f32_to_bf16(bias.astype(np.float32))


def _round_half_away(v: np.ndarray) -> np.ndarray:
    v64 = v.astype(np.float64)
    return (np.sign(v64) * np.floor(np.abs(v64) + 0.5)).astype(np.float32)


# --------------------------------------------------------------- matvec -----

def ref_affine_matvec(x_bf16, packed_bytes, scales_bytes, biases_bytes, out_dim, in_dim, gs, bits) -> np.ndarray:
    """ReferenceAffineMatVec (enginetest/quant_reference.go:79-127); byte arrays in, bf16 u16 out."""
    x = np.ascontiguousarray(x_bf16).view(np.uint8).reshape(-1)
    p = np.ascontiguousarray(packed_bytes).view(np.uint8).reshape(-1)
    s = np.ascontiguousarray(scales_bytes).view(np.uint8).reshape(-1)
    b = np.ascontiguousarray(biases_bytes).view(np.uint8).reshape(-1)
    out = np.zeros(max(out_dim, 0), dtype=np.uint16)
    _check(lib().lthn_o_ref_affine_matvec(_p(x), x.size, _p(p), p.size, _p(s), s.size, _p(b), b.size,
                                          out_dim, in_dim, gs, bits, _p(out)), "ref_affine_matvec")
    return out


def hip_affine_projection(x_f32, words, scales, biases, rows, cols, gs, bits=4) -> np.ndarray:
    """hipReferenceMLXAffineProjection (engine/hip/hip_projection_reference.go:92-116)."""
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    w = np.ascontiguousarray(words, dtype=np.uint32)
    s = np.ascontiguousarray(scales, dtype=np.uint16)
    b = np.ascontiguousarray(biases, dtype=np.uint16)
    if x.size != cols or (bits in (4, 6, 8) and w.size != rows * (cols * bits // 32)) or \
            (gs > 0 and cols % gs == 0 and (s.size != rows * (cols // gs) or b.size != s.size)):
        raise OracleError("hip_affine_projection: shape mismatch")
    out = np.empty(rows, dtype=np.float32)
    _check(lib().lthn_o_hip_affine_projection(_p(x), _p(w), _p(s), _p(b), rows, cols, gs, bits, _p(out)),
           "hip_affine_projection")
    return out


def hip_affine_projection_rows(x_f32, words, scales, biases, gs=64, bits=4) -> np.ndarray:
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    w = np.ascontiguousarray(words, dtype=np.uint32)
    t, cols = x.shape
    rows = w.shape[0]
    out = np.empty((t, rows), dtype=np.float32)
    _check(lib().lthn_o_hip_affine_projection_rows(_p(x), t, _p(w), _p(np.ascontiguousarray(scales)),
                                                   _p(np.ascontiguousarray(biases)), rows, cols, gs, bits, _p(out)),
           "hip_affine_projection_rows")
    return out


def matnt_quant_host(x_f32, packed, scales, biases, gs=64, bits=4, threads=1) -> np.ndarray:
    """attn.matNTQuantHost (model/attn/gated_delta.go:63-89): out[M,N] f32, f64 accumulate."""
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    if x.ndim == 1:
        x = x[None, :]
    m, k = x.shape
    pk = np.ascontiguousarray(packed, dtype=np.uint32)
    n = pk.shape[0]
    out = np.empty((m, n), dtype=np.float32)
    _check(lib().lthn_o_matnt_quant_host(_p(out), _p(x), _p(pk), _p(np.ascontiguousarray(scales, dtype=np.uint16)),
                                         _p(np.ascontiguousarray(biases, dtype=np.uint16)), m, k, n, gs, bits, threads),
           "matnt_quant_host")
    return out


def matnt(x_f32, w_f32) -> np.ndarray:
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    w = np.ascontiguousarray(w_f32, dtype=np.float32)
    out = np.empty((x.shape[0], w.shape[0]), dtype=np.float32)
    lib().lthn_o_matnt(_p(x), _p(w), x.shape[0], x.shape[1], w.shape[0], _p(out))
    return out


def qmm_bf16(x_bf16, packed, scales, biases, gs=64, bits=4) -> np.ndarray:
    x = np.ascontiguousarray(x_bf16, dtype=np.uint16)
    pk = np.ascontiguousarray(packed, dtype=np.uint32)
    m, k = x.shape
    n = pk.shape[0]
    out = np.empty((m, n), dtype=np.uint16)
    _check(lib().lthn_o_qmm_bf16(_p(x), _p(pk), _p(np.ascontiguousarray(scales, dtype=np.uint16)),
                                 _p(np.ascontiguousarray(biases, dtype=np.uint16)), m, k, n, gs, bits, _p(out)), "qmm_bf16")
    return out


def proj_bf16_contract(x_f32, packed, scales, biases, gs=64, bits=4) -> np.ndarray:
    """The tensor-core contract with f32 results: x and the dequantised weights rounded to bf16,
    f64 accumulation, no output rounding (lthn_o_proj_bf16_contract). out [M, N] f32."""
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    if x.ndim == 1:
        x = x[None, :]
    pk = np.ascontiguousarray(packed, dtype=np.uint32)
    m, k = x.shape
    n = pk.shape[0]
    out = np.empty((m, n), dtype=np.float32)
    _check(lib().lthn_o_proj_bf16_contract(_p(x), m, _p(pk), _p(np.ascontiguousarray(scales, dtype=np.uint16)),
                                           _p(np.ascontiguousarray(biases, dtype=np.uint16)), n, k, gs, bits, _p(out)),
           "proj_bf16_contract")
    return out


# ------------------------------------------------------ transformer refs ----

def rmsnorm(x, w, eps) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    if w.size != x.size:
        raise OracleError("rmsnorm: weight length must match input length")
    out = np.empty_like(x)
    _check(lib().lthn_o_rmsnorm(_p(x), _p(w), x.size, eps, _p(out)), "rmsnorm")
    return out


def rope_neox(x, position, base, freq_dim=0, rotary=0, freq_scale=1.0) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    _check(lib().lthn_o_rope_neox(_p(x), x.size, position, base, freq_dim, rotary, freq_scale, _p(out)), "rope_neox")
    return out


def rope_interleaved(x, position, base, freq_dim=0, freq_scale=1.0) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    _check(lib().lthn_o_rope_interleaved(_p(x), x.size, position, base, freq_dim, freq_scale, _p(out)), "rope")
    return out


def qknorm_rope_bf16(x_bf16, w_bf16, heads, head_dim, rotary, eps, scale, position, log2_theta) -> np.ndarray:
    x = np.ascontiguousarray(x_bf16, dtype=np.uint16)
    w = np.ascontiguousarray(w_bf16, dtype=np.uint16)
    out = np.empty_like(x)
    _check(lib().lthn_o_qknorm_rope_bf16(_p(x), _p(w), heads, head_dim, rotary, eps, scale, position, log2_theta,
                                         _p(out)), "qknorm_rope_bf16")
    return out


def attention_single_head(q, keys, values, scale=0.0) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.float32)
    keys = np.ascontiguousarray(keys, dtype=np.float32)
    values = np.ascontiguousarray(values, dtype=np.float32)
    count, dim = keys.shape
    out = np.empty(dim, dtype=np.float32)
    scratch = np.empty(count, dtype=np.float32)
    _check(lib().lthn_o_attention_single_head(_p(q), _p(keys), _p(values), count, dim, dim, scale, _p(out),
                                              _p(scratch)), "attention")
    return out


def gelu_tanh(x) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    lib().lthn_o_gelu_tanh(_p(x), x.size, _p(out))
    return out


def greedy_f32(logits) -> int:
    a = np.ascontiguousarray(logits, dtype=np.float32)
    return int(lib().lthn_o_greedy_f32(_p(a), a.size))


def greedy_bf16(logits_u16) -> int:
    a = np.ascontiguousarray(logits_u16, dtype=np.uint16)
    return int(lib().lthn_o_greedy_bf16(_p(a), a.size))


def synth_normal(seed: int, first: int, n: int, sigma: float) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().lthn_o_synth_normal_fill(seed, first, n, sigma, _p(out))
    return out


# ---------------------------------------------------------------- decoder ---

ROLE = dict(q=0, k=1, v=2, o=3, gate=4, up=5, down=6)
NORM = dict(input=0, post_attn=1, pre_ff=2, post_ff=3, q_norm=4, k_norm=5)


class Decoder:
    """CPU reference decoder (see lthn_oracle_decoder.c). Keeps the arrays alive."""

    def __init__(self, cfg: DecoderConfig):
        self.cfg = cfg
        self._keep = []
        self.h = lib().lthn_o_decoder_create(C.byref(cfg))

    def set_linear(self, layer, role, packed, scales, biases, bits=None):
        """bits: the linear's own code width where a quantization override gives one (default: the model's)."""
        pk = np.ascontiguousarray(packed, dtype=np.uint32)
        s = np.ascontiguousarray(scales, dtype=np.uint16)
        b = np.ascontiguousarray(biases, dtype=np.uint16)
        self._keep += [pk, s, b]
        rows, cols = pk.shape[0], pk.shape[1] * 32 // (bits or self.cfg.bits)
        r = ROLE[role] if isinstance(role, str) else role
        _check(lib().lthn_o_decoder_set_linear(self.h, layer, r, _p(pk), _p(s), _p(b), rows, cols), "set_linear")
        if bits and bits != self.cfg.bits:
            _check(lib().lthn_o_decoder_set_linear_bits(self.h, layer, r, bits), "set_linear_bits")

    def set_norm(self, layer, role, w):
        a = np.ascontiguousarray(w, dtype=np.float32)
        self._keep.append(a)
        r = NORM[role] if isinstance(role, str) else role
        _check(lib().lthn_o_decoder_set_norm(self.h, layer, r, _p(a)), "set_norm")

    @property
    def pos(self):
        return int(lib().lthn_o_decoder_pos(self.h))

    def reset(self):
        lib().lthn_o_decoder_reset(self.h)

    def forward(self, ids, want_hidden=False):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        logits = np.empty(self.cfg.vocab, dtype=np.float32)
        hidden = np.empty(self.cfg.hidden, dtype=np.float32) if want_hidden else None
        _check(lib().lthn_o_decoder_forward(self.h, _p(ids), ids.size, _p(logits), _p(hidden)), "decoder_forward")
        return (logits, hidden) if want_hidden else logits

    def generate(self, first_logits, max_new):
        out = np.empty(max_new, dtype=np.int32)
        margin = np.empty(max_new, dtype=np.float32)
        fl = np.ascontiguousarray(first_logits, dtype=np.float32)
        _check(lib().lthn_o_decoder_generate(self.h, _p(fl), max_new, _p(out), _p(margin)), "decoder_generate")
        return out, margin

    def tap(self, layer, which, tokens, width):
        buf = np.zeros((tokens, width), dtype=np.float32)
        self._keep.append(buf)
        lib().lthn_o_decoder_set_tap(self.h, layer, which, _p(buf))
        return buf

    def read_kv(self, layer, which):
        kr = self.cfg.kv_heads * self.cfg.head_dim
        out = np.empty((self.pos, kr), dtype=np.float32)
        lib().lthn_o_decoder_read_kv(self.h, layer, which, _p(out))
        return out

    def close(self):
        if self.h:
            lib().lthn_o_decoder_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
