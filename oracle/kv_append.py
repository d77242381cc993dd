"""TEST INFRASTRUCTURE: Python face of oracle/kv_append_oracle.c plus the rotary table restatement.

Arrays are numpy; bf16 travels as uint16 bit patterns. See the C file's header for what each function follows in
the reference and for the parity status of the quantise rule."""

import ctypes
import functools

import numpy as np

from . import build_oracle

HEAD_DIM = 128
HALF = 64


@functools.cache
def _lib() -> ctypes.CDLL:
    lib = ctypes.CDLL(str(build_oracle.build()))
    lib.oracle_kv_append.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                                                              ctypes.c_longlong] + [ctypes.c_void_p] * 6
    lib.oracle_kv_append.restype = None
    lib.oracle_kv_append_ve.argtypes = lib.oracle_kv_append.argtypes + [ctypes.c_void_p] * 4 + [ctypes.c_int]
    lib.oracle_kv_append_ve.restype = None
    lib.oracle_f32_to_e4m3_n.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong]
    lib.oracle_f32_to_e4m3_n.restype = None
    lib.oracle_quant_rows.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong]
    lib.oracle_quant_rows.restype = None
    lib.oracle_qk_row.argtypes = [ctypes.c_void_p] * 5
    lib.oracle_qk_row.restype = None
    return lib


def _p(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def rotary_table(positions: int, theta: float, head_dim: int = HEAD_DIM) -> tuple[np.ndarray, np.ndarray]:
    """cos, sin fp32 (positions, head_dim / 2) of the angles t theta^(-2i/D), computed in fp64 then rounded
    (reference: model/modeling.py:169-176, inference/modeling_nanochat.py:29-34)."""
    exponent = np.arange(0, head_dim, 2, dtype=np.float64) / head_dim
    freqs = np.arange(positions, dtype=np.float64)[:, None] * theta ** -exponent
    return np.cos(freqs).astype(np.float32), np.sin(freqs).astype(np.float32)


def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    """e4m3 bytes of fp32 values: round to nearest even, finite values saturate at +-448."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(x.shape, dtype=np.uint8)
    _lib().oracle_f32_to_e4m3_n(_p(x), _p(y), x.size)
    return y


E4M3_TABLE = np.array([(-1.0 if b & 0x80 else 1.0) * (float("nan") if (b & 0x7f) == 0x7f else
                       ((b & 7) * 2.0 ** -9 if ((b >> 3) & 15) == 0 else
                        (1 + (b & 7) / 8) * 2.0 ** (((b >> 3) & 15) - 7))) for b in range(256)], dtype=np.float32)


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    return E4M3_TABLE[b]


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (h.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round to nearest even (finite inputs)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7fff + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def quant_rows(x_bf16: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """x (..., 128) bf16 bit patterns -> (bytes (..., 128) u8, scale (...) fp32): scale = amax / 448,
    byte = e4m3(x / scale), zero rows give scale 0 and zero bytes."""
    x = np.ascontiguousarray(x_bf16, dtype=np.uint16)
    assert x.shape[-1] == HEAD_DIM
    rows = x.size // HEAD_DIM
    b = np.empty(x.shape, dtype=np.uint8)
    s = np.empty(x.shape[:-1], dtype=np.float32)
    _lib().oracle_quant_rows(_p(x), _p(b), _p(s), rows)
    return b, s


def kv_append(qkv: np.ndarray, q_gain: np.ndarray, k_gain: np.ndarray, cos: np.ndarray, sin: np.ndarray,
              pos: np.ndarray, Hq: int, Hkv: int, ve: "dict | None" = None) -> dict[str, np.ndarray]:
    """qkv (rows, (Hq + 2 Hkv) * 128) bf16 bit patterns; returns q (rows, Hq, 128) bf16 bits, k_bf16 (the rotated
    k before quantisation), k_bytes, v_bytes (rows, Hkv, 128) u8 and k_scale, v_scale (rows, Hkv) fp32.
    ve: the optional value-embedding mix on v (model/kernels/decode.cu:482-494): dict with h (rows, C) bf16 bits (the
    layer's normed input), tokens (rows,) int64, table (vocab, Hkv * 128) bf16 bits, gate (Hkv, C) fp32."""
    qkv = np.ascontiguousarray(qkv, dtype=np.uint16)
    rows, stride = qkv.shape
    assert stride >= (Hq + 2 * Hkv) * HEAD_DIM
    q_gain, k_gain = (np.ascontiguousarray(g, dtype=np.float32) for g in (q_gain, k_gain))
    cos, sin = (np.ascontiguousarray(t, dtype=np.float32) for t in (cos, sin))
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    assert pos.shape == (rows,) and (pos >= 0).all() and (pos < cos.shape[0]).all()
    out = {"q": np.empty((rows, Hq, HEAD_DIM), np.uint16), "k_bf16": np.empty((rows, Hkv, HEAD_DIM), np.uint16),
           "k_bytes": np.empty((rows, Hkv, HEAD_DIM), np.uint8), "k_scale": np.empty((rows, Hkv), np.float32),
           "v_bytes": np.empty((rows, Hkv, HEAD_DIM), np.uint8), "v_scale": np.empty((rows, Hkv), np.float32)}
    head = [_p(qkv), _p(q_gain), _p(k_gain), _p(cos), _p(sin), _p(pos), rows, Hq, Hkv, stride, _p(out["q"]),
            _p(out["k_bf16"]), _p(out["k_bytes"]), _p(out["k_scale"]), _p(out["v_bytes"]), _p(out["v_scale"])]
    if ve is None:
        _lib().oracle_kv_append(*head)
        return out
    h = np.ascontiguousarray(ve["h"], dtype=np.uint16)
    tokens = np.ascontiguousarray(ve["tokens"], dtype=np.int64)
    table = np.ascontiguousarray(ve["table"], dtype=np.uint16)
    gate = np.ascontiguousarray(ve["gate"], dtype=np.float32)
    C = h.shape[1]
    assert h.shape == (rows, C) and C % 256 == 0 and gate.shape == (Hkv, C) and table.shape[1] == Hkv * HEAD_DIM
    assert tokens.shape == (rows,) and (tokens >= 0).all() and (tokens < table.shape[0]).all()
    _lib().oracle_kv_append_ve(*head, _p(h), _p(tokens), _p(table), _p(gate), C)
    return out
