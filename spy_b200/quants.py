"""Block formats of the quantized weight types on the hot path, in numpy.

Encoders and decoders for the on-disk (= in-memory) block layouts the
reference declares in ``orchestration/include/number/number_impl/quant.h:10-33``
(Q4_0, 18 B / 32), ``quant.h:124-147`` (Q8_0, 34 B / 32) and
``k-quant.h:79-117`` / ``k-quant.h:162-188`` (Q4_K 144 B / 256, Q6_K 210 B / 256).

These run on the host only, to build synthetic GGUF models and to state the
block layout for tests; the GPU kernels read the same bytes.
"""
from __future__ import annotations

import numpy as np

# NumberType numbering (orchestration/include/number/number_impl/type.h:12-45) == GGML type ids
FP32, FP16, Q4_0, Q8_0, Q4_K, Q6_K, INT32 = 0, 1, 2, 8, 12, 14, 26

BLOCK_ELEMS = {FP32: 1, FP16: 1, Q4_0: 32, Q8_0: 32, Q4_K: 256, Q6_K: 256, INT32: 1}
BLOCK_BYTES = {FP32: 4, FP16: 2, Q4_0: 18, Q8_0: 34, Q4_K: 144, Q6_K: 210, INT32: 4}
TYPE_NAMES = {FP32: "f32", FP16: "f16", Q4_0: "q4_0", Q8_0: "q8_0", Q4_K: "q4_k", Q6_K: "q6_k"}
NAME_TO_TYPE = {v: k for k, v in TYPE_NAMES.items()}


def row_bytes(number_type: int, num_element: int) -> int:
    """get_row_size (orchestration/include/number/number.h:61-63)."""
    return num_element * BLOCK_BYTES[number_type] // BLOCK_ELEMS[number_type]


def _blocks(x: np.ndarray, n: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    if x.shape[-1] % n != 0:
        raise ValueError(f"row length {x.shape[-1]} is not a multiple of the block size {n}")
    return x.reshape(-1, n)


# --------------------------------------------------------------------------- Q4_0
def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    """f32 [..., K] -> uint8 [..., K/32*18]. Scale = (signed value of largest magnitude) / -8;
    element k < 16 is the low nibble of byte k, element 16 + k the high nibble."""
    b = _blocks(x, 32)
    idx = np.argmax(np.abs(b), axis=1)
    vmax = b[np.arange(b.shape[0]), idx]
    d = (vmax / np.float32(-8.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    q = (b * inv[:, None] + np.float32(8.5)).astype(np.float32)
    q = np.minimum(q.astype(np.int32), 15).astype(np.uint8)  # truncation toward zero; values are >= 0
    out = np.empty((b.shape[0], 18), dtype=np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(*x.shape[:-1], x.shape[-1] // 32 * 18)


def dequantize_q4_0(raw: np.ndarray) -> np.ndarray:
    r = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1, 18)
    d = r[:, 0:2].copy().view(np.float16).astype(np.float32)
    qs = r[:, 2:]
    lo = (qs & 0xF).astype(np.int8) - 8
    hi = (qs >> 4).astype(np.int8) - 8
    y = np.concatenate([lo, hi], axis=1).astype(np.float32) * d
    return y.reshape(*raw.shape[:-1], raw.shape[-1] // 18 * 32)


# --------------------------------------------------------------------------- Q8_0
def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """f32 [..., K] -> uint8 [..., K/32*34] (weight-side encoder: round half away from zero)."""
    b = _blocks(x, 32)
    amax = np.max(np.abs(b), axis=1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    v = (b * inv[:, None]).astype(np.float32)
    q = (np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))).astype(np.int8)
    out = np.empty((b.shape[0], 34), dtype=np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(*x.shape[:-1], x.shape[-1] // 32 * 34)


def dequantize_q8_0(raw: np.ndarray) -> np.ndarray:
    r = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1, 34)
    d = r[:, 0:2].copy().view(np.float16).astype(np.float32)
    q = r[:, 2:].view(np.int8).astype(np.float32)
    return (q * d).reshape(*raw.shape[:-1], raw.shape[-1] // 34 * 32)


# --------------------------------------------------------------------------- Q4_K
def _unpack_scale_min_k4(scales: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """12 packed bytes -> 8 six-bit scales and 8 six-bit mins per super-block."""
    s = scales.astype(np.uint8)
    sc = np.empty((s.shape[0], 8), dtype=np.uint8)
    mn = np.empty((s.shape[0], 8), dtype=np.uint8)
    sc[:, :4] = s[:, 0:4] & 63
    mn[:, :4] = s[:, 4:8] & 63
    sc[:, 4:] = (s[:, 8:12] & 0xF) | ((s[:, 0:4] >> 6) << 4)
    mn[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    return sc, mn


def _pack_scale_min_k4(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    out = np.zeros((sc.shape[0], 12), dtype=np.uint8)
    out[:, 0:4] = (sc[:, :4] & 63) | ((sc[:, 4:] >> 4) << 6)
    out[:, 4:8] = (mn[:, :4] & 63) | ((mn[:, 4:] >> 4) << 6)
    out[:, 8:12] = (sc[:, 4:] & 0xF) | ((mn[:, 4:] & 0xF) << 4)
    return out


def quantize_q4_k(x: np.ndarray) -> np.ndarray:
    """f32 [..., K] -> uint8 [..., K/256*144]. A plain min/max encoder: per 32-element
    sub-block value = d*sc*q - dmin*m with q in 0..15, sc and m six-bit."""
    b = _blocks(x, 256).reshape(-1, 8, 32)
    lo = np.minimum(b.min(axis=2), 0.0)
    hi = np.maximum(b.max(axis=2), 0.0)
    scale = (hi - lo) / np.float32(15.0)
    minv = -lo
    d = (scale.max(axis=1) / np.float32(63.0)).astype(np.float16)
    dmin = (minv.max(axis=1) / np.float32(63.0)).astype(np.float16)
    d32, dmin32 = d.astype(np.float32), dmin.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(d32[:, None] > 0, np.rint(scale / d32[:, None]), 0).clip(0, 63).astype(np.uint8)
        mn = np.where(dmin32[:, None] > 0, np.rint(minv / dmin32[:, None]), 0).clip(0, 63).astype(np.uint8)
        eff = d32[:, None] * sc.astype(np.float32)
        off = dmin32[:, None] * mn.astype(np.float32)
        q = np.where(eff[:, :, None] > 0, np.rint((b + off[:, :, None]) / eff[:, :, None]), 0).clip(0, 15).astype(np.uint8)
    out = np.empty((b.shape[0], 144), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(-1, 2)
    out[:, 4:16] = _pack_scale_min_k4(sc, mn)
    q = q.reshape(-1, 4, 2, 32)  # 64-element groups: low nibbles = first 32, high nibbles = next 32
    out[:, 16:] = (q[:, :, 0, :] | (q[:, :, 1, :] << 4)).reshape(-1, 128)
    return out.reshape(*x.shape[:-1], x.shape[-1] // 256 * 144)


def dequantize_q4_k(raw: np.ndarray) -> np.ndarray:
    r = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1, 144)
    d = r[:, 0:2].copy().view(np.float16).astype(np.float32)
    dmin = r[:, 2:4].copy().view(np.float16).astype(np.float32)
    sc, mn = _unpack_scale_min_k4(r[:, 4:16])
    qs = r[:, 16:].reshape(-1, 4, 32)
    q = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(-1, 8, 32).astype(np.float32)
    y = (d * sc.astype(np.float32))[:, :, None] * q - (dmin * mn.astype(np.float32))[:, :, None]
    return y.reshape(*raw.shape[:-1], raw.shape[-1] // 144 * 256).astype(np.float32)


# --------------------------------------------------------------------------- Q6_K
def quantize_q6_k(x: np.ndarray) -> np.ndarray:
    """f32 [..., K] -> uint8 [..., K/256*210]. value = d * sc * q, q in -32..31, sc int8 per 16 elements."""
    b = _blocks(x, 256).reshape(-1, 16, 16)
    amax = np.abs(b).max(axis=2)
    scale = amax / np.float32(31.0)
    d = (scale.max(axis=1) / np.float32(127.0)).astype(np.float16)
    d32 = d.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(d32[:, None] > 0, np.rint(scale / d32[:, None]), 0).clip(0, 127).astype(np.int8)
        eff = d32[:, None] * sc.astype(np.float32)
        q = np.where(eff[:, :, None] > 0, np.rint(b / eff[:, :, None]), 0).clip(-32, 31).astype(np.int8)
    u = (q.reshape(-1, 256).astype(np.int16) + 32).astype(np.uint8)  # 0..63
    u = u.reshape(-1, 2, 4, 32)  # half, quarter (l, l+32, l+64, l+96), l
    ql = np.empty((u.shape[0], 2, 64), dtype=np.uint8)
    ql[:, :, :32] = (u[:, :, 0, :] & 0xF) | ((u[:, :, 2, :] & 0xF) << 4)
    ql[:, :, 32:] = (u[:, :, 1, :] & 0xF) | ((u[:, :, 3, :] & 0xF) << 4)
    qh = (u[:, :, 0, :] >> 4) | ((u[:, :, 1, :] >> 4) << 2) | ((u[:, :, 2, :] >> 4) << 4) | ((u[:, :, 3, :] >> 4) << 6)
    out = np.empty((u.shape[0], 210), dtype=np.uint8)
    out[:, 0:128] = ql.reshape(-1, 128)
    out[:, 128:192] = qh.reshape(-1, 64)
    out[:, 192:208] = sc.view(np.uint8)
    out[:, 208:210] = d.view(np.uint8).reshape(-1, 2)
    return out.reshape(*x.shape[:-1], x.shape[-1] // 256 * 210)


def dequantize_q6_k(raw: np.ndarray) -> np.ndarray:
    r = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1, 210)
    ql = r[:, 0:128].reshape(-1, 2, 64)
    qh = r[:, 128:192].reshape(-1, 2, 32)
    sc = r[:, 192:208].copy().view(np.int8).astype(np.float32)
    d = r[:, 208:210].copy().view(np.float16).astype(np.float32)
    u = np.empty((r.shape[0], 2, 4, 32), dtype=np.int16)
    u[:, :, 0, :] = (ql[:, :, :32] & 0xF) | (((qh >> 0) & 3) << 4)
    u[:, :, 1, :] = (ql[:, :, 32:] & 0xF) | (((qh >> 2) & 3) << 4)
    u[:, :, 2, :] = (ql[:, :, :32] >> 4) | (((qh >> 4) & 3) << 4)
    u[:, :, 3, :] = (ql[:, :, 32:] >> 4) | (((qh >> 6) & 3) << 4)
    q = (u - 32).reshape(-1, 16, 16).astype(np.float32)
    y = q * (d * sc)[:, :, None]
    return y.reshape(*raw.shape[:-1], raw.shape[-1] // 210 * 256).astype(np.float32)


QUANTIZE = {Q4_0: quantize_q4_0, Q8_0: quantize_q8_0, Q4_K: quantize_q4_k, Q6_K: quantize_q6_k}
DEQUANTIZE = {Q4_0: dequantize_q4_0, Q8_0: dequantize_q8_0, Q4_K: dequantize_q4_k, Q6_K: dequantize_q6_k}


def quantize(x: np.ndarray, number_type: int) -> np.ndarray:
    if number_type == FP32:
        return np.ascontiguousarray(x, dtype=np.float32).view(np.uint8)
    if number_type == FP16:
        return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint8)
    return QUANTIZE[number_type](x)


def dequantize(raw: np.ndarray, number_type: int) -> np.ndarray:
    if number_type == FP32:
        return np.ascontiguousarray(raw).view(np.float32)
    if number_type == FP16:
        return np.ascontiguousarray(raw).view(np.float16).astype(np.float32)
    return DEQUANTIZE[number_type](raw)


# ---------------------------------------------------------------------------------------------
# e4m3 codes of small integers, as the prompt GEMM feeds them to the tensor cores (spyb_prefill.cu: a Q4_0 weight nibble - 8
# directly; an 8-bit value y as the two codes of y - y mod 16 and y mod 16). Kept here for tools that want to read or build
# the kernel's operand tiles on the host, and checked against an independent e4m3 decoder in the tests.
def e4m3_of_small(v: int) -> int:
    """Code of the integer 0 <= v <= 15 (exact: three mantissa bits cover 8..15)."""
    if v == 0:
        return 0
    e = v.bit_length() - 1
    return ((e + 7) << 3) | ((v << (3 - e)) & 7)


def e4m3_of_signed(v: int) -> int:
    return (0x80 | e4m3_of_small(-v)) if v < 0 else e4m3_of_small(v)


def e4m3_split(y: int) -> tuple[int, int]:
    """(code of y - y mod 16, code of y mod 16) for -128 <= y <= 127."""
    yl = y & 15
    yh = (y - yl) >> 4
    return (0 if yh == 0 else e4m3_of_signed(yh) + 0x20), e4m3_of_small(yl)

