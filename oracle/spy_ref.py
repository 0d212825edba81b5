"""Test infrastructure: ctypes binding of oracle/_ref/libspy_ref.so, the reference's own
CPU path compiled unmodified (see oracle/Makefile, oracle/ref_driver.cpp).

Only tests/, the fixture generator under tests/golden/, smoke() and bench.py's CPU
baseline may import this module; the product package never does.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libspy_ref.so")
# the same reference sources with the sm_100a backend registered through the reference's device-backend hook
# (adapter spy_b200/adapter/b200_backend.cpp): the reference's graph / scheduler / loader driving libspyb200.so
LIB_B200_PATH = os.path.join(_HERE, "_ref", "libspy_ref_b200.so")

# OperatorType numbering (orchestration/include/operator/type.h:38-52)
OP = dict(Input=0, Nop=1, Dup=2, Copy=3, View=4, Reshape=5, MaskedCopy=6, MaskedSelect=7, GetRow=8,
          Transpose=9, Permute=10, Contiguous=11, Relu=12, Silu=13, Gelu=14, Max=15, Min=16, Softmax=17,
          Add=18, Sub=19, Mul=20, Div=21, Mod=22, MatMul=23, Sum=24, Norm=25, NormRMS=26, Rope=27, Quantize=28)


class Tensor(C.Structure):
    _fields_ = [("number_type", C.c_int32), ("dim", C.c_int32), ("ne", C.c_int64 * 4), ("nb", C.c_int64 * 4),
                ("data", C.c_void_p)]


class OpParam(C.Structure):
    _fields_ = [("scale", C.c_float), ("eps", C.c_float), ("rope_mode", C.c_int32), ("num_past", C.c_int32),
                ("num_dim", C.c_int32), ("num_context", C.c_int32), ("num_origin_context", C.c_int32),
                ("freq_base", C.c_float), ("freq_scale", C.c_float), ("extend_factor", C.c_float),
                ("attention_factor", C.c_float), ("beta_fast", C.c_float), ("beta_slow", C.c_float)]


_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        l = C.CDLL(LIB_PATH)
        l.spy_ref_init.argtypes = [C.c_int]
        l.spy_ref_quantize_q8_0.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
        l.spy_ref_quantize_q8_0.restype = None
        l.spy_ref_quantize_f16.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
        l.spy_ref_quantize_f16.restype = None
        l.spy_ref_dot.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64]
        l.spy_ref_dot.restype = C.c_float
        l.spy_ref_tables.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        l.spy_ref_tables.restype = None
        l.spy_ref_run_op.argtypes = [C.c_int, C.c_int, C.POINTER(Tensor), C.POINTER(Tensor), C.POINTER(OpParam), C.c_int]
        l.spy_ref_generate.argtypes = [C.c_char_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                       C.c_void_p, C.c_void_p, C.c_void_p]
        _lib = l
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.size // 32 * 34, dtype=np.uint8)
    lib().spy_ref_quantize_q8_0(_ptr(x), x.size, _ptr(out))
    return out


def quantize_f16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.size, dtype=np.uint16)
    lib().spy_ref_quantize_f16(_ptr(x), x.size, _ptr(out))
    return out


DOT_Q4_0_Q8_0, DOT_Q8_0_Q8_0, DOT_F16_F16 = 0, 1, 2


def dot(kind: int, w: np.ndarray, x: np.ndarray, n: int) -> float:
    return float(lib().spy_ref_dot(kind, _ptr(w), _ptr(x), n))


def tables():
    f32 = np.empty(65536, dtype=np.float32)
    silu = np.empty(65536, dtype=np.float32)
    exp = np.empty(65536, dtype=np.float32)
    lib().spy_ref_tables(_ptr(f32), _ptr(silu), _ptr(exp))
    return f32, silu, exp


def make_tensor(a: np.ndarray, number_type: int, ne, nb=None) -> Tensor:
    t = Tensor()
    t.number_type = number_type
    t.dim = len(ne)
    for i in range(4):
        t.ne[i] = ne[i] if i < len(ne) else 1
        t.nb[i] = (nb[i] if (nb is not None and i < len(nb)) else 0)
    t.data = a.ctypes.data
    return t


def run_op(op: str, inputs: list, out_buf: np.ndarray, param: OpParam | None = None, threads: int = 4) -> Tensor:
    arr = (Tensor * len(inputs))(*inputs)
    out = Tensor()
    out.data = out_buf.ctypes.data
    p = param if param is not None else OpParam()
    rc = lib().spy_ref_run_op(OP[op], len(inputs), arr, C.byref(out), C.byref(p), threads)
    if rc != 0:
        raise RuntimeError(f"spy_ref_run_op({op}) failed: {rc}")
    return out


_lib_b200 = None


def b200_available() -> bool:
    return os.path.exists(LIB_B200_PATH)


def lib_b200():
    global _lib_b200
    if _lib_b200 is None:
        l = C.CDLL(LIB_B200_PATH)
        l.spy_ref_generate.argtypes = [C.c_char_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                       C.c_void_p, C.c_void_p, C.c_void_p]
        _lib_b200 = l
    return _lib_b200


def generate(gguf_path: str, prompt, n_predict: int, n_ctx: int = 512, threads: int = 8, warmup: bool = False,
             want_logits: bool = True, n_vocab: int | None = None, device_backend: bool = False, plan: bool = False):
    """Returns (ids [n_predict], logits [n_predict, n_vocab] or None, step_ms [n_predict]).
    device_backend=True runs the reference's token loop on its "gpu:b200" backend (the adapter over libspyb200.so),
    operator by operator or, with plan=True, with the steps served from the library's fused step plan."""
    prompt = np.ascontiguousarray(prompt, dtype=np.int32)
    ids = np.zeros(n_predict, dtype=np.int32)
    ms = np.zeros(n_predict, dtype=np.float64)
    logits = None
    if want_logits:
        if n_vocab is None:
            raise ValueError("n_vocab is required to size the logits buffer")
        logits = np.zeros((n_predict, n_vocab), dtype=np.float32)
    l = lib_b200() if device_backend else lib()
    v = l.spy_ref_generate(gguf_path.encode(), _ptr(prompt), len(prompt), n_predict, n_ctx, (-2 if plan else -1) if device_backend else threads, int(warmup),
                           _ptr(ids), _ptr(logits) if logits is not None else None, _ptr(ms))
    if v < 0:
        raise RuntimeError("spy_ref_generate failed")
    return ids, logits, ms
