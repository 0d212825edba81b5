"""Test infrastructure: ctypes binding of oracle/libspy_oracle.so (spy_oracle.c), the plain-C
restatement of the reference CPU algorithm. Only tests/, smoke() and bench.py's CPU-baseline
leg may import this; the product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libspy_oracle.so")

T_F32, T_F16, T_Q4_0, T_Q8_0, T_Q4_K, T_Q6_K = 0, 1, 2, 8, 12, 14
ROW_BYTES = {T_F32: (1, 4), T_F16: (1, 2), T_Q4_0: (32, 18), T_Q8_0: (32, 34), T_Q4_K: (256, 144), T_Q6_K: (256, 210)}


def build() -> None:
    subprocess.run(["make", "-s", "-C", _HERE, "oracle"], check=True)


class Model(C.Structure):
    _fields_ = [("n_layer", C.c_int32), ("d_model", C.c_int32), ("n_head", C.c_int32), ("n_ff", C.c_int32),
                ("n_vocab", C.c_int32), ("n_ctx", C.c_int32), ("rms_eps", C.c_float), ("rope_base", C.c_float),
                ("embd_type", C.c_int32), ("output_type", C.c_int32),
                ("token_embd", C.c_void_p), ("output_norm", C.c_void_p), ("output", C.c_void_p),
                ("attn_norm", C.POINTER(C.c_void_p)), ("ffn_norm", C.POINTER(C.c_void_p)),
                ("wq", C.POINTER(C.c_void_p)), ("wk", C.POINTER(C.c_void_p)), ("wv", C.POINTER(C.c_void_p)),
                ("wo", C.POINTER(C.c_void_p)), ("w_up", C.POINTER(C.c_void_p)), ("w_gate", C.POINTER(C.c_void_p)),
                ("w_down", C.POINTER(C.c_void_p)),
                ("t_wq", C.POINTER(C.c_int32)), ("t_wk", C.POINTER(C.c_int32)), ("t_wv", C.POINTER(C.c_int32)),
                ("t_wo", C.POINTER(C.c_int32)), ("t_up", C.POINTER(C.c_int32)), ("t_gate", C.POINTER(C.c_int32)),
                ("t_down", C.POINTER(C.c_int32))]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        l = C.CDLL(LIB_PATH)
        l.oracle_fp16_to_fp32.argtypes = [C.c_uint16]; l.oracle_fp16_to_fp32.restype = C.c_float
        l.oracle_fp32_to_fp16.argtypes = [C.c_float]; l.oracle_fp32_to_fp16.restype = C.c_uint16
        l.oracle_tables.argtypes = [C.c_void_p, C.c_void_p]; l.oracle_tables.restype = None
        l.oracle_quantize_q8_0.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]; l.oracle_quantize_q8_0.restype = None
        l.oracle_quantize_f16.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]; l.oracle_quantize_f16.restype = None
        for name in ("oracle_blockdot_q4_0_q8_0", "oracle_blockdot_q8_0_q8_0"):
            getattr(l, name).argtypes = [C.c_void_p, C.c_void_p]; getattr(l, name).restype = C.c_int32
        for name in ("oracle_dot_q4_0_q8_0", "oracle_dot_q8_0_q8_0", "oracle_dot_f16_f16", "oracle_dot_q4_k_q8_0", "oracle_dot_q6_k_q8_0"):
            getattr(l, name).argtypes = [C.c_void_p, C.c_void_p, C.c_int64]; getattr(l, name).restype = C.c_float
        l.oracle_matmul.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
        l.oracle_rmsnorm.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_void_p]; l.oracle_rmsnorm.restype = None
        l.oracle_mul_rows.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]; l.oracle_mul_rows.restype = None
        l.oracle_add.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]; l.oracle_add.restype = None
        l.oracle_mul.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]; l.oracle_mul.restype = None
        l.oracle_silu.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]; l.oracle_silu.restype = None
        l.oracle_softmax_masked.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_float, C.c_void_p]; l.oracle_softmax_masked.restype = None
        l.oracle_rope.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_float, C.c_void_p]; l.oracle_rope.restype = None
        l.oracle_argmax.argtypes = [C.c_void_p, C.c_int64]; l.oracle_argmax.restype = C.c_int32
        l.oracle_state_new.argtypes = [C.POINTER(Model)]; l.oracle_state_new.restype = C.c_void_p
        l.oracle_state_free.argtypes = [C.c_void_p]; l.oracle_state_free.restype = None
        l.oracle_eval.argtypes = [C.POINTER(Model), C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
        _lib = l
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def quantize_q8_0(x) -> np.ndarray:
    x = f32(x)
    out = np.empty(x.size // 32 * 34, dtype=np.uint8)
    lib().oracle_quantize_q8_0(_p(x), x.size, _p(out))
    return out


def quantize_f16(x) -> np.ndarray:
    x = f32(x)
    out = np.empty(x.size, dtype=np.uint16)
    lib().oracle_quantize_f16(_p(x), x.size, _p(out))
    return out


def blockdots(wtype: int, w_row: np.ndarray, xq: np.ndarray) -> np.ndarray:
    """Per-block int32 dots of one weight row against one Q8_0 activation column."""
    eb, bb = ROW_BYTES[wtype]
    nb = w_row.size // bb
    fn = lib().oracle_blockdot_q4_0_q8_0 if wtype == T_Q4_0 else lib().oracle_blockdot_q8_0_q8_0
    out = np.empty(nb, dtype=np.int32)
    base_w, base_x = w_row.ctypes.data, xq.ctypes.data
    for b in range(nb):
        out[b] = fn(base_w + b * bb, base_x + b * 34)
    return out


def dot(name: str, a: np.ndarray, b: np.ndarray, n: int) -> float:
    return float(getattr(lib(), "oracle_dot_" + name)(_p(a), _p(b), n))


def matmul(wtype: int, w: np.ndarray, k: int, n_out: int, x, want_xq: bool = False):
    """w: raw blocks of n_out rows; x: [t, k] f32 -> [t, n_out] f32 (and the Q8_0 blocks of x)."""
    x = f32(x).reshape(-1, k)
    t = x.shape[0]
    out = np.empty((t, n_out), dtype=np.float32)
    xq = np.empty(t * (k // 32 * 34), dtype=np.uint8) if want_xq else None
    rc = lib().oracle_matmul(wtype, _p(w), k, n_out, _p(x), t, _p(out), _p(xq) if want_xq else None)
    if rc != 0:
        raise RuntimeError(f"oracle_matmul failed: {rc}")
    return (out, xq) if want_xq else out


def rmsnorm(x, eps: float):
    x = f32(x); x2 = x.reshape(-1, x.shape[-1])
    out = np.empty_like(x2)
    lib().oracle_rmsnorm(_p(x2), x2.shape[1], x2.shape[0], eps, _p(out))
    return out.reshape(x.shape)


def mul_rows(x, w):
    x = f32(x); w = f32(w); x2 = x.reshape(-1, x.shape[-1])
    out = np.empty_like(x2)
    lib().oracle_mul_rows(_p(x2), _p(w), x2.shape[1], x2.shape[0], _p(out))
    return out.reshape(x.shape)


def silu(x):
    x = f32(x); out = np.empty_like(x)
    lib().oracle_silu(_p(x), x.size, _p(out))
    return out


def softmax_masked(scores, mask, scale: float):
    s = f32(scores); m = f32(mask); out = np.empty_like(s)
    lib().oracle_softmax_masked(_p(s), _p(m), s.size, scale, _p(out))
    return out


def rope(x, pos, freq_base: float):
    """x: [tokens, heads, hd]."""
    x = f32(x); pos = np.ascontiguousarray(pos, dtype=np.int32); out = np.empty_like(x)
    t, h, hd = x.shape
    lib().oracle_rope(_p(x), _p(pos), hd, h, t, freq_base, _p(out))
    return out


def argmax(x) -> int:
    x = f32(x)
    return int(lib().oracle_argmax(_p(x), x.size))


def tables():
    s = np.empty(65536, dtype=np.float32); e = np.empty(65536, dtype=np.float32)
    lib().oracle_tables(_p(s), _p(e))
    return s, e


class OracleLlama:
    """Whole-model restatement over a GGUF file (read with spy_b200.gguf_io.read_gguf)."""

    def __init__(self, gguf_path: str, n_ctx: int = 512):
        from spy_b200 import gguf_io

        kv, tensors = gguf_io.read_gguf(gguf_path)
        self._keep = []
        L = kv["llama.block_count"]
        m = Model()
        m.n_layer, m.d_model, m.n_head = L, kv["llama.embedding_length"], kv["llama.attention.head_count"]
        m.n_ff, m.n_ctx = kv["llama.feed_forward_length"], n_ctx
        m.n_vocab = len(kv["tokenizer.ggml.tokens"])
        m.rms_eps, m.rope_base = kv["llama.attention.layer_norm_rms_epsilon"], kv.get("llama.rope.freq_base", 10000.0)

        def raw(name):
            ne, number_type, data = tensors[name]
            a = np.ascontiguousarray(data)
            self._keep.append(a)
            return a.ctypes.data, number_type

        m.token_embd, m.embd_type = raw("token_embd.weight")
        m.output_norm, _ = raw("output_norm.weight")
        m.output, m.output_type = raw("output.weight" if "output.weight" in tensors else "token_embd.weight")

        def per_layer(role, want_types):
            ptrs = (C.c_void_p * L)(); types = (C.c_int32 * L)()
            for i in range(L):
                ptrs[i], types[i] = raw(f"blk.{i}.{role}.weight")
            self._keep += [ptrs, types]
            return (ptrs, types) if want_types else ptrs

        m.attn_norm = per_layer("attn_norm", False)
        m.ffn_norm = per_layer("ffn_norm", False)
        m.wq, m.t_wq = per_layer("attn_q", True)
        m.wk, m.t_wk = per_layer("attn_k", True)
        m.wv, m.t_wv = per_layer("attn_v", True)
        m.wo, m.t_wo = per_layer("attn_output", True)
        m.w_up, m.t_up = per_layer("ffn_up", True)
        m.w_gate, m.t_gate = per_layer("ffn_gate", True)
        m.w_down, m.t_down = per_layer("ffn_down", True)
        self.model = m
        self.n_vocab = m.n_vocab
        self.d_model = m.d_model
        self.state = lib().oracle_state_new(C.byref(m))
        self.n_past = 0

    def eval(self, tokens, want_tap: bool = False):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        t = len(tokens)
        logits = np.empty((t, self.n_vocab), dtype=np.float32)
        tap = np.zeros(self.d_model // 32 * 34, dtype=np.uint8) if want_tap else None
        rc = lib().oracle_eval(C.byref(self.model), self.state, _p(tokens), t, self.n_past, _p(logits),
                               _p(tap) if want_tap else None)
        if rc != 0:
            raise RuntimeError(f"oracle_eval failed: {rc}")
        self.n_past += t
        return (logits, tap) if want_tap else logits

    def generate(self, prompt, n_predict: int):
        """Greedy loop as AutoModelGenerator::generate (app/cli/include/cli.h:60-129):
        step 0 = all prompt tokens, later steps one token. Returns (ids, last-token logits per step)."""
        ids = np.zeros(n_predict, dtype=np.int32)
        out = np.zeros((n_predict, self.n_vocab), dtype=np.float32)
        cur = np.asarray(prompt, dtype=np.int32)
        for s in range(n_predict):
            logits = self.eval(cur)
            out[s] = logits[-1]
            ids[s] = argmax(out[s])
            cur = np.array([ids[s]], dtype=np.int32)
        return ids, out

    def close(self):
        if self.state:
            lib().oracle_state_free(self.state)
            self.state = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
