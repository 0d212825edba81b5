"""Host-side mirror of the reference's backend interface over the C ABI of libspyb200.so.

``B200Backend`` offers what ``spy::Backend`` declares
(backend/interface/include/backend/backend.h:31-95): ``alloc_memory``, ``dealloc_memory``,
``is_support``, ``submit``; ``LlamaModel`` is the whole-model path (GGUF load, eval, on-device
greedy decode). Everything here is plumbing around the library: there is no Python or CPU
implementation of any operator, and importing this module without the built library, or creating a
backend without a CUDA device, raises.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libspyb200.so")

SUCCESS, FAIL, UNSUPPORTED = 0, 1, 2
FP32, FP16, Q4_0, Q8_0, Q4_K, Q6_K, INT32 = 0, 1, 2, 8, 12, 14, 26
OP = dict(Input=0, Nop=1, Dup=2, Copy=3, View=4, Reshape=5, GetRow=8, Transpose=9, Permute=10, Contiguous=11, Silu=13,
          Softmax=17, Add=18, Mul=20, MatMul=23, NormRMS=26, Rope=27)
NODE_CONSTANT, NODE_IO, NODE_CACHE, NODE_DYNAMIC = 0, 1, 2, 6
_BLOCK = {FP32: (1, 4), FP16: (1, 2), INT32: (1, 4), Q4_0: (32, 18), Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210)}


class SpybError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"spyb status {status} ({'Unsupport' if status == UNSUPPORTED else 'Fail'}): {message}")
        self.status = status


class Config(C.Structure):
    _fields_ = [("device_id", C.c_int32), ("tp_size", C.c_int32), ("tp_rank", C.c_int32), ("use_pdl", C.c_int32),
                ("use_graph", C.c_int32), ("reserved", C.c_int32), ("arena_bytes", C.c_uint64)]


class Tensor(C.Structure):
    _fields_ = [("number_type", C.c_int32), ("dim", C.c_uint32), ("elements", C.c_int64 * 4), ("bytes", C.c_int64 * 4),
                ("data", C.c_void_p), ("node_type", C.c_int32), ("reserved", C.c_int32)]


class RopeParam(C.Structure):
    _fields_ = [("mode", C.c_int32), ("num_past", C.c_int32), ("num_dim", C.c_int32), ("num_context", C.c_int32),
                ("num_origin_context", C.c_int32), ("freq_base", C.c_float), ("freq_scale", C.c_float),
                ("extend_factor", C.c_float), ("attention_factor", C.c_float), ("beta_fast", C.c_float),
                ("beta_slow", C.c_float), ("xpos_base", C.c_float), ("xpos_down", C.c_int32)]


class OpDesc(C.Structure):
    _fields_ = [("op_type", C.c_int32), ("num_input", C.c_int32), ("input", Tensor * 3), ("output", Tensor),
                ("softmax_scale", C.c_float), ("norm_eps", C.c_float), ("view_offset", C.c_int64), ("rope", RopeParam)]


class ModelInfo(C.Structure):
    _fields_ = [("n_layer", C.c_int32), ("d_model", C.c_int32), ("n_head", C.c_int32), ("n_ff", C.c_int32),
                ("n_vocab", C.c_int32), ("n_ctx", C.c_int32), ("head_dim", C.c_int32), ("tp_size", C.c_int32),
                ("tp_rank", C.c_int32), ("rms_eps", C.c_float), ("rope_base", C.c_float), ("weight_bytes", C.c_uint64),
                ("kv_bytes_per_token", C.c_uint64)]


CALLBACK = C.CFUNCTYPE(None, C.c_void_p)

_lib = None


def lib():
    """Loads libspyb200.so; raises if it has not been built (there is nothing to fall back to)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `make -C spy_b200/csrc` (or __graft_entry__.build())")
    l = C.CDLL(LIB_PATH)
    vp, i32, i64, u64 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64
    sig = {
        "spyb_create": (i32, [C.POINTER(Config), C.POINTER(vp)]),
        "spyb_destroy": (None, [vp]),
        "spyb_last_error": (C.c_char_p, [vp]),
        "spyb_max_memory": (u64, [vp]),
        "spyb_avail_memory": (u64, [vp]),
        "spyb_alloc": (vp, [vp, u64]),
        "spyb_free": (None, [vp, vp, u64]),
        "spyb_is_support": (i32, [i32]),
        "spyb_upload_constant": (vp, [vp, C.c_char_p, vp, u64, i32, C.POINTER(i64)]),
        "spyb_submit": (i32, [vp, C.POINTER(OpDesc), vp, vp]),
        "spyb_submit_timed": (i32, [vp, C.POINTER(OpDesc), i32, i32, C.POINTER(C.c_float)]),
        "spyb_sync": (i32, [vp]),
        "spyb_memcpy_h2d": (i32, [vp, vp, vp, u64]),
        "spyb_memcpy_d2h": (i32, [vp, vp, vp, u64]),
        "spyb_quantize_q8_0": (i32, [vp, vp, i64, vp]),
        "spyb_block_dots": (i32, [vp, i32, vp, vp, i64, vp]),
        "spyb_read_tables": (i32, [vp, vp, vp]),
        "spyb_attention": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32]),
        "spyb_model_read_activation": (i32, [vp, i32, vp, u64]),
        "spyb_model_bench_kernel": (C.c_float, [vp, i32, i32, C.POINTER(u64)]),
        "spyb_model_load_gguf": (i32, [vp, C.c_char_p, i32, C.POINTER(vp)]),
        "spyb_model_free": (None, [vp]),
        "spyb_model_info_get": (i32, [vp, C.POINTER(ModelInfo)]),
        "spyb_nccl_unique_id": (i32, [vp]),
        "spyb_model_init_tp": (i32, [vp, vp]),
        "spyb_model_eval": (i32, [vp, vp, i32, i32, vp]),
        "spyb_model_decode": (i32, [vp, i32, i32, i32, vp, vp]),
        "spyb_model_set_sequences": (i32, [vp, i32]),
        "spyb_model_select_sequence": (i32, [vp, i32]),
        "spyb_model_decode_batch": (i32, [vp, vp, i32, i32, i32, vp, vp]),
        "spyb_model_last_ms": (C.c_float, [vp]),
        "spyb_model_last_launches": (i64, [vp]),
        "spyb_model_tap_xq": (i32, [vp, vp]),
        "spyb_matmul_noalloc": (i32, [vp, i32, vp, i64, i64, vp, i64, vp]),
        "spyb_prefill_matmul": (i32, [vp, i32, vp, i64, i64, vp, i64, vp, C.c_float, vp]),
        "spyb_prefill_selftest_wait_timeout": (i32, [vp, u64, C.POINTER(i32)]),
        "spyb_model_tp_export": (i32, [vp, vp]),
        "spyb_model_tp_import": (i32, [vp, vp]),
        "spyb_model_read_timeline": (i32, [vp, vp, i32]),
        "spyb_model_read_step_timeline": (i32, [vp, vp, i32]),
        "spyb_set_wait_limit_ns": (i32, [vp, u64]),
        "spyb_selftest_host": (i32, []),
        "spyb_tp_layer_shard": (i32, [i32, i32, i32, i32, i32, C.POINTER(i64)]),
        "spyb_model_selftest_wait_timeout": (i32, [vp, u64, C.POINTER(i32)]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(l, name)
        fn.restype, fn.argtypes = res, args
    _lib = l
    return l


def exported_symbols() -> list:
    """Entry points declared in include/spyb.h, parsed from the header (used by the CPU load test)."""
    import re

    header = os.path.join(os.path.dirname(_PKG), "include", "spyb.h")
    text = open(header).read()
    return sorted(set(re.findall(r"\b(spyb_[a-z0-9_]+)\s*\(", text)))


def _np_ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def contiguous_strides(number_type: int, ne) -> list:
    """Shape's default byte strides (orchestration/include/number/tensor.h:41-58)."""
    be, bb = _BLOCK[number_type]
    nb = [bb, ne[0] // be * bb, 0, 0]
    nb[2] = nb[1] * ne[1]
    nb[3] = nb[2] * ne[2]
    return nb


def make_tensor(data_ptr, number_type: int, ne, nb=None, node_type: int = NODE_DYNAMIC) -> Tensor:
    ne = list(ne) + [1] * (4 - len(ne))
    t = Tensor()
    t.number_type, t.dim, t.node_type = number_type, 4, node_type
    nb = list(nb) + [0] * (4 - len(nb)) if nb is not None else contiguous_strides(number_type, ne)
    for i in range(4):
        t.elements[i], t.bytes[i] = ne[i], nb[i]
    t.data = data_ptr
    return t


class B200Backend:
    """One GPU behind the reference's Backend contract."""

    def __init__(self, device_id: int = 0, tp_size: int = 1, tp_rank: int = 0, use_pdl: bool = True,
                 use_graph: bool = True, arena_bytes: int = 0):
        self._l = lib()
        cfg = Config(device_id, tp_size, tp_rank, int(use_pdl), int(use_graph), 0, arena_bytes)
        h = C.c_void_p()
        st = self._l.spyb_create(C.byref(cfg), C.byref(h))
        if st != SUCCESS or not h.value:
            raise SpybError(st, "spyb_create failed: no usable CUDA device (this backend has no CPU path)")
        self.h = h
        self.config = cfg
        self._callbacks = []

    def close(self):
        if getattr(self, "h", None) and self.h.value:
            self._l.spyb_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st: int):
        if st != SUCCESS:
            raise SpybError(st, self._l.spyb_last_error(self.h).decode())

    # --- Backend::alloc_memory / dealloc_memory / capacity / is_support
    def alloc_memory(self, size: int) -> int:
        p = self._l.spyb_alloc(self.h, size)
        if not p:
            raise SpybError(FAIL, self._l.spyb_last_error(self.h).decode())
        return p

    def dealloc_memory(self, ptr: int, size: int) -> None:
        self._l.spyb_free(self.h, ptr, size)

    def get_max_memory_capacity(self) -> int:
        return self._l.spyb_max_memory(self.h)

    def get_avail_memory_capacity(self) -> int:
        return self._l.spyb_avail_memory(self.h)

    def is_support(self, op: str | int) -> bool:
        return bool(self._l.spyb_is_support(OP[op] if isinstance(op, str) else op))

    # --- data movement for tests and IO tensors
    def upload(self, a: np.ndarray) -> int:
        a = np.ascontiguousarray(a)
        p = self.alloc_memory(max(1, a.nbytes))
        if a.nbytes:
            self._check(self._l.spyb_memcpy_h2d(self.h, p, _np_ptr(a), a.nbytes))
        return p

    def download(self, ptr: int, shape, dtype) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        if out.nbytes:
            self._check(self._l.spyb_memcpy_d2h(self.h, _np_ptr(out), ptr, out.nbytes))
        return out

    def upload_constant(self, name: str, raw: np.ndarray, number_type: int, ne) -> int:
        raw = np.ascontiguousarray(raw)
        ne4 = (C.c_int64 * 4)(*(list(ne) + [1] * (4 - len(ne))))
        p = self._l.spyb_upload_constant(self.h, name.encode(), _np_ptr(raw), raw.nbytes, number_type, ne4)
        if not p:
            raise SpybError(FAIL, self._l.spyb_last_error(self.h).decode())
        return p

    # --- Backend::submit
    def submit(self, desc: OpDesc, callback=None) -> None:
        cb = None
        if callback is not None:
            cb = CALLBACK(lambda _user: callback())
            self._callbacks.append(cb)   # keep alive until it has fired
        self._check(self._l.spyb_submit(self.h, C.byref(desc), cb, None))

    def submit_timed(self, descs, repeats: int) -> float:
        """Device time in ms of `repeats` submits that walk round-robin over the descriptors (measurement aid)."""
        arr = (OpDesc * len(descs))(*descs)
        ms = C.c_float(0.0)
        self._check(self._l.spyb_submit_timed(self.h, arr, len(descs), int(repeats), C.byref(ms)))
        return float(ms.value)

    def set_wait_limit_ns(self, ns: int) -> None:
        self._check(self._l.spyb_set_wait_limit_ns(self.h, int(ns)))

    def sync(self) -> None:
        self._check(self._l.spyb_sync(self.h))
        self._callbacks.clear()

    # --- parity probes
    def quantize_q8_0(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        n = x.size
        if n == 0:
            return np.zeros(0, dtype=np.uint8)
        px = self.upload(x)
        nbytes = n // 32 * 34
        po = self.alloc_memory(max(1, nbytes))
        try:
            self._check(self._l.spyb_quantize_q8_0(self.h, px, n, po))
            return self.download(po, (nbytes,), np.uint8)
        finally:
            self.dealloc_memory(px, x.nbytes)
            self.dealloc_memory(po, max(1, nbytes))

    def block_dots(self, weight_type: int, w_row: np.ndarray, x_blocks: np.ndarray, n: int) -> np.ndarray:
        pw, px = self.upload(w_row), self.upload(x_blocks)
        po = self.alloc_memory(max(4, n // 32 * 4))
        try:
            self._check(self._l.spyb_block_dots(self.h, weight_type, pw, px, n, po))
            return self.download(po, (n // 32,), np.int32)
        finally:
            self.dealloc_memory(pw, w_row.nbytes)
            self.dealloc_memory(px, x_blocks.nbytes)
            self.dealloc_memory(po, max(4, n // 32 * 4))


    def read_tables(self):
        silu = np.empty(65536, dtype=np.float32); ex = np.empty(65536, dtype=np.float32)
        self._check(self._l.spyb_read_tables(self.h, _np_ptr(silu), _np_ptr(ex)))
        return silu, ex

    def matmul_noalloc(self, weight_type: int, w_dev: int, n_rows: int, k: int, x_dev: int, n_cols: int, out_dev: int) -> None:
        """MatMul of raw-layout quantized rows (device pointers throughout) that allocates nothing; enqueues only (use sync())."""
        self._check(self._l.spyb_matmul_noalloc(self.h, weight_type, w_dev, n_rows, k, x_dev, n_cols, out_dev))

    def prefill_matmul(self, weight_type: int, w_rows: np.ndarray, n_rows: int, k: int, x: np.ndarray, norm_w=None, eps: float = 0.0) -> np.ndarray:
        """MatMul of raw-layout quantized rows (host bytes) with the columns x [T, k] on the tensor-core prompt kernel; returns f32 [T, n_rows]."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        w_rows = np.ascontiguousarray(w_rows)
        t = x.shape[0]
        out = np.empty((t, n_rows), dtype=np.float32)
        nw = None if norm_w is None else np.ascontiguousarray(norm_w, dtype=np.float32)
        self._check(self._l.spyb_prefill_matmul(self.h, weight_type, _np_ptr(w_rows), n_rows, k, _np_ptr(x), t, None if nw is None else _np_ptr(nw),
                                                C.c_float(eps), _np_ptr(out)))
        return out

    def prefill_selftest_wait_timeout(self, limit_ns: int) -> int:
        """Runs the prompt kernel with one batch withheld; returns the code of the wait that gave up (4, 5 or 6)."""
        code = C.c_int32(0)
        self._check(self._l.spyb_prefill_selftest_wait_timeout(self.h, limit_ns, C.byref(code)))
        return int(code.value)

    def attention(self, q16: np.ndarray, k_cache16: np.ndarray, v_cache_t16: np.ndarray, pos0: int, n_head: int, head_dim: int, n_ctx: int,
                  n_total: int = 0) -> np.ndarray:
        """q16: uint16 [T, n_head*head_dim] fp16 bits; k_cache16: [n_ctx, d]; v_cache_t16: [d, n_ctx]. Returns f32 [T, d]."""
        t = q16.shape[0]
        d = n_head * head_dim
        pq, pk, pv = self.upload(q16), self.upload(k_cache16), self.upload(v_cache_t16)
        po = self.alloc_memory(t * d * 4)
        try:
            self._check(self._l.spyb_attention(self.h, pq, pk, pv, po, pos0, t, n_total, n_head, head_dim, n_ctx))
            return self.download(po, (t, d), np.float32)
        finally:
            self.dealloc_memory(pq, q16.nbytes); self.dealloc_memory(pk, k_cache16.nbytes); self.dealloc_memory(pv, v_cache_t16.nbytes)
            self.dealloc_memory(po, t * d * 4)


class LlamaModel:
    """GGUF model resident on one GPU (or one tensor-parallel shard of it)."""

    def __init__(self, backend: B200Backend, gguf_path: str, n_ctx: int = 512):
        self.backend = backend
        self._l = backend._l
        h = C.c_void_p()
        backend._check(self._l.spyb_model_load_gguf(backend.h, gguf_path.encode(), n_ctx, C.byref(h)))
        self.h = h
        info = ModelInfo()
        backend._check(self._l.spyb_model_info_get(self.h, C.byref(info)))
        self.info = info

    def close(self):
        if getattr(self, "h", None) and self.h.value:
            self._l.spyb_model_free(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def init_tp(self, unique_id: bytes) -> None:
        buf = C.create_string_buffer(unique_id, 128)
        self.backend._check(self._l.spyb_model_init_tp(self.h, buf))

    def eval(self, tokens, n_past: int, want_logits: bool = True):
        """One execute() of the graph for these tokens; returns the last token's logits (host)."""
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = np.empty(self.info.n_vocab, dtype=np.float32) if want_logits else None
        self.backend._check(self._l.spyb_model_eval(self.h, _np_ptr(tokens), len(tokens), n_past,
                                                    _np_ptr(logits) if want_logits else None))
        return logits

    def decode(self, first_token: int, n_past: int, n_steps: int, want_logits: bool = False):
        """n_steps greedy single-token steps kept on the device; returns (ids, logits or None)."""
        ids = np.zeros(n_steps, dtype=np.int32)
        logits = np.empty((n_steps, self.info.n_vocab), dtype=np.float32) if want_logits else None
        self.backend._check(self._l.spyb_model_decode(self.h, int(first_token), n_past, n_steps, _np_ptr(ids),
                                                      _np_ptr(logits) if want_logits else None))
        return ids, logits

    def set_sequences(self, n_seq: int) -> None:
        """n_seq independent KV caches (sequences that share the weights); select_sequence picks the one eval / decode act on."""
        self.backend._check(self._l.spyb_model_set_sequences(self.h, n_seq))

    def select_sequence(self, seq: int) -> None:
        self.backend._check(self._l.spyb_model_select_sequence(self.h, seq))

    def decode_batch(self, first_tokens, n_past: int, n_steps: int, want_logits: bool = False):
        """Greedy decoding of len(first_tokens) sequences in lockstep from the common position n_past; returns
        (ids [n_steps, n_seq], logits [n_steps, n_seq, n_vocab] or None)."""
        first = np.ascontiguousarray(first_tokens, dtype=np.int32)
        n_seq = len(first)
        ids = np.zeros((n_steps, n_seq), dtype=np.int32)
        logits = np.empty((n_steps, n_seq, self.info.n_vocab), dtype=np.float32) if want_logits else None
        self.backend._check(self._l.spyb_model_decode_batch(self.h, _np_ptr(first), n_seq, n_past, n_steps, _np_ptr(ids),
                                                            _np_ptr(logits) if want_logits else None))
        return ids, logits

    def generate(self, prompt, n_predict: int, want_logits: bool = True):
        """The loop of AutoModelGenerator::generate (app/cli/include/cli.h:88-128) through eval():
        host token ids in, host logits out, argmax on the host. Returns (ids, logits[n_predict, n_vocab])."""
        ids = np.zeros(n_predict, dtype=np.int32)
        out = np.zeros((n_predict, self.info.n_vocab), dtype=np.float32)
        cur = np.asarray(prompt, dtype=np.int32)
        n_past = 0
        for s in range(n_predict):
            out[s] = self.eval(cur, n_past)
            n_past += len(cur)
            ids[s] = int(np.argmax(out[s]))   # first maximum, as std::max_element
            cur = np.array([ids[s]], dtype=np.int32)
        return ids, (out if want_logits else None)

    @property
    def last_ms(self) -> float:
        return float(self._l.spyb_model_last_ms(self.h))

    @property
    def last_launches(self) -> int:
        return int(self._l.spyb_model_last_launches(self.h))

    def tp_export(self) -> bytes:
        """64-byte IPC handle of this rank's exchange buffer (fused tensor-parallel exchange)."""
        buf = C.create_string_buffer(64)
        self.backend._check(self._l.spyb_model_tp_export(self.h, buf))
        return buf.raw

    def tp_import(self, handles) -> None:
        """handles: the tp_export() results of all ranks, in rank order."""
        blob = b"".join(handles)
        self.backend._check(self._l.spyb_model_tp_import(self.h, C.c_char_p(blob)))

    def timeline(self) -> np.ndarray:
        """[n_kernels, 8] device-clock stamps (ns) of the last step; empty unless loaded with SPYB_TIMELINE=1."""
        n = 5 * self.info.n_layer + 1
        out = np.zeros((n, 8), dtype=np.uint64)
        got = self._l.spyb_model_read_timeline(self.h, _np_ptr(out), n)
        return out[:got]

    def step_timeline(self) -> np.ndarray:
        """[n_checkpoints, 2] device-clock stamps (ns) of the last single-token step on the persistent kernel: CTA 0's
        time and the latest CTA's time at every check point; empty unless loaded with SPYB_TIMELINE=1."""
        n = 16 * self.info.n_layer + 8
        out = np.zeros((n, 2), dtype=np.uint64)
        got = self._l.spyb_model_read_step_timeline(self.h, _np_ptr(out), n)
        return out[:got]

    def selftest_wait_timeout(self, limit_ns: int) -> int:
        """Runs a step whose first grid barrier cannot complete, bounded by limit_ns; returns the recorded error code."""
        code = C.c_int32(-1)
        self.backend._check(self._l.spyb_model_selftest_wait_timeout(self.h, int(limit_ns), C.byref(code)))
        return int(code.value)

    def tap_xq(self) -> np.ndarray:
        out = np.empty(self.info.d_model // 32 * 34, dtype=np.uint8)
        self.backend._check(self._l.spyb_model_tap_xq(self.h, _np_ptr(out)))
        return out


def nccl_unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    if lib().spyb_nccl_unique_id(buf) != SUCCESS:
        raise SpybError(FAIL, "ncclGetUniqueId failed (libnccl.so.2 not loadable?)")
    return buf.raw
