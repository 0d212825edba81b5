"""GGUF v3 files for synthetic LLaMa models: a writer, a reader and the model builder.

The on-disk format is the one the reference parses in
``storage/src/adapter/gguf_adapter.cpp:90-190`` (magic, version u32, n_tensors u64,
n_kv u64, typed KV pairs, tensor infos, data section aligned to
``general.alignment``; every tensor padded to that alignment because the reference
sums aligned sizes to get the data-section length). Tensor names and the metadata
keys a LLaMa graph needs follow ``model/src/llm/model/llama.cpp:7-84`` and
``model/include/llm/model/abstract_model.h:72-101``.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np

from . import quants

GGUF_MAGIC = b"GGUF"
GGUF_VERSION = 3
ALIGNMENT = 32

# value type ids (storage/include/adapter/type.h ModelMetaDataType order == GGUF spec)
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)
_SCALAR_FMT = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i",
               T_F32: "<f", T_BOOL: "<?", T_U64: "<Q", T_I64: "<q", T_F64: "<d"}


def _pack_str(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _pack_value(vtype: int, value) -> bytes:
    if vtype == T_STR:
        return _pack_str(value)
    if vtype == T_ARR:
        etype, items = value
        out = [struct.pack("<IQ", etype, len(items))]
        if etype == T_STR:
            out.extend(_pack_str(s) for s in items)
        else:
            out.append(np.asarray(items, dtype=np.dtype(_SCALAR_FMT[etype][1]).newbyteorder("<")).tobytes())
        return b"".join(out)
    return struct.pack(_SCALAR_FMT[vtype], value)


@dataclass
class TensorEntry:
    name: str
    ne: tuple          # element counts, innermost (ne0) first, as the reference's Shape
    number_type: int
    data: object       # bytes-like (numpy uint8 array / memoryview) of exactly row_bytes(type, prod(ne))


def write_gguf(path: str, kv: list, tensors: list) -> None:
    """kv: [(key, value_type, value)], tensors: [TensorEntry]."""
    with open(path, "wb") as f:
        f.write(GGUF_MAGIC)
        f.write(struct.pack("<IQQ", GGUF_VERSION, len(tensors), len(kv)))
        for key, vtype, value in kv:
            f.write(_pack_str(key))
            f.write(struct.pack("<I", vtype))
            f.write(_pack_value(vtype, value))
        offset = 0
        for t in tensors:
            nbytes = quants.row_bytes(t.number_type, int(np.prod(t.ne)))
            f.write(_pack_str(t.name))
            f.write(struct.pack("<I", len(t.ne)))
            f.write(struct.pack(f"<{len(t.ne)}Q", *t.ne))
            f.write(struct.pack("<IQ", t.number_type, offset))
            offset += -(-nbytes // ALIGNMENT) * ALIGNMENT
        pos = f.tell()
        f.write(b"\0" * (-pos % ALIGNMENT))
        for t in tensors:
            buf = memoryview(t.data).cast("B") if not isinstance(t.data, (bytes, bytearray)) else t.data
            nbytes = quants.row_bytes(t.number_type, int(np.prod(t.ne)))
            if len(buf) != nbytes:
                raise ValueError(f"{t.name}: {len(buf)} bytes given, {nbytes} expected")
            f.write(buf)
            f.write(b"\0" * (-nbytes % ALIGNMENT))


def read_gguf(path: str) -> tuple[dict, dict]:
    """Returns (kv, tensors): kv maps key -> python value; tensors maps
    name -> (ne tuple, number_type, uint8 memmap of the raw blocks)."""
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    pos = 0

    def take(fmt):
        nonlocal pos
        v = struct.unpack_from(fmt, mm, pos)
        pos += struct.calcsize(fmt)
        return v

    def take_str():
        nonlocal pos
        (n,) = take("<Q")
        s = bytes(mm[pos:pos + n]).decode("utf-8")
        pos += n
        return s

    def take_value(vtype):
        if vtype == T_STR:
            return take_str()
        if vtype == T_ARR:
            etype, n = take("<IQ")
            return [take_value(etype) for _ in range(n)]
        return take(_SCALAR_FMT[vtype])[0]

    if bytes(mm[0:4]) != GGUF_MAGIC:
        raise ValueError("not a GGUF file")
    pos = 4
    version, n_tensors, n_kv = take("<IQQ")
    if version != GGUF_VERSION:
        raise ValueError(f"unsupported GGUF version {version}")
    kv = {}
    for _ in range(n_kv):
        key = take_str()
        (vtype,) = take("<I")
        kv[key] = take_value(vtype)
    infos = []
    for _ in range(n_tensors):
        name = take_str()
        (nd,) = take("<I")
        ne = take(f"<{nd}Q")
        number_type, offset = take("<IQ")
        infos.append((name, tuple(ne), number_type, offset))
    align = kv.get("general.alignment", ALIGNMENT)
    base = -(-pos // align) * align
    tensors = {}
    for name, ne, number_type, offset in infos:
        nbytes = quants.row_bytes(number_type, int(np.prod(ne)))
        tensors[name] = (ne, number_type, mm[base + offset: base + offset + nbytes])
    return kv, tensors


# ----------------------------------------------------------------------------------------------
@dataclass
class LlamaConfig:
    """Architecture of a synthetic LLaMa2-style model."""
    n_layer: int = 2
    d_model: int = 256
    n_head: int = 2
    n_ff: int = 512
    n_vocab: int = 320
    n_ctx_train: int = 4096
    rms_eps: float = 1e-5
    rope_base: float = 10000.0
    wtype: int = quants.Q4_0                      # weight type of the matrices
    embd_type: int = quants.FP32                  # the reference can only gather F32 / Q8_0 rows
    overrides: dict = field(default_factory=dict)  # tensor-role -> type, e.g. {"attn_v": Q6_K}
    weight_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_head


LLAMA2_7B = dict(n_layer=32, d_model=4096, n_head=32, n_ff=11008, n_vocab=32000)
LLAMA2_13B = dict(n_layer=40, d_model=5120, n_head=40, n_ff=13824, n_vocab=32000)


def llama_kv(cfg: LlamaConfig, description: str) -> list:
    tokens = [f"<0x{i:02X}>" if i < 256 else f"t{i}" for i in range(cfg.n_vocab)]
    return [
        ("general.architecture", T_STR, "llama"),
        ("general.name", T_STR, "synthetic-llama"),
        ("general.description", T_STR, description),
        ("general.alignment", T_U32, ALIGNMENT),
        ("llama.context_length", T_U32, cfg.n_ctx_train),
        ("llama.embedding_length", T_U32, cfg.d_model),
        ("llama.feed_forward_length", T_U32, cfg.n_ff),
        ("llama.block_count", T_U32, cfg.n_layer),
        ("llama.attention.head_count", T_U32, cfg.n_head),
        ("llama.attention.head_count_kv", T_U32, cfg.n_head),
        ("llama.attention.layer_norm_rms_epsilon", T_F32, cfg.rms_eps),
        ("llama.rope.dimension_count", T_U32, cfg.head_dim),
        ("llama.rope.freq_base", T_F32, cfg.rope_base),
        ("tokenizer.ggml.model", T_STR, "llama"),
        ("tokenizer.ggml.tokens", T_ARR, (T_STR, tokens)),
    ]


def llama_tensor_plan(cfg: LlamaConfig) -> list:
    """[(name, (ne0, ne1) or (ne0,), number_type, kind)] in file order; kind is 'norm' or 'matrix'.
    A matrix [ne0 = input features, ne1 = output rows] stores each output row contiguously."""
    d, f, v = cfg.d_model, cfg.n_ff, cfg.n_vocab

    def wt(role):
        return cfg.overrides.get(role, cfg.wtype)

    plan = [("token_embd.weight", (d, v), cfg.embd_type, "matrix"),
            ("output_norm.weight", (d,), quants.FP32, "norm"),
            ("output.weight", (d, v), wt("output"), "matrix")]
    for i in range(cfg.n_layer):
        p = f"blk.{i}."
        plan += [(p + "attn_norm.weight", (d,), quants.FP32, "norm"),
                 (p + "attn_q.weight", (d, d), wt("attn_q"), "matrix"),
                 (p + "attn_k.weight", (d, d), wt("attn_k"), "matrix"),
                 (p + "attn_v.weight", (d, d), wt("attn_v"), "matrix"),
                 (p + "attn_output.weight", (d, d), wt("attn_output"), "matrix"),
                 (p + "ffn_norm.weight", (d,), quants.FP32, "norm"),
                 (p + "ffn_up.weight", (d, f), wt("ffn_up"), "matrix"),
                 (p + "ffn_gate.weight", (d, f), wt("ffn_gate"), "matrix"),
                 (p + "ffn_down.weight", (f, d), wt("ffn_down"), "matrix")]
    return plan


def make_llama_gguf(path: str, cfg: LlamaConfig, seed: int = 1234, embeddings: np.ndarray | None = None) -> None:
    """Seeded synthetic model on the host: matrices N(0, weight_std) quantized to their type, norms = 1.
    `embeddings` ([n_vocab, d_model] f32) replaces the random token embeddings (embd_type must be FP32)."""
    rng = np.random.default_rng(seed)
    tensors = []
    for name, ne, number_type, kind in llama_tensor_plan(cfg):
        if kind == "norm":
            raw = np.ones(ne[0], dtype=np.float32).view(np.uint8)
        elif name == "token_embd.weight" and embeddings is not None:
            assert number_type == quants.FP32 and embeddings.shape == (ne[1], ne[0])
            raw = np.ascontiguousarray(embeddings, dtype=np.float32).view(np.uint8).reshape(-1)
        else:
            w = rng.standard_normal((ne[1], ne[0]), dtype=np.float32) * np.float32(cfg.weight_std)
            raw = quants.quantize(w, number_type).reshape(-1)
        tensors.append(TensorEntry(name, ne, number_type, raw))
    write_gguf(path, llama_kv(cfg, f"seed={seed}"), tensors)


def make_llama_gguf_cuda(path: str, cfg: LlamaConfig, seed: int = 1234, device: str = "cuda:0") -> None:
    """Same model family generated with torch on a GPU (Q4_0 / Q8_0 / Q4_K / Q6_K / F32 / F16), for
    full-size models where host generation would take minutes. The file is the ground truth
    shared by the GPU arm and the CPU baseline; it is not bit-identical to make_llama_gguf."""
    import torch

    gen = torch.Generator(device=device).manual_seed(seed)

    def q4_0(w):
        b = w.reshape(-1, 32)
        idx = b.abs().argmax(dim=1, keepdim=True)
        d = b.gather(1, idx).squeeze(1) / -8.0
        inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
        q = (b * inv[:, None] + 8.5).to(torch.int32).clamp_(max=15).to(torch.uint8)
        out = torch.empty((b.shape[0], 18), dtype=torch.uint8, device=w.device)
        out[:, 0:2] = d.to(torch.float16).view(torch.uint8).reshape(-1, 2)
        out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
        return out

    def q8_0(w):
        b = w.reshape(-1, 32)
        d = b.abs().amax(dim=1) / 127.0
        inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
        v = b * inv[:, None]
        q = (torch.sign(v) * torch.floor(v.abs() + 0.5)).to(torch.int8)
        out = torch.empty((b.shape[0], 34), dtype=torch.uint8, device=w.device)
        out[:, 0:2] = d.to(torch.float16).view(torch.uint8).reshape(-1, 2)
        out[:, 2:] = q.view(torch.uint8)
        return out

    def pack_scale_min(sc, mn):
        out = torch.zeros((sc.shape[0], 12), dtype=torch.uint8, device=sc.device)
        out[:, 0:4] = (sc[:, :4] & 63) | ((sc[:, 4:] >> 4) << 6)
        out[:, 4:8] = (mn[:, :4] & 63) | ((mn[:, 4:] >> 4) << 6)
        out[:, 8:12] = (sc[:, 4:] & 0xF) | ((mn[:, 4:] & 0xF) << 4)
        return out

    def q4_k(w):   # the plain min/max encoder of quants.quantize_q4_k
        b = w.reshape(-1, 8, 32)
        lo = torch.clamp(b.amin(dim=2), max=0.0)
        hi = torch.clamp(b.amax(dim=2), min=0.0)
        scale, minv = (hi - lo) / 15.0, -lo
        d = (scale.amax(dim=1) / 63.0).to(torch.float16)
        dmin = (minv.amax(dim=1) / 63.0).to(torch.float16)
        d32, dmin32 = d.float()[:, None], dmin.float()[:, None]
        sc = torch.where(d32 > 0, torch.round(scale / d32), torch.zeros_like(scale)).clamp(0, 63).to(torch.uint8)
        mn = torch.where(dmin32 > 0, torch.round(minv / dmin32), torch.zeros_like(minv)).clamp(0, 63).to(torch.uint8)
        eff, off = (d32 * sc.float())[:, :, None], (dmin32 * mn.float())[:, :, None]
        q = torch.where(eff > 0, torch.round((b + off) / eff), torch.zeros_like(b)).clamp(0, 15).to(torch.uint8)
        out = torch.empty((b.shape[0], 144), dtype=torch.uint8, device=w.device)
        out[:, 0:2] = d.view(torch.uint8).reshape(-1, 2)
        out[:, 2:4] = dmin.view(torch.uint8).reshape(-1, 2)
        out[:, 4:16] = pack_scale_min(sc, mn)
        q = q.reshape(-1, 4, 2, 32)
        out[:, 16:] = (q[:, :, 0, :] | (q[:, :, 1, :] << 4)).reshape(-1, 128)
        return out

    def q6_k(w):   # the encoder of quants.quantize_q6_k
        b = w.reshape(-1, 16, 16)
        scale = b.abs().amax(dim=2) / 31.0
        d = (scale.amax(dim=1) / 127.0).to(torch.float16)
        d32 = d.float()[:, None]
        sc = torch.where(d32 > 0, torch.round(scale / d32), torch.zeros_like(scale)).clamp(0, 127).to(torch.int8)
        eff = (d32 * sc.float())[:, :, None]
        q = torch.where(eff > 0, torch.round(b / eff), torch.zeros_like(b)).clamp(-32, 31).to(torch.int16)
        u = (q.reshape(-1, 256) + 32).to(torch.uint8).reshape(-1, 2, 4, 32)
        ql = torch.empty((u.shape[0], 2, 64), dtype=torch.uint8, device=w.device)
        ql[:, :, :32] = (u[:, :, 0, :] & 0xF) | ((u[:, :, 2, :] & 0xF) << 4)
        ql[:, :, 32:] = (u[:, :, 1, :] & 0xF) | ((u[:, :, 3, :] & 0xF) << 4)
        qh = (u[:, :, 0, :] >> 4) | ((u[:, :, 1, :] >> 4) << 2) | ((u[:, :, 2, :] >> 4) << 4) | ((u[:, :, 3, :] >> 4) << 6)
        out = torch.empty((u.shape[0], 210), dtype=torch.uint8, device=w.device)
        out[:, 0:128] = ql.reshape(-1, 128)
        out[:, 128:192] = qh.reshape(-1, 64)
        out[:, 192:208] = sc.view(torch.uint8)
        out[:, 208:210] = d.view(torch.uint8).reshape(-1, 2)
        return out

    enc = {quants.Q4_0: q4_0, quants.Q8_0: q8_0, quants.Q4_K: q4_k, quants.Q6_K: q6_k,
           quants.FP32: lambda w: w.contiguous().view(torch.uint8),
           quants.FP16: lambda w: w.to(torch.float16).contiguous().view(torch.uint8)}
    tensors = []
    for name, ne, number_type, kind in llama_tensor_plan(cfg):
        if kind == "norm":
            raw = np.ones(ne[0], dtype=np.float32).view(np.uint8)
        else:
            w = torch.randn((ne[1], ne[0]), generator=gen, device=device, dtype=torch.float32) * cfg.weight_std
            raw = enc[number_type](w).reshape(-1).cpu().numpy()
            del w
        tensors.append(TensorEntry(name, ne, number_type, raw))
    write_gguf(path, llama_kv(cfg, f"seed={seed} (torch generator on {device})"), tensors)
