"""Generates the golden fixtures in this folder by running the reference's own CPU code
(oracle/_ref/libspy_ref.so, built by oracle/Makefile from the reference checkout).

Run from the repo root where the reference is present:  python tests/golden/make_golden.py
The fixtures are small .npz files; inputs are seeded so they can be regenerated exactly.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import spy_ref  # noqa: E402
from spy_b200 import gguf_io, quants  # noqa: E402


def rope_param(hd, n_ctx):
    p = spy_ref.OpParam()
    p.rope_mode, p.num_dim, p.num_context, p.num_origin_context = 0, hd, n_ctx, 4096
    p.freq_base, p.freq_scale, p.extend_factor, p.attention_factor, p.beta_fast, p.beta_slow = 10000.0, 1.0, 0.0, 1.0, 32.0, 1.0
    return p


def ops_fixture():
    rng = np.random.default_rng(20240601)
    out = {}
    # Q8_0 activation quantizer: mixed magnitudes, an all-zero block, exact .5 ties
    x = (rng.standard_normal(32 * 64) * rng.choice([1e-3, 1.0, 50.0], size=32 * 64)).astype(np.float32)
    x[:32] = 0.0
    x[32:64] = np.arange(32, dtype=np.float32) - 15.5
    x[32 + 31] = 127.0
    out["q8_x"] = x
    out["q8_blocks"] = spy_ref.quantize_q8_0(x)
    out["f16_bits"] = spy_ref.quantize_f16(x)
    # block dots and MatMul
    K, N, T = 1024, 48, 4
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    xs = rng.standard_normal((T, K)).astype(np.float32)
    out["mm_x"] = xs
    for name, qt in (("q4_0", quants.Q4_0), ("q8_0", quants.Q8_0)):
        wq = quants.quantize(w, qt)
        res = np.empty((T, N), dtype=np.float32)
        spy_ref.run_op("MatMul", [spy_ref.make_tensor(wq, qt, (K, N)), spy_ref.make_tensor(xs, 0, (K, T))], res)
        out[f"mm_w_{name}"] = wq
        out[f"mm_out_{name}"] = res
    # F16 dot at the lengths attention uses (head_dim and ragged n_kv)
    for n in (32, 128, 129, 333):
        a = spy_ref.quantize_f16(rng.standard_normal(n).astype(np.float32))
        b = spy_ref.quantize_f16(rng.standard_normal(n).astype(np.float32))
        out[f"f16dot_a_{n}"], out[f"f16dot_b_{n}"] = a, b
        out[f"f16dot_r_{n}"] = np.float32(spy_ref.dot(spy_ref.DOT_F16_F16, a, b, n))
    # RMSNorm
    xn = rng.standard_normal((3, 4096)).astype(np.float32)
    res = np.empty_like(xn)
    p = spy_ref.OpParam(); p.eps = 1e-5
    spy_ref.run_op("NormRMS", [spy_ref.make_tensor(xn, 0, (4096, 3))], res, p)
    out["norm_x"], out["norm_out"] = xn, res
    # masked softmax [n_kv, T=1, H=2], mask row of n_ctx
    n_ctx, n_kv = 64, 37
    sc = (rng.standard_normal((2, 1, n_kv)) * 3).astype(np.float32)
    mask = np.full((1, n_ctx), -np.inf, dtype=np.float32); mask[0, :n_kv] = 0
    res = np.empty_like(sc)
    p = spy_ref.OpParam(); p.scale = float(np.float32(1.0) / np.sqrt(np.float32(128.0)))
    spy_ref.run_op("Softmax", [spy_ref.make_tensor(sc, 0, (n_kv, 1, 2)), spy_ref.make_tensor(mask, 26, (n_ctx, 1))], res, p)
    out["sm_scores"], out["sm_mask"], out["sm_out"], out["sm_scale"] = sc, mask, res, np.float32(p.scale)
    # RoPE [hd=128, heads=4, tokens=3]
    xr = rng.standard_normal((3, 4, 128)).astype(np.float32)
    pos = np.array([0, 17, 511], dtype=np.int32)
    res = np.empty_like(xr)
    spy_ref.run_op("Rope", [spy_ref.make_tensor(xr, 0, (128, 4, 3)), spy_ref.make_tensor(pos, 26, (3,))], res, rope_param(128, 512))
    out["rope_x"], out["rope_pos"], out["rope_out"] = xr, pos, res
    # SiLU
    g = (rng.standard_normal(2048) * 4).astype(np.float32)
    res = np.empty_like(g)
    spy_ref.run_op("Silu", [spy_ref.make_tensor(g, 0, (2048,))], res)
    out["silu_x"], out["silu_out"] = g, res
    # the two 65 536-entry tables, stored as samples (every 97th key) plus a checksum
    _, silu_t, exp_t = spy_ref.tables()
    out["tbl_keys"] = np.arange(0, 65536, 97, dtype=np.int32)
    out["tbl_silu"], out["tbl_exp"] = silu_t[::97].copy(), exp_t[::97].copy()
    np.savez_compressed(os.path.join(HERE, "ops_reference.npz"), **out)


MODEL_CASES = {
    # name: (config kwargs, seed, n_prompt, n_predict, n_ctx)
    "tiny_q4_0": (dict(wtype=quants.Q4_0, embd_type=quants.FP32, weight_std=0.05), 1234, 8, 12, 64),
    "tiny_q8_0": (dict(wtype=quants.Q8_0, embd_type=quants.Q8_0, weight_std=0.05), 1235, 8, 12, 64),
    "small_q4_0": (dict(n_layer=3, d_model=512, n_head=4, n_ff=1024, n_vocab=640, wtype=quants.Q4_0, weight_std=0.04), 1236, 5, 10, 32),
}


def model_fixture():
    out = {}
    for name, (kw, seed, n_prompt, n_predict, n_ctx) in MODEL_CASES.items():
        cfg = gguf_io.LlamaConfig(**kw)
        path = f"/tmp/golden_{name}.gguf"
        gguf_io.make_llama_gguf(path, cfg, seed=seed)
        prompt = np.random.default_rng(4321).integers(3, cfg.n_vocab, size=n_prompt).astype(np.int32)
        ids, logits, _ = spy_ref.generate(path, prompt, n_predict, n_ctx=n_ctx, threads=4, n_vocab=cfg.n_vocab)
        out[f"{name}_prompt"], out[f"{name}_ids"], out[f"{name}_logits"] = prompt, ids, logits
        os.remove(path)
    np.savez_compressed(os.path.join(HERE, "models_reference.npz"), **out)


if __name__ == "__main__":
    ops_fixture()
    model_fixture()
    print("golden fixtures written to", HERE)
