"""CPU: block layouts and the GGUF writer/reader."""
import numpy as np
import pytest

from spy_b200 import gguf_io, quants


@pytest.mark.parametrize("qt,tol", [(quants.Q4_0, 0.13), (quants.Q8_0, 0.005), (quants.Q4_K, 0.15), (quants.Q6_K, 0.03)])
def test_quantize_roundtrip_error(qt, tol):
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((8, 1024)) * 0.02).astype(np.float32)
    raw = quants.quantize(x, qt)
    assert raw.shape == (8, quants.row_bytes(qt, 1024))
    y = quants.dequantize(raw, qt)
    assert np.abs(y - x).max() <= tol * np.abs(x).max()


@pytest.mark.parametrize("name,qt", [("Q4_0", quants.Q4_0), ("Q8_0", quants.Q8_0), ("Q4_K", quants.Q4_K), ("Q6_K", quants.Q6_K)])
def test_layout_matches_gguf_package(name, qt):
    gguf = pytest.importorskip("gguf")
    rng = np.random.default_rng(2)
    x = (rng.standard_normal((4, 512)) * 0.02).astype(np.float32)
    raw = quants.quantize(x, qt)
    gt = getattr(gguf.GGMLQuantizationType, name)
    assert np.array_equal(gguf.quants.dequantize(raw, gt), quants.dequantize(raw, qt))
    if qt in (quants.Q4_0, quants.Q8_0):
        assert np.array_equal(gguf.quants.quantize(x, gt).reshape(-1), raw.reshape(-1))


def test_zero_block_and_empty():
    z = np.zeros((1, 256), dtype=np.float32)
    for qt in (quants.Q4_0, quants.Q8_0, quants.Q4_K, quants.Q6_K):
        assert np.all(quants.dequantize(quants.quantize(z, qt), qt) == 0)
    assert quants.quantize(np.zeros((0, 32), dtype=np.float32), quants.Q4_0).size == 0
    with pytest.raises(ValueError):
        quants.quantize(np.zeros((1, 33), dtype=np.float32), quants.Q4_0)


def test_gguf_roundtrip(tmp_path):
    cfg = gguf_io.LlamaConfig(overrides={"attn_v": quants.Q6_K, "ffn_down": quants.Q6_K}, wtype=quants.Q4_K)
    path = str(tmp_path / "m.gguf")
    gguf_io.make_llama_gguf(path, cfg, seed=9)
    kv, tensors = gguf_io.read_gguf(path)
    assert kv["general.architecture"] == "llama" and kv["llama.block_count"] == cfg.n_layer
    assert len(kv["tokenizer.ggml.tokens"]) == cfg.n_vocab
    plan = gguf_io.llama_tensor_plan(cfg)
    assert set(tensors) == {p[0] for p in plan}
    ne, qt, data = tensors["blk.1.attn_v.weight"]
    assert qt == quants.Q6_K and ne == (cfg.d_model, cfg.d_model) and data.size == quants.row_bytes(qt, cfg.d_model ** 2)
    assert np.all(tensors["output_norm.weight"][2].view(np.float32) == 1.0)
    for name, (ne, qt, data) in tensors.items():
        assert (data.ctypes.data - tensors["token_embd.weight"][2].ctypes.data) % gguf_io.ALIGNMENT == 0
    gguf = pytest.importorskip("gguf")
    r = gguf.GGUFReader(path)
    assert len(r.tensors) == len(plan)
