"""CPU, only where the reference was compiled (oracle/_ref): the plain-C oracle against the
reference's own code on fresh seeded inputs and edge cases. Skipped where _ref is absent."""
import numpy as np
import pytest

from spy_b200 import gguf_io, quants


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_q8_quantizer_random(ref, oracle, seed):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(32 * 512) * rng.choice([1e-6, 1e-2, 1.0, 1e3], size=32 * 512)).astype(np.float32)
    assert np.array_equal(ref.quantize_q8_0(x), oracle.quantize_q8_0(x))


def test_q8_quantizer_edges(ref, oracle):
    x = np.zeros(32 * 4, dtype=np.float32)
    x[32:64] = np.linspace(-1, 1, 32)            # symmetric
    x[64:96] = np.float32(65504.0)               # fp16 max magnitude scale
    x[96:128] = np.arange(32) * 0.5              # ties at .5 after scaling
    assert np.array_equal(ref.quantize_q8_0(x), oracle.quantize_q8_0(x))


@pytest.mark.parametrize("kind,name,qt", [(0, "q4_0_q8_0", quants.Q4_0), (1, "q8_0_q8_0", quants.Q8_0)])
@pytest.mark.parametrize("k", [32, 4096, 11008])
def test_block_dot_rows(ref, oracle, kind, name, qt, k):
    rng = np.random.default_rng(k)
    w = quants.quantize((rng.standard_normal((4, k)) * 0.02).astype(np.float32), qt)
    xq = oracle.quantize_q8_0(rng.standard_normal(k).astype(np.float32))
    for r in range(4):
        a = np.float32(ref.dot(kind, w[r], xq, k)); b = np.float32(oracle.dot(name, w[r], xq, k))
        assert a.tobytes() == b.tobytes()


def test_model_prefill_then_decode(ref, oracle, tmp_models):
    cfg = gguf_io.LlamaConfig(n_layer=2, d_model=256, n_head=2, n_ff=768, n_vocab=400, weight_std=0.06)
    path = str(tmp_models / "vs_ref.gguf")
    gguf_io.make_llama_gguf(path, cfg, seed=77)
    prompt = np.random.default_rng(5).integers(3, cfg.n_vocab, size=11)
    ids, logits, _ = ref.generate(path, prompt, 9, n_ctx=32, threads=3, n_vocab=cfg.n_vocab)
    m = oracle.OracleLlama(path, n_ctx=32)
    ids2, logits2 = m.generate(prompt, 9)
    assert np.array_equal(ids, ids2)
    assert np.array_equal(bits(logits), bits(logits2))


def test_reference_is_thread_count_invariant(ref, tmp_models):
    cfg = gguf_io.LlamaConfig(weight_std=0.05)
    path = str(tmp_models / "threads.gguf")
    gguf_io.make_llama_gguf(path, cfg, seed=3)
    prompt = np.arange(3, 9)
    base = ref.generate(path, prompt, 4, n_ctx=32, threads=1, n_vocab=cfg.n_vocab)[1]
    for t in (2, 5):
        assert np.array_equal(bits(base), bits(ref.generate(path, prompt, 4, n_ctx=32, threads=t, n_vocab=cfg.n_vocab)[1]))
