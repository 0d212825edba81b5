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


# ---- wide-range stress: the two ways of fusing a*a + b*b (and similar choices the compiler makes) agree on
# most inputs and differ on a few per cent of them, so every reduction is compared on many inputs whose
# magnitudes span several orders
def _wide(rng, n):
    return (rng.standard_normal(n) * rng.choice([1e-3, 0.3, 1.0, 5.0, 40.0], size=n)).astype(np.float32)


@pytest.mark.parametrize("n", [4, 64, 100, 4096, 11008])
def test_rmsnorm_wide_range(ref, oracle, n):
    rng = np.random.default_rng(n)
    for _ in range(40):
        x = _wide(rng, n) * np.float32(rng.choice([0.05, 1.0, 20.0]))
        out = np.empty_like(x)
        p = ref.OpParam(); p.eps = 1e-5
        ref.run_op("NormRMS", [ref.make_tensor(x, 0, (n, 1))], out, p)
        assert np.array_equal(bits(out), bits(oracle.rmsnorm(x, 1e-5)))


@pytest.mark.parametrize("n_kv", [1, 3, 4, 37, 129, 512])
def test_softmax_wide_range(ref, oracle, n_kv):
    rng = np.random.default_rng(n_kv)
    n_ctx = 512
    scale = float(np.float32(1.0) / np.sqrt(np.float32(128.0)))
    for _ in range(25):
        sc = (_wide(rng, n_kv) * 8).reshape(1, 1, n_kv)
        mask = np.full((1, n_ctx), -np.inf, dtype=np.float32); mask[0, :n_kv] = 0
        out = np.empty_like(sc)
        p = ref.OpParam(); p.scale = scale
        ref.run_op("Softmax", [ref.make_tensor(sc, 0, (n_kv, 1, 1)), ref.make_tensor(mask, 26, (n_ctx, 1))], out, p)
        assert np.array_equal(bits(out[0, 0]), bits(oracle.softmax_masked(sc[0, 0], mask[0, :n_kv], scale)))


def test_rope_silu_f16dot_wide_range(ref, oracle):
    rng = np.random.default_rng(3)
    for _ in range(20):
        x = _wide(rng, 2 * 3 * 128).reshape(2, 3, 128)
        pos = rng.integers(0, 4096, size=2).astype(np.int32)
        out = np.empty_like(x)
        p = ref.OpParam()
        p.rope_mode, p.num_dim, p.num_context, p.num_origin_context = 0, 128, 4096, 4096
        p.freq_base, p.freq_scale, p.extend_factor, p.attention_factor, p.beta_fast, p.beta_slow = 10000.0, 1.0, 0.0, 1.0, 32.0, 1.0
        ref.run_op("Rope", [ref.make_tensor(x, 0, (128, 3, 2)), ref.make_tensor(pos, 26, (2,))], out, p)
        assert np.array_equal(bits(out), bits(oracle.rope(x, pos, 10000.0)))
        g = _wide(rng, 4096)
        out = np.empty_like(g)
        ref.run_op("Silu", [ref.make_tensor(g, 0, (4096,))], out)
        assert np.array_equal(bits(out), bits(oracle.silu(g)))
        for n in (1, 31, 32, 33, 64, 128, 500):
            a = oracle.quantize_f16(_wide(rng, n)); b = oracle.quantize_f16(_wide(rng, n))
            assert np.float32(ref.dot(2, a, b, n)).tobytes() == np.float32(oracle.dot("f16_f16", a, b, n)).tobytes()


@pytest.mark.parametrize("qt", [quants.Q4_0, quants.Q8_0])
def test_matmul_wide_range(ref, oracle, qt):
    rng = np.random.default_rng(qt)
    k, n = 1024, 64
    for _ in range(10):
        w = quants.quantize((_wide(rng, n * k) * 0.05).reshape(n, k), qt)
        x = _wide(rng, 3 * k).reshape(3, k)
        out = np.empty((3, n), dtype=np.float32)
        ref.run_op("MatMul", [ref.make_tensor(w, qt, (k, n)), ref.make_tensor(x, 0, (k, 3))], out)
        assert np.array_equal(bits(out), bits(oracle.matmul(qt, w, k, n, x)))


def test_deep_model_with_growing_activations(ref, oracle, tmp_models):
    """Eight layers with large weights: the residual stream grows by orders of magnitude with depth."""
    cfg = gguf_io.LlamaConfig(n_layer=8, d_model=256, n_head=2, n_ff=512, n_vocab=400, weight_std=0.15)
    path = str(tmp_models / "deep.gguf")
    gguf_io.make_llama_gguf(path, cfg, seed=123)
    prompt = np.random.default_rng(9).integers(3, cfg.n_vocab, size=40)
    ids, logits, _ = ref.generate(path, prompt, 6, n_ctx=64, threads=4, n_vocab=cfg.n_vocab)
    ids2, logits2 = oracle.OracleLlama(path, n_ctx=64).generate(prompt, 6)
    assert np.array_equal(ids, ids2) and np.array_equal(bits(logits), bits(logits2))
