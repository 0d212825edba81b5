"""CPU: the plain-C oracle against the golden vectors generated from the reference's own code
(tests/golden/make_golden.py). Bit-exact everywhere: these fixtures are what pins the oracle."""
import os
import sys

import numpy as np
import pytest

from spy_b200 import gguf_io, quants

GOLD = os.path.join(os.path.dirname(__file__), "golden")
sys.path.insert(0, GOLD)
from make_golden import MODEL_CASES  # noqa: E402


@pytest.fixture(scope="module")
def ops():
    return np.load(os.path.join(GOLD, "ops_reference.npz"))


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_q8_0_quantizer_bytes(oracle, ops):
    assert np.array_equal(oracle.quantize_q8_0(ops["q8_x"]), ops["q8_blocks"])


def test_f16_rounding(oracle, ops):
    assert np.array_equal(oracle.quantize_f16(ops["q8_x"]), ops["f16_bits"])


@pytest.mark.parametrize("name,qt", [("q4_0", quants.Q4_0), ("q8_0", quants.Q8_0)])
def test_matmul_bits(oracle, ops, name, qt):
    x, w = ops["mm_x"], ops[f"mm_w_{name}"]
    t, k = x.shape
    n = w.shape[0]
    got = oracle.matmul(qt, w, k, n, x)
    assert np.array_equal(bits(got), bits(ops[f"mm_out_{name}"]))


@pytest.mark.parametrize("n", [32, 128, 129, 333])
def test_f16_dot(oracle, ops, n):
    got = np.float32(oracle.dot("f16_f16", ops[f"f16dot_a_{n}"], ops[f"f16dot_b_{n}"], n))
    assert got.tobytes() == np.float32(ops[f"f16dot_r_{n}"]).tobytes()


def test_rmsnorm(oracle, ops):
    assert np.array_equal(bits(oracle.rmsnorm(ops["norm_x"], 1e-5)), bits(ops["norm_out"]))


def test_softmax(oracle, ops):
    sc, mask = ops["sm_scores"], ops["sm_mask"]
    for h in range(sc.shape[0]):
        got = oracle.softmax_masked(sc[h, 0], mask[0, : sc.shape[2]], float(ops["sm_scale"]))
        assert np.array_equal(bits(got), bits(ops["sm_out"][h, 0]))


def test_rope(oracle, ops):
    assert np.array_equal(bits(oracle.rope(ops["rope_x"], ops["rope_pos"], 10000.0)), bits(ops["rope_out"]))


def test_silu_and_tables(oracle, ops):
    assert np.array_equal(bits(oracle.silu(ops["silu_x"])), bits(ops["silu_out"]))
    silu_t, exp_t = oracle.tables()
    keys = ops["tbl_keys"]
    assert np.array_equal(bits(silu_t[keys]), bits(ops["tbl_silu"]))
    assert np.array_equal(bits(exp_t[keys]), bits(ops["tbl_exp"]))


@pytest.mark.parametrize("name", sorted(MODEL_CASES))
def test_model_logits_and_ids(oracle, name, tmp_models):
    gold = np.load(os.path.join(GOLD, "models_reference.npz"))
    kw, seed, n_prompt, n_predict, n_ctx = MODEL_CASES[name]
    path = str(tmp_models / f"{name}.gguf")
    gguf_io.make_llama_gguf(path, gguf_io.LlamaConfig(**kw), seed=seed)
    m = oracle.OracleLlama(path, n_ctx=n_ctx)
    ids, logits = m.generate(gold[f"{name}_prompt"], n_predict)
    assert np.array_equal(ids, gold[f"{name}_ids"])
    assert np.array_equal(bits(logits), bits(gold[f"{name}_logits"]))
