"""GPU: the drop-in boundary. The reference's own graph builder, loader, scheduler and greedy sampler (compiled
unmodified into oracle/_ref/libspy_ref_b200.so with the reference's device-backend hook enabled) run their token loop
on `spy::gpu::B200Backend` (spy_b200/adapter/b200_backend.cpp), which forwards every operator node to libspyb200.so
through the C ABI. The result must equal the golden vectors that the reference's CPU backend produced."""
import os
import sys

import numpy as np
import pytest

from spy_b200 import gguf_io

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
sys.path.insert(0, GOLD)
from make_golden import MODEL_CASES  # noqa: E402


@pytest.mark.parametrize("name", sorted(MODEL_CASES))
def test_reference_token_loop_on_the_device_backend(name, tmp_models):
    from oracle import spy_ref
    if not spy_ref.b200_available():
        pytest.skip("oracle/_ref/libspy_ref_b200.so not built (reference checkout absent at build time)")
    gold = np.load(os.path.join(GOLD, "models_reference.npz"))
    kw, seed, n_prompt, n_predict, n_ctx = MODEL_CASES[name]
    cfg = gguf_io.LlamaConfig(**kw)
    path = str(tmp_models / f"adapter_{name}.gguf")
    gguf_io.make_llama_gguf(path, cfg, seed=seed)
    ids, logits, _ = spy_ref.generate(path, gold[f"{name}_prompt"], n_predict, n_ctx=n_ctx, n_vocab=cfg.n_vocab, device_backend=True)
    want = gold[f"{name}_logits"]
    print(f"{name}: max |dlogit| = {np.abs(logits - want).max():.3e}")
    assert np.array_equal(ids, gold[f"{name}_ids"])
    assert np.array_equal(logits.view(np.uint32), want.view(np.uint32))
