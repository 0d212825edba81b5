"""GPU: the drop-in boundary. The reference's own graph builder, loader, scheduler and greedy sampler (compiled
unmodified into oracle/_ref/libspy_ref_b200.so with the reference's device-backend hook enabled) run their token loop
on `spy::gpu::B200Backend` (spy_b200/adapter/b200_backend.cpp), which forwards every operator node to libspyb200.so
through the C ABI - or, in plan mode, lets the scheduler walk its graph while the steps are served from the library's
fused step plan. Either way the result must equal the golden vectors that the reference's CPU backend produced."""
import os
import sys

import numpy as np
import pytest

from spy_b200 import gguf_io

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
sys.path.insert(0, GOLD)
from make_golden import MODEL_CASES  # noqa: E402


@pytest.mark.parametrize("plan", [False, True])
@pytest.mark.parametrize("name", sorted(MODEL_CASES))
def test_reference_token_loop_on_the_device_backend(name, plan, tmp_models):
    from oracle import spy_ref
    if not spy_ref.b200_available():
        pytest.skip("oracle/_ref/libspy_ref_b200.so not built (reference checkout absent at build time)")
    gold = np.load(os.path.join(GOLD, "models_reference.npz"))
    kw, seed, n_prompt, n_predict, n_ctx = MODEL_CASES[name]
    cfg = gguf_io.LlamaConfig(**kw)
    path = str(tmp_models / f"adapter_{name}.gguf")
    gguf_io.make_llama_gguf(path, cfg, seed=seed)
    ids, logits, _ = spy_ref.generate(path, gold[f"{name}_prompt"], n_predict, n_ctx=n_ctx, n_vocab=cfg.n_vocab, device_backend=True, plan=plan)
    want = gold[f"{name}_logits"]
    print(f"{name}: max |dlogit| = {np.abs(logits - want).max():.3e}")
    assert np.array_equal(ids, gold[f"{name}_ids"])
    assert np.array_equal(logits.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("plan", ["0", "1"])
def test_command_line_driver_gives_the_cpu_backends_tokens(plan, tmp_models):
    """oracle/_ref/spy_b200_cli (spy_b200/adapter/spy_b200_cli.cpp): the reference's token loop from the command line,
    `--backend gpu:b200` against `--backend cpu:default` on the same file and prompt ids."""
    import subprocess
    cli = os.path.join(os.path.dirname(os.path.dirname(__file__)), "oracle", "_ref", "spy_b200_cli")
    if not os.path.exists(cli):
        pytest.skip("oracle/_ref/spy_b200_cli not built (reference checkout absent at build time)")
    cfg = gguf_io.LlamaConfig(n_layer=2, d_model=256, n_head=2, n_ff=512, n_vocab=512, weight_std=0.05)
    path = str(tmp_models / "cli.gguf")
    if not os.path.exists(path):
        gguf_io.make_llama_gguf(path, cfg, seed=3)
    common = [cli, "-m", path, "--token-ids", "5,9,11,300,7", "-n", "8", "-c", "64"]
    cpu = subprocess.run(common + ["--backend", "cpu:default", "-t", "4"], capture_output=True, text=True, timeout=300)
    gpu = subprocess.run(common + ["--backend", "gpu:b200", "--plan", plan], capture_output=True, text=True, timeout=300)
    assert cpu.returncode == 0 and gpu.returncode == 0, (cpu.stderr[-500:], gpu.stderr[-500:])
    ids = lambda out: [l for l in out.splitlines() if l.startswith("token ids:")][0]
    assert ids(gpu.stdout) == ids(cpu.stdout)
    assert "[Performance Timer] decode stage:" in gpu.stdout
