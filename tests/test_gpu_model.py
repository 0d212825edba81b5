"""GPU: the whole-model path (GGUF upload, fused step plan, on-device decode) against the golden
vectors generated from the reference's CPU backend and against the CPU oracle.
Gates: identical greedy ids, logits within max-abs 2e-2 and rel 1e-2 (measured far tighter)."""
import os
import sys

import numpy as np
import pytest

from spy_b200 import backend as B
from spy_b200 import gguf_io, quants

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
sys.path.insert(0, GOLD)
from make_golden import MODEL_CASES  # noqa: E402

ABS_TOL, REL_TOL = 2e-2, 1e-2


def logits_ok(got, want):
    """The stated gate is max-abs 2e-2 / rel 1e-2; the kernels reproduce the CPU's f32 summation order, so the
    logits are in fact required to be bit-identical (anything less is amplified by the per-layer Q8_0
    re-quantization to percent-level differences on deep models)."""
    err = np.abs(got - want)
    within = float(err.max()) <= ABS_TOL and float(err.max()) <= REL_TOL * float(np.abs(want).max())
    return within and np.array_equal(np.ascontiguousarray(got).view(np.uint32), np.ascontiguousarray(want).view(np.uint32))


def top2_gap(logits):
    s = np.sort(logits, axis=-1)
    return float((s[..., -1] - s[..., -2]).min())


@pytest.fixture(scope="module")
def be():
    b = B.B200Backend(0)
    yield b
    b.close()


@pytest.mark.parametrize("name", sorted(MODEL_CASES))
def test_generate_matches_reference_golden(be, name, tmp_models):
    gold = np.load(os.path.join(GOLD, "models_reference.npz"))
    kw, seed, n_prompt, n_predict, n_ctx = MODEL_CASES[name]
    path = str(tmp_models / f"{name}.gguf")
    gguf_io.make_llama_gguf(path, gguf_io.LlamaConfig(**kw), seed=seed)
    m = B.LlamaModel(be, path, n_ctx=n_ctx)
    ids, logits = m.generate(gold[f"{name}_prompt"], n_predict)
    want = gold[f"{name}_logits"]
    print(f"{name}: max |dlogit| = {np.abs(logits - want).max():.3e}, min top-2 gap = {top2_gap(want):.3e}")
    assert logits_ok(logits, want)
    assert np.array_equal(ids, gold[f"{name}_ids"])
    m.close()


def test_device_decode_equals_host_loop_and_oracle(be, oracle, tmp_models):
    cfg = gguf_io.LlamaConfig(n_layer=2, d_model=256, n_head=2, n_ff=768, n_vocab=400, weight_std=0.06)
    path = str(tmp_models / "decode.gguf")
    gguf_io.make_llama_gguf(path, cfg, seed=77)
    prompt = np.random.default_rng(5).integers(3, cfg.n_vocab, size=11)
    om = oracle.OracleLlama(path, n_ctx=48)
    want_ids, want_logits = om.generate(prompt, 20)

    m = B.LlamaModel(be, path, n_ctx=48)
    ids_host, logits_host = m.generate(prompt, 20)
    assert np.array_equal(ids_host, want_ids) and logits_ok(logits_host, want_logits)

    # prefill through eval, then the device-resident loop (CUDA graph replay + device argmax)
    m2 = B.LlamaModel(be, path, n_ctx=48)
    first = m2.eval(prompt, 0)
    tok0 = int(np.argmax(first))
    ids_dev, logits_dev = m2.decode(tok0, len(prompt), 19, want_logits=True)
    assert tok0 == want_ids[0] and np.array_equal(ids_dev, want_ids[1:])
    # same kernels either way: bitwise the same logits as the host-driven loop
    assert np.array_equal(logits_dev.view(np.uint32), logits_host[1:].view(np.uint32))
    # and again without returning logits (pure replay)
    m3 = B.LlamaModel(be, path, n_ctx=48)
    m3.eval(prompt, 0)
    ids_fast, _ = m3.decode(tok0, len(prompt), 19)
    assert np.array_equal(ids_fast, want_ids[1:])
    assert m3.last_launches in (19 * 2, 19 * (5 * cfg.n_layer + 2)) and m3.last_ms > 0   # persistent step kernel + argmax, or one kernel per matrix
    for x in (m, m2, m3):
        x.close()


@pytest.mark.parametrize("pdl,graph", [(False, False), (True, False), (False, True)])
def test_launch_modes_agree(pdl, graph, oracle, tmp_models):
    cfg = gguf_io.LlamaConfig(weight_std=0.05)
    path = str(tmp_models / "modes.gguf")
    if not os.path.exists(path):
        gguf_io.make_llama_gguf(path, cfg, seed=11)
    prompt = np.arange(3, 12)
    want_ids, _ = oracle.OracleLlama(path, n_ctx=32).generate(prompt, 10)
    b = B.B200Backend(0, use_pdl=pdl, use_graph=graph)
    m = B.LlamaModel(b, path, n_ctx=32)
    tok0 = int(np.argmax(m.eval(prompt, 0)))
    ids, _ = m.decode(tok0, len(prompt), 9)
    assert tok0 == want_ids[0] and np.array_equal(ids, want_ids[1:])
    m.close(); b.close()


def test_activation_blocks_of_first_layer(be, oracle, tmp_models):
    """Q8_0 blocks of layer 0's attention-norm output for the first prompt token: RMSNorm (in the CPU's
    summation order), the norm weight and the quantizer together must give the CPU's bytes."""
    cfg = gguf_io.LlamaConfig(weight_std=0.05)
    path = str(tmp_models / "tap.gguf")
    gguf_io.make_llama_gguf(path, cfg, seed=21)
    prompt = np.arange(5, 13)
    om = oracle.OracleLlama(path, n_ctx=32)
    _, want = om.eval(prompt, want_tap=True)
    m = B.LlamaModel(be, path, n_ctx=32)
    m.eval(prompt, 0)
    got = m.tap_xq()
    assert np.array_equal(got, want)   # byte-identical Q8_0 activation blocks
    m.close()


def test_prompt_longer_than_one_pass_and_context_edge(be, oracle, tmp_models):
    """21 prompt tokens (three passes of <= 8 columns), decoding until the context is exactly full."""
    cfg = gguf_io.LlamaConfig(weight_std=0.05)
    path = str(tmp_models / "long.gguf")
    gguf_io.make_llama_gguf(path, cfg, seed=31)
    prompt = np.random.default_rng(1).integers(3, cfg.n_vocab, size=21)
    n_ctx = 32
    want_ids, want_logits = oracle.OracleLlama(path, n_ctx=n_ctx).generate(prompt, n_ctx - 21 + 1)
    m = B.LlamaModel(be, path, n_ctx=n_ctx)
    ids, logits = m.generate(prompt, n_ctx - 21 + 1)
    assert np.array_equal(ids, want_ids) and logits_ok(logits, want_logits)
    with pytest.raises(B.SpybError):
        m.eval(np.array([1], dtype=np.int32), n_ctx)       # one past the context
    with pytest.raises(B.SpybError):
        m.eval(np.array([cfg.n_vocab], dtype=np.int32), 0)  # token id out of range
    m.close()


@pytest.mark.parametrize("wtype", [quants.Q4_0, quants.Q8_0])
@pytest.mark.parametrize("env", [{}, {"SPYB_PREFILL_CHUNK": "32"}, {"SPYB_PREFILL": "0"}])
def test_prompt_on_the_tensor_cores(env, wtype, oracle, tmp_models, monkeypatch):
    """An 83-token prompt: as one GEMM chunk (default), as chunks of 32 + 32 + 19 tokens, and as mat-vec passes
    (SPYB_PREFILL=0): the same bits as the CPU restatement each time, for the prompt's logits and for the tokens
    decoded afterwards from the KV cache the prompt left behind."""
    cfg = gguf_io.LlamaConfig(n_layer=3, d_model=384, n_head=3, n_ff=640, n_vocab=500, wtype=wtype, weight_std=0.05)
    path = str(tmp_models / f"tc_prompt_{wtype}.gguf")
    if not os.path.exists(path):
        gguf_io.make_llama_gguf(path, cfg, seed=53)
    prompt = np.random.default_rng(8).integers(3, cfg.n_vocab, size=83)
    want_ids, want_logits = oracle.OracleLlama(path, n_ctx=96).generate(prompt, 8)
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    b = B.B200Backend(0)
    m = B.LlamaModel(b, path, n_ctx=96)
    ids, logits = m.generate(prompt, 8)
    assert np.array_equal(ids, want_ids) and logits_ok(logits, want_logits)
    # a second prompt appended behind the first one's context (n_past > 0), again through the GEMM path
    m2 = B.LlamaModel(b, path, n_ctx=96)
    m2.eval(prompt[:40], 0)
    again = m2.eval(prompt[40:], 40)
    assert np.array_equal(again.view(np.uint32), want_logits[0].view(np.uint32))
    m.close(); m2.close(); b.close()


def test_prompt_widths_the_gemm_tile_does_not_divide(be, oracle, tmp_models):
    """n_ff = 416 is no multiple of the 128-row GEMM tile (the stacked up|gate matrix has 832 rows: the last tile is half
    padding, and W_gate starts in the middle of a tile): the padded rows are neither computed into anything nor stored."""
    cfg = gguf_io.LlamaConfig(n_layer=2, d_model=256, n_head=2, n_ff=416, n_vocab=300, weight_std=0.05)
    path = str(tmp_models / "odd_ff.gguf")
    gguf_io.make_llama_gguf(path, cfg, seed=59)
    prompt = np.random.default_rng(9).integers(3, cfg.n_vocab, size=20)
    want_ids, want_logits = oracle.OracleLlama(path, n_ctx=32).generate(prompt, 4)
    m = B.LlamaModel(be, path, n_ctx=32)
    ids, logits = m.generate(prompt, 4)
    assert np.array_equal(ids, want_ids) and logits_ok(logits, want_logits)
    m.close()


@pytest.mark.parametrize("n_seq,n_ctx,kq", [(3, 64, False), (8, 64, False), (6, 1100, False), (20, 64, False), (17, 1100, False),
                                            (3, 64, True), (6, 64, True), (18, 64, True)])
def test_batch_of_sequences_equals_single_sequence_runs(n_seq, n_ctx, kq, oracle, tmp_models):
    """Independent sequences that share the weights and advance in lockstep: every sequence must give the ids and the
    logits of a run on its own (the batch > 1 configurations are replicas of the single-sequence reference). Prompts of
    one length, different contents; 3 sequences = one group of activation columns, 8 and 6 = two groups; 16 and more go
    through the tensor-core GEMM kernels as the tokens of one pass; a context above 1024 positions takes the three-kernel
    attention. kq: the Q4_K_M-style mix (groups of four columns through the K-quant mat-vec kernel, or the K-quant GEMM)."""
    cfg = gguf_io.LlamaConfig(n_layer=2, d_model=256, n_head=2, n_ff=512, n_vocab=400, weight_std=0.06,
                              **(dict(wtype=quants.Q4_K, overrides={"attn_v": quants.Q6_K, "ffn_down": quants.Q6_K, "output": quants.Q6_K}) if kq else {}))
    path = str(tmp_models / ("batch_kq.gguf" if kq else "batch.gguf"))
    if not os.path.exists(path):
        gguf_io.make_llama_gguf(path, cfg, seed=61)
    rng = np.random.default_rng(n_seq)
    n_prompt, n_steps = 19, 9
    prompts = [rng.integers(3, cfg.n_vocab, size=n_prompt) for _ in range(n_seq)]
    want = [oracle.OracleLlama(path, n_ctx=n_ctx).generate(p, n_steps + 1) for p in prompts]
    b = B.B200Backend(0)
    m = B.LlamaModel(b, path, n_ctx=n_ctx)
    m.set_sequences(n_seq)
    first = []
    for c, p in enumerate(prompts):
        m.select_sequence(c)
        lg = m.eval(p, 0)
        assert np.array_equal(lg.view(np.uint32), want[c][1][0].view(np.uint32))
        first.append(int(np.argmax(lg)))
    ids, logits = m.decode_batch(first, n_prompt, n_steps, want_logits=True)
    for c in range(n_seq):
        assert first[c] == want[c][0][0] and np.array_equal(ids[:, c], want[c][0][1:]), c
        assert np.array_equal(np.ascontiguousarray(logits[:, c]).view(np.uint32), want[c][1][1:].view(np.uint32)), c
    # a single sequence continues from the batch's caches with the single-sequence entry point
    m.select_sequence(n_seq - 1)
    nxt = m.eval(np.array([ids[-1, n_seq - 1]], dtype=np.int32), n_prompt + n_steps)
    assert np.isfinite(nxt).all()
    m.close(); b.close()


def test_long_context_attention(be, oracle, tmp_models):
    """A 600-token prompt in a 1024-token context: many 32-wide accumulator steps and ragged tails in both
    attention products."""
    cfg = gguf_io.LlamaConfig(n_layer=1, weight_std=0.05)
    path = str(tmp_models / "split.gguf")
    gguf_io.make_llama_gguf(path, cfg, seed=41)
    prompt = np.random.default_rng(2).integers(3, cfg.n_vocab, size=600)
    om = oracle.OracleLlama(path, n_ctx=1024)
    want_ids, want_logits = om.generate(prompt, 3)
    m = B.LlamaModel(be, path, n_ctx=1024)
    ids, logits = m.generate(prompt, 3)
    assert logits_ok(logits, want_logits)
    assert np.array_equal(ids, want_ids)
    m.close()


@pytest.mark.parametrize("name,cfg", [
    ("q4k", dict(wtype=quants.Q4_K)),
    ("q4k_m", dict(wtype=quants.Q4_K, overrides={"attn_v": quants.Q6_K, "ffn_down": quants.Q6_K, "output": quants.Q6_K})),
    ("q6k_long_rows", dict(wtype=quants.Q6_K, n_ff=4608, overrides={"ffn_gate": quants.Q4_K, "ffn_down": quants.Q4_K})),   # 18 super-blocks per W_down row
    ("q4k_embd", dict(wtype=quants.Q4_K, embd_type=quants.Q4_K, overrides={"output": quants.Q6_K})),   # token embeddings as K-quant rows, as stock files keep them
    ("q6k_embd", dict(wtype=quants.Q4_K, embd_type=quants.Q6_K)),
])
def test_k_quant_models_match_the_restatement(name, cfg, oracle, tmp_models):
    """Q4_K / Q6_K weights through the step plan (the Q4_K_M-style mix: Q6_K for attn_v, ffn_down and the output head).
    The reference has block layouts but no arithmetic for these types, so parity is unpinned: the checker is the CPU
    restatement (activations quantized to Q8_0, integer sub-block sums, one f32 chain per super-block), whose order the
    kernel follows - the gate is the stated tolerance and identical ids, and the bits are expected to agree as well."""
    c = gguf_io.LlamaConfig(**dict(dict(n_layer=2, d_model=256, n_head=2, n_ff=512, n_vocab=512, weight_std=0.05), **cfg))
    path = str(tmp_models / f"{name}.gguf")
    gguf_io.make_llama_gguf(path, c, seed=51)
    prompt = np.random.default_rng(13).integers(3, c.n_vocab, size=7)
    want_ids, want_logits = oracle.OracleLlama(path, n_ctx=32).generate(prompt, 6)
    b = B.B200Backend(0)
    m = B.LlamaModel(b, path, n_ctx=32)
    ids, logits = m.generate(prompt, 6)
    assert np.array_equal(ids, want_ids) and logits_ok(logits, want_logits)
    assert np.array_equal(np.asarray(logits, dtype=np.float32).view(np.uint32), np.asarray(want_logits, dtype=np.float32).view(np.uint32))
    ids_dev, _ = m.decode(int(ids[0]), len(prompt), 5)          # and the device-side decode loop (graph replay)
    assert np.array_equal(ids_dev, want_ids[1:])
    m.close()
    # a prompt long enough for the tensor-core GEMM kernels (two tiles of 64 tokens, the second ragged), then decode
    long_prompt = np.random.default_rng(14).integers(3, c.n_vocab, size=75)
    want_ids2, want_logits2 = oracle.OracleLlama(path, n_ctx=96).generate(long_prompt, 4)
    m2 = B.LlamaModel(b, path, n_ctx=96)
    ids2, logits2 = m2.generate(long_prompt, 4)
    assert np.array_equal(ids2, want_ids2)
    assert np.array_equal(np.asarray(logits2, dtype=np.float32).view(np.uint32), np.asarray(want_logits2, dtype=np.float32).view(np.uint32))
    m2.close(); b.close()


def test_unsupported_models_are_reported(be, tmp_models):
    path = str(tmp_models / "mixed.gguf")      # K-quants beside Q4_0 matrices: no kernel mixes the two activation layouts
    gguf_io.make_llama_gguf(path, gguf_io.LlamaConfig(wtype=quants.Q4_K, overrides={"attn_q": quants.Q4_0}), seed=1)
    with pytest.raises(B.SpybError) as e:
        B.LlamaModel(be, path, n_ctx=32)
    assert e.value.status == B.UNSUPPORTED
    with pytest.raises(B.SpybError):
        B.LlamaModel(be, str(tmp_models / "missing.gguf"), n_ctx=32)
    bad = str(tmp_models / "trunc.gguf")
    with open(path, "rb") as f, open(bad, "wb") as g:
        g.write(f.read(300))
    with pytest.raises(B.SpybError):
        B.LlamaModel(be, bad, n_ctx=32)


def _tiles(t):
    return {f"SPYB_TILE_{n}": str(t) for n in ("QKV", "WO", "UPGATE", "DOWN", "HEAD")}


@pytest.mark.parametrize("env", [{}, _tiles(8), _tiles(16), _tiles(32), {"SPYB_TILE_QKV": "4", "SPYB_TILE_DOWN": "4", "SPYB_TILE_UPGATE": "32"},
                                 {"SPYB_NO_ROWS_KERNEL": "1"}, {"SPYB_MV_S": "1", "SPYB_MV_WACT": "2"},
                                 dict(_tiles(8), SPYB_MV_S="1", SPYB_MV_WACT="3"),
                                 dict(_tiles(16), SPYB_MV_S="1", SPYB_MV_WACT="3"),
                                 {"SPYB_MMA": "1"}, dict(_tiles(8), SPYB_MMA="1"), dict(_tiles(16), SPYB_MMA="1"),
                                 dict(_tiles(8), SPYB_MMA="1", SPYB_MV_S="1", SPYB_MV_WACT="3"),
                                 {"SPYB_STEP": "1"}, dict(_tiles(16), SPYB_STEP="1"), dict(_tiles(8), SPYB_STEP="1"),
                                 {"SPYB_STEP": "1", "SPYB_STEP_STAGES": "16"}, dict(_tiles(16), SPYB_STEP="1", SPYB_STEP_STAGES="17", SPYB_STEP_CTAS="37"),
                                 {"SPYB_STEP": "1", "SPYB_STEP_COOP": "0"}])
@pytest.mark.parametrize("wtype", [quants.Q4_0, quants.Q8_0])
def test_every_matvec_variant_matches_oracle(env, wtype, oracle, tmp_models, monkeypatch):
    """The weight layouts (4-, 8-, 16- and 32-row tiles, fused up|gate), the lane-per-row kernels with one, two or four
    lanes per row (the default), the lane-per-accumulator kernel, the tensor-core kernels on 8- and 16-row tiles
    (SPYB_MMA=1), stage sizes and stream counts are tuning choices: every combination must give the CPU's bits. So must
    single-token steps as one persistent kernel (SPYB_STEP=1), whatever its ring depth and grid size. The vocabulary is large enough for the head to take the lane-per-row path."""
    cfg = gguf_io.LlamaConfig(n_layer=2, d_model=256, n_head=2, n_ff=512, n_vocab=8192, weight_std=0.05, wtype=wtype)
    path = str(tmp_models / f"variants_{wtype}.gguf")
    if not os.path.exists(path):
        gguf_io.make_llama_gguf(path, cfg, seed=41)
    prompt = np.random.default_rng(9).integers(3, cfg.n_vocab, size=10)
    want_ids, want_logits = oracle.OracleLlama(path, n_ctx=32).generate(prompt, 6)
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    b = B.B200Backend(0)
    m = B.LlamaModel(b, path, n_ctx=32)
    ids, logits = m.generate(prompt, 6)
    assert np.array_equal(ids, want_ids) and logits_ok(logits, want_logits)
    m.close(); b.close()


def test_step_kernel_wait_runs_out_and_is_reported(oracle, tmp_models, monkeypatch):
    """The failure path of the bounded waits, without a fault: a step whose first grid barrier expects one arrival more
    than there are CTAs gives up after the limit (2 ms), records code 2 and returns; the model works afterwards."""
    cfg = gguf_io.LlamaConfig(n_layer=2, d_model=256, n_head=2, n_ff=512, n_vocab=512, weight_std=0.05)
    path = str(tmp_models / "timeout.gguf")
    gguf_io.make_llama_gguf(path, cfg, seed=43)
    prompt = np.random.default_rng(10).integers(3, cfg.n_vocab, size=5)
    want_ids, want_logits = oracle.OracleLlama(path, n_ctx=32).generate(prompt, 4)
    monkeypatch.setenv("SPYB_STEP", "1")
    b = B.B200Backend(0)
    m = B.LlamaModel(b, path, n_ctx=32)
    assert m.selftest_wait_timeout(2_000_000) == 2
    ids, logits = m.generate(prompt, 4)
    assert np.array_equal(ids, want_ids) and logits_ok(logits, want_logits)
    m.close(); b.close()


@pytest.mark.parametrize("env", [{}, {"SPYB_STEP": "1"}])
def test_long_context_attention_path_in_the_model(env, oracle, tmp_models, monkeypatch):
    """A context above 1024 positions switches attention to the three-kernel path (scores / softmax / PV spread over the
    chip); prompt passes of several tokens and single-token steps through it must give the CPU's bits."""
    cfg = gguf_io.LlamaConfig(n_layer=2, d_model=256, n_head=2, n_ff=512, n_vocab=512, weight_std=0.05)
    path = str(tmp_models / "longctx.gguf")
    if not os.path.exists(path):
        gguf_io.make_llama_gguf(path, cfg, seed=47)
    prompt = np.random.default_rng(12).integers(3, cfg.n_vocab, size=70)
    want_ids, want_logits = oracle.OracleLlama(path, n_ctx=2048).generate(prompt, 6)
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    b = B.B200Backend(0)
    m = B.LlamaModel(b, path, n_ctx=2048)
    ids, logits = m.generate(prompt, 6)
    assert np.array_equal(ids, want_ids) and logits_ok(logits, want_logits)
    m.close(); b.close()


def test_rmsnorm_running_sum_on_hard_inputs(oracle, tmp_models):
    """The RMSNorm sum of squares is a serial f32 running sum on the CPU (groups of four squares added to one
    accumulator in order); the GPU forms the groups in parallel and runs the same chain on one thread. Inputs that
    stress the order of the additions - exact ties (ones, powers of two, small dyadic numbers), huge outliers, leading
    zeros, underflowing squares, all zeros - must give the CPU's bits. d_model = 4096 exercises the full 1024-group sum."""
    d, v = 4096, 16
    rng = np.random.default_rng(77)
    E = rng.standard_normal((v, d)).astype(np.float32)
    E[0] = 1.0                                                                  # every group sum is 4: all ties
    E[1] = np.float32(2.0) ** rng.integers(-3, 4, d) * rng.choice([-1.0, 1.0], d)
    E[2, rng.integers(0, d, 3)] *= 1000.0                                       # massive outliers
    E[3] = 0.0; E[3, rng.integers(0, d, 9)] = rng.standard_normal(9)            # mostly zeros
    E[4] *= 1e-20                                                               # squares underflow to denormals / zero
    E[5, :2000] = 0.0                                                           # leading zeros
    E[6] = rng.integers(-8, 9, d) / 8.0                                         # small dyadic numbers: many ties
    E[7] = 0.0                                                                  # sum == 0
    E[8] *= 1e4; E[9] *= 1e-4
    E[10, 0] = 3e4                                                              # the first element dominates
    cfg = gguf_io.LlamaConfig(n_layer=1, d_model=d, n_head=32, n_ff=256, n_vocab=v, weight_std=0.02)
    path = str(tmp_models / "hard_norm.gguf")
    gguf_io.make_llama_gguf(path, cfg, seed=5, embeddings=E)
    orc = oracle.OracleLlama(path, n_ctx=8)
    b = B.B200Backend(0)
    m = B.LlamaModel(b, path, n_ctx=8)
    bad = []
    for tok in range(v):
        orc.n_past = 0                                   # every token starts a fresh sequence (the cache is overwritten)
        want_ids, want_logits = orc.generate(np.array([tok]), 2)
        ids, logits = m.generate(np.array([tok]), 2)
        same = np.array_equal(np.asarray(logits, dtype=np.float32).view(np.uint32), np.asarray(want_logits, dtype=np.float32).view(np.uint32))
        if not (np.array_equal(ids, want_ids) and same):
            bad.append((tok, float(np.nanmax(np.abs(np.asarray(logits) - np.asarray(want_logits))))))
    m.close(); b.close()
    assert not bad, f"tokens whose logits differ from the CPU's (token, max abs difference): {bad}"
