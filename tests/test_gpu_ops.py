"""GPU: every kernel of the per-operator path through the C ABI against the CPU oracle.
Integer and byte results must be identical; f32 results differ only by summation order."""
import ctypes as C
import os

import numpy as np
import pytest

from spy_b200 import backend as B
from spy_b200 import quants

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def be():
    b = B.B200Backend(0)
    yield b
    b.close()


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def close(got, want, rel=0.0):
    """f32 results are required to be bit-identical: every kernel follows the CPU's summation order."""
    return np.array_equal(bits(got), bits(want))


def run(be, op, inputs, out_ne, out_type=B.FP32, host_out=False, **params):
    """inputs: list of (np array, number_type, ne, nb or None, node_type). Returns the f32/u16 output array."""
    d = B.OpDesc()
    d.op_type, d.num_input = B.OP[op], len(inputs)
    dev = []
    for i, (a, nt, ne, nb, node) in enumerate(inputs):
        if node == B.NODE_IO:
            a = np.ascontiguousarray(a)
            ptr = a.ctypes.data
            dev.append((None, a))
        else:
            ptr = be.upload(a)
            dev.append((ptr, a))
        d.input[i] = B.make_tensor(ptr, nt, ne, nb, node)
    esz = 4 if out_type in (B.FP32, B.INT32) else 2
    n_out = int(np.prod(out_ne))
    host_buf = np.zeros(n_out, dtype=np.float32 if esz == 4 else np.uint16)
    if op == "Copy":
        d.output = B.make_tensor(None, out_type, out_ne)
    elif host_out:
        d.output = B.make_tensor(host_buf.ctypes.data, out_type, out_ne, None, B.NODE_IO)
    else:
        po = be.alloc_memory(max(1, n_out * esz))
        d.output = B.make_tensor(po, out_type, out_ne)
    d.softmax_scale = params.get("scale", 0.0)
    d.norm_eps = params.get("eps", 0.0)
    d.view_offset = params.get("offset", 0)
    if op == "Rope":
        r = d.rope
        r.mode, r.num_dim, r.num_context, r.num_origin_context = 0, params["n_dim"], 512, 4096
        r.freq_base, r.freq_scale, r.extend_factor, r.attention_factor, r.beta_fast, r.beta_slow = 10000.0, 1.0, 0.0, 1.0, 32.0, 1.0
    be.submit(d)
    be.sync()
    if op == "Copy":
        return d
    if host_out:
        res = host_buf
    else:
        res = be.download(d.output.data, (n_out,), np.float32 if esz == 4 else np.uint16)
        be.dealloc_memory(d.output.data, max(1, n_out * esz))
    for ptr, a in dev:
        if ptr:
            be.dealloc_memory(ptr, max(1, a.nbytes))
    return res


# ----------------------------------------------------------------------------- exact arithmetic
def test_q8_quantizer_bytes_golden(be):
    g = np.load(os.path.join(GOLD, "ops_reference.npz"))
    assert np.array_equal(be.quantize_q8_0(g["q8_x"]), g["q8_blocks"])


@pytest.mark.parametrize("seed", [0, 1])
def test_q8_quantizer_bytes_random(be, oracle, seed):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(32 * 4096) * rng.choice([1e-6, 1e-2, 1.0, 1e3], size=32 * 4096)).astype(np.float32)
    x[:64] = 0.0
    x[64:96] = np.arange(32) * 0.5
    assert np.array_equal(be.quantize_q8_0(x), oracle.quantize_q8_0(x))


def test_q8_quantizer_empty(be):
    assert be.quantize_q8_0(np.zeros(0, dtype=np.float32)).size == 0


@pytest.mark.parametrize("qt", [quants.Q4_0, quants.Q8_0])
@pytest.mark.parametrize("k", [32, 4096, 11008])
def test_integer_block_dots_identical(be, oracle, qt, k):
    rng = np.random.default_rng(k + qt)
    w = quants.quantize((rng.standard_normal((1, k)) * 0.02).astype(np.float32), qt)[0]
    xq = oracle.quantize_q8_0(rng.standard_normal(k).astype(np.float32))
    assert np.array_equal(be.block_dots(qt, w, xq, k), oracle.blockdots(qt, w, xq))


def test_block_dots_extreme_values(be, oracle):
    k = 64
    w = np.zeros(k // 32 * 18, dtype=np.uint8)
    w[0:2] = np.frombuffer(np.float16(1.0).tobytes(), dtype=np.uint8)
    w[2:18] = 0xFF; w[18:20] = w[0:2]; w[20:36] = 0x00          # all nibbles 15, then all 0 (i.e. -8)
    xq = np.zeros(k // 32 * 34, dtype=np.uint8)
    xq[0:2] = w[0:2]; xq[2:34] = 127; xq[34:36] = w[0:2]; xq[36:68] = 128   # int8 127 and -128
    assert np.array_equal(be.block_dots(quants.Q4_0, w, xq, k), oracle.blockdots(quants.Q4_0, w, xq))


# ----------------------------------------------------------------------------- MatMul
SHAPES = [(4096, 4096), (11008, 4096), (4096, 11008), (32000, 4096)]   # (rows N, inner K)


@pytest.mark.parametrize("qt", [quants.Q4_0, quants.Q8_0])
@pytest.mark.parametrize("n,k", [(64, 256), (132, 1024), (4, 32)])
@pytest.mark.parametrize("t", [1, 3, 8, 11])
def test_matmul_small_shapes(be, oracle, qt, n, k, t):
    rng = np.random.default_rng(n * k + t)
    w = quants.quantize((rng.standard_normal((n, k)) * 0.02).astype(np.float32), qt)
    x = rng.standard_normal((t, k)).astype(np.float32)
    got = run(be, "MatMul", [(w, qt, (k, n), None, B.NODE_CONSTANT), (x, B.FP32, (k, t), None, B.NODE_DYNAMIC)], (n, t)).reshape(t, n)
    want = oracle.matmul(qt, w, k, n, x)
    assert close(got, want)


# MatMul of a prompt on the tensor cores (tcgen05): the same operator, the same bits
@pytest.mark.parametrize("qt", [quants.Q4_0, quants.Q8_0])
@pytest.mark.parametrize("n,k,t,norm", [(128, 32, 1, False), (128, 256, 16, False), (256, 1024, 37, True), (384, 96, 5, False), (128, 4096, 64, True),
                                        (1024, 11008, 19, False), (200, 512, 21, False), (4, 64, 3, False)])
def test_prefill_matmul_matches_oracle(be, oracle, qt, n, k, t, norm):
    """Block counts below, at and above the pipeline depths (1, 3, 8, 32, 128, 344 blocks), ragged token tiles, row counts that
    leave the last 128-row tile partly padding, with and without the RMSNorm in front; activations with a few outliers so that block scales differ widely."""
    rng = np.random.default_rng(n + k + t + qt)
    w = quants.quantize((rng.standard_normal((n, k)) * 0.02).astype(np.float32), qt)
    x = rng.standard_normal((t, k)).astype(np.float32)
    x[rng.integers(0, t, 8), rng.integers(0, k, 8)] *= 40.0
    nw = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32) if norm else None
    got = be.prefill_matmul(qt, w, n, k, x, nw, 1e-5)
    xin = oracle.mul_rows(oracle.rmsnorm(x, 1e-5), nw) if norm else x
    want = oracle.matmul(qt, w, k, n, xin)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("qt", [quants.Q4_K, quants.Q6_K])
@pytest.mark.parametrize("n,k,t,norm", [(128, 256, 1, False), (256, 1024, 70, True), (128, 2048, 64, False), (384, 4096, 129, True), (256, 11008 - 11008 % 256, 33, False)])
def test_prefill_matmul_k_quants_match_the_restatement(be, oracle, qt, n, k, t, norm):
    """K-quant weights through the tensor-core prompt kernel: 1 to 43 super-blocks, ragged tiles of 64 tokens, with and without
    the RMSNorm in front; bit-identical to the CPU restatement (the reference has no arithmetic for these types)."""
    rng = np.random.default_rng(n + k + t + qt)
    w = quants.quantize((rng.standard_normal((n, k)) * 0.02).astype(np.float32), qt)
    x = rng.standard_normal((t, k)).astype(np.float32)
    x[rng.integers(0, t, 8), rng.integers(0, k, 8)] *= 40.0
    nw = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32) if norm else None
    got = be.prefill_matmul(qt, w, n, k, x, nw, 1e-5)
    xin = oracle.mul_rows(oracle.rmsnorm(x, 1e-5), nw) if norm else x
    want = oracle.matmul(qt, w, k, n, xin)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("qt", [quants.Q4_0, quants.Q8_0])
def test_prefill_matmul_extreme_bytes(be, oracle, qt):
    """Weight blocks written byte by byte over the whole range (Q8_0: -128 and 127 included, Q4_0: nibbles 0 and 15) against
    activations whose blocks quantize to +-127 and to zeros: the tensor-core operands split every 8-bit value into two e4m3
    values, and every split must add up."""
    rng = np.random.default_rng(77 + qt)
    n, k, t = 136, 512, 21
    nb = k // 32
    bb = 18 if qt == quants.Q4_0 else 34
    raw = rng.integers(0, 256, size=(n, nb, bb), dtype=np.uint8)
    raw[:, :, 0:2] = rng.uniform(0.001, 0.05, size=(n, nb)).astype(np.float16).view(np.uint8).reshape(n, nb, 2)   # fp16 scales
    raw[0, :, 2:] = 0x80 if qt == quants.Q8_0 else 0x00          # a row of -128 / of nibble 0 (value -8)
    raw[1, :, 2:] = 0x7F if qt == quants.Q8_0 else 0xFF          # a row of 127 / of nibble 15 (value 7)
    w = np.ascontiguousarray(raw.reshape(n, nb * bb))
    x = rng.standard_normal((t, k)).astype(np.float32)
    x[0] = np.where(rng.random(k) < 0.5, 1.0, -1.0)              # every byte +-127
    x[1] = 0.0                                                   # every byte 0, scales 0
    x[2, ::2] = 0.0
    got = be.prefill_matmul(qt, w, n, k, x)
    want = oracle.matmul(qt, w, k, n, x)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_prefill_matmul_full_size_rows_sample(be, oracle):
    """The 7B FFN-down shape with a 512-token prompt: a row and token sample against the oracle, bit for bit."""
    n, k, t = 4096, 11008, 512
    rng = np.random.default_rng(5)
    w = quants.quantize((rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)), quants.Q4_0)
    x = rng.standard_normal((t, k)).astype(np.float32)
    got = be.prefill_matmul(quants.Q4_0, w, n, k, x)
    rows = np.unique(np.concatenate([[0, 127, 128, n - 1], rng.integers(0, n, size=28)]))
    cols = np.unique(np.concatenate([[0, 15, 16, t - 1], rng.integers(0, t, size=12)]))
    want = oracle.matmul(quants.Q4_0, np.ascontiguousarray(w[rows]), k, len(rows), x[cols])
    assert np.array_equal(got[np.ix_(cols, rows)].view(np.uint32), want.view(np.uint32))
    assert np.isfinite(got).all()


def test_prefill_kernel_wait_runs_out_and_is_reported():
    """A batch of blocks that is never copied: every role of the prompt kernel that waits for it gives up after the 2 ms
    bound, the kernel returns by itself, the status names the wait, and the backend computes correctly afterwards."""
    b = B.B200Backend(0)
    assert b.prefill_selftest_wait_timeout(2_000_000) in (4, 5, 6)
    w = quants.quantize((np.random.default_rng(1).standard_normal((128, 64)) * 0.02).astype(np.float32), quants.Q8_0)
    x = np.random.default_rng(2).standard_normal((3, 64)).astype(np.float32)
    got = b.prefill_matmul(quants.Q8_0, w, 128, 64, x)
    assert np.isfinite(got).all() and np.abs(got).max() > 0
    b.close()


def test_prefill_matmul_rejects_what_does_not_fit(be):
    w = np.zeros(100 * 18, dtype=np.uint8)
    x = np.zeros((2, 48), dtype=np.float32)
    with pytest.raises(B.SpybError) as e:
        be.prefill_matmul(quants.Q4_0, w, 100, 48, x)          # k not a multiple of 32
    assert e.value.status == B.UNSUPPORTED
    with pytest.raises(B.SpybError) as e:
        be.prefill_matmul(quants.Q4_K, w, 128, 128, np.zeros((2, 128), dtype=np.float32))   # K-quant rows: k a multiple of 256
    assert e.value.status == B.UNSUPPORTED


@pytest.mark.parametrize("qt", [quants.Q4_0, quants.Q8_0])
@pytest.mark.parametrize("n,k", SHAPES)
@pytest.mark.parametrize("t", [1, 4, 16])
def test_matmul_operator_sweep(be, oracle, qt, n, k, t):
    """The operator sweep of the benchmark configurations: weights N(0, 0.02), activations N(0, 1); the oracle checks a row sample."""
    rng = np.random.default_rng(99)
    w = quants.quantize((rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)), qt)
    x = rng.standard_normal((t, k)).astype(np.float32)
    pw = be.upload_constant(f"sweep_{qt}_{n}_{k}", w, qt, (k, n))
    d = B.OpDesc(); d.op_type, d.num_input = B.OP["MatMul"], 2
    px = be.upload(x); po = be.alloc_memory(n * t * 4)
    d.input[0] = B.make_tensor(pw, qt, (k, n), None, B.NODE_CONSTANT)
    d.input[1] = B.make_tensor(px, B.FP32, (k, t))
    d.output = B.make_tensor(po, B.FP32, (n, t))
    be.submit(d); be.sync()
    got = be.download(po, (t, n), np.float32)
    be.dealloc_memory(px, x.nbytes); be.dealloc_memory(po, n * t * 4)
    rows = np.unique(np.concatenate([[0, 1, n - 2, n - 1], rng.integers(0, n, size=60)]))
    want = oracle.matmul(qt, np.ascontiguousarray(w[rows]), k, len(rows), x)
    assert close(got[:, rows], want)
    assert np.isfinite(got).all()


@pytest.mark.parametrize("qt", [quants.Q4_0, quants.Q8_0, quants.Q4_K, quants.Q6_K])
@pytest.mark.parametrize("n,k,t", [(132, 512, 1), (132, 512, 5), (200, 1024, 16), (260, 2816, 41), (1100, 512, 150)])
def test_matmul_on_uploaded_constants_takes_the_model_kernels(be, oracle, qt, n, k, t):
    """MatMul through spyb_submit against a constant from spyb_upload_constant: K-quant constants run the K-quant mat-vec
    kernel in passes of four columns, and 16 columns and more run the tcgen05 GEMM against a tile copy made at first use (K-quants
    always, Q4_0 / Q8_0 when rows x columns give the GEMM enough tiles: the last case). Either way the oracle's bits (for
    K-quants: the restatement's)."""
    rng = np.random.default_rng(n + k + t + qt)
    w = quants.quantize((rng.standard_normal((n, k)) * 0.02).astype(np.float32), qt)
    x = rng.standard_normal((t, k)).astype(np.float32)
    pw = be.upload_constant(f"const_{qt}_{n}_{k}_{t}", w, qt, (k, n))
    want = oracle.matmul(qt, w, k, n, x)
    for _ in range(2):   # the second call finds the copies the first one made
        d = B.OpDesc(); d.op_type, d.num_input = B.OP["MatMul"], 2
        px = be.upload(x); po = be.alloc_memory(n * t * 4)
        d.input[0] = B.make_tensor(pw, qt, (k, n), None, B.NODE_CONSTANT)
        d.input[1] = B.make_tensor(px, B.FP32, (k, t))
        d.output = B.make_tensor(po, B.FP32, (n, t))
        be.submit(d); be.sync()
        got = be.download(po, (t, n), np.float32)
        be.dealloc_memory(px, x.nbytes); be.dealloc_memory(po, n * t * 4)
        assert np.array_equal(bits(got), bits(want))


def test_matmul_linearity_full_size(be):
    """Size-independent property at the 7B head shape: W(2x) == 2 W(x) exactly (power-of-two scaling commutes with Q8_0)."""
    rng = np.random.default_rng(5)
    n, k = 32000, 4096
    w = quants.quantize((rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)), quants.Q4_0)
    pw = be.upload_constant("lin_head", w, quants.Q4_0, (k, n))
    x = rng.standard_normal((1, k)).astype(np.float32)
    outs = [_mm(be, pw, quants.Q4_0, n, k, xx) for xx in (x, 2 * x)]
    assert np.array_equal(bits(outs[1]), bits(2 * outs[0]))


def _mm(be, pw, qt, n, k, x):
    t = x.shape[0]
    d = B.OpDesc(); d.op_type, d.num_input = B.OP["MatMul"], 2
    px = be.upload(x); po = be.alloc_memory(n * t * 4)
    d.input[0] = B.make_tensor(pw, qt, (k, n), None, B.NODE_CONSTANT)
    d.input[1] = B.make_tensor(px, B.FP32, (k, t))
    d.output = B.make_tensor(po, B.FP32, (n, t))
    be.submit(d); be.sync()
    got = be.download(po, (t, n), np.float32)
    be.dealloc_memory(px, x.nbytes); be.dealloc_memory(po, n * t * 4)
    return got


@pytest.mark.parametrize("qt", [quants.Q4_K, quants.Q6_K])
@pytest.mark.parametrize("n,k,t", [(64, 256, 1), (132, 1024, 3), (4096, 4096, 1), (11008, 4096, 4), (4096, 11008 // 256 * 256, 16)])
def test_matmul_k_quants_within_tolerance(be, qt, n, k, t):
    """Q4_K / Q6_K: the reference only defines the block layouts (no compute), so parity is unpinned: the kernel is
    compared with decoded weights (numpy) times the f32 activations in float64, gate max-abs 2e-2 / rel 1e-2."""
    rng = np.random.default_rng(n + k + t)
    w = quants.quantize((rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)), qt)
    x = rng.standard_normal((t, k)).astype(np.float32)
    got = _mm(be, be.upload(w), qt, n, k, x)
    want = x.astype(np.float64) @ quants.dequantize(w, qt).astype(np.float64).T
    err = float(np.abs(got - want).max())
    print(f"type {qt} {n}x{k} t={t}: max |d| = {err:.3e}, max |y| = {np.abs(want).max():.3e}")
    assert err <= 2e-2 and err <= 1e-2 * float(np.abs(want).max())


def test_matmul_unsupported_weight_type_is_reported(be):
    d = B.OpDesc(); d.op_type, d.num_input = B.OP["MatMul"], 2
    p = be.alloc_memory(144 * 4)
    d.input[0] = B.make_tensor(p, 3, (256, 4), (20, 160, 640, 640)); d.input[1] = B.make_tensor(p, B.FP32, (256, 1)); d.output = B.make_tensor(p, B.FP32, (4, 1))   # type 3 = Q4_1: no kernel
    with pytest.raises(B.SpybError) as e:
        be.submit(d)
    assert e.value.status == B.UNSUPPORTED


# ----------------------------------------------------------------------------- the small operators
def test_rmsnorm_mul_add_silu(be, oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3, 4096)).astype(np.float32)
    w = rng.standard_normal(4096).astype(np.float32)
    got = run(be, "NormRMS", [(x, B.FP32, (4096, 3), None, B.NODE_DYNAMIC)], (4096, 3), eps=1e-5).reshape(3, 4096)
    assert close(got, oracle.rmsnorm(x, 1e-5), rel=5e-6)
    got = run(be, "Mul", [(x, B.FP32, (4096, 3), None, B.NODE_DYNAMIC), (w, B.FP32, (4096,), None, B.NODE_CONSTANT)], (4096, 3)).reshape(3, 4096)
    assert np.array_equal(bits(got), bits(oracle.mul_rows(x, w)))
    y = rng.standard_normal((3, 4096)).astype(np.float32)
    got = run(be, "Add", [(x, B.FP32, (4096, 3), None, B.NODE_DYNAMIC), (y, B.FP32, (4096, 3), None, B.NODE_DYNAMIC)], (4096, 3)).reshape(3, 4096)
    assert np.array_equal(bits(got), bits(x + y))
    g = (rng.standard_normal(11008) * 4).astype(np.float32)
    got = run(be, "Silu", [(g, B.FP32, (11008,), None, B.NODE_DYNAMIC)], (11008,))
    assert np.array_equal(bits(got), bits(oracle.silu(g)))   # table built with the same libm: identical bits


def test_silu_golden(be):
    g = np.load(os.path.join(GOLD, "ops_reference.npz"))
    got = run(be, "Silu", [(g["silu_x"], B.FP32, (2048,), None, B.NODE_DYNAMIC)], (2048,))
    assert np.array_equal(bits(got), bits(g["silu_out"]))


def test_softmax_masked_with_host_mask(be, oracle):
    rng = np.random.default_rng(4)
    n_ctx, n_kv, heads = 64, 37, 3
    sc = (rng.standard_normal((heads, 1, n_kv)) * 3).astype(np.float32)
    mask = np.full((1, n_ctx), -np.inf, dtype=np.float32); mask[0, : n_kv - 2] = 0
    scale = float(np.float32(1.0) / np.sqrt(np.float32(128.0)))
    got = run(be, "Softmax", [(sc, B.FP32, (n_kv, 1, heads), None, B.NODE_DYNAMIC), (mask, B.INT32, (n_ctx, 1), None, B.NODE_IO)],
              (n_kv, 1, heads), scale=scale).reshape(heads, n_kv)
    for h in range(heads):
        want = oracle.softmax_masked(sc[h, 0], mask[0, :n_kv], scale)
        assert close(got[h], want, rel=2e-6)
        assert np.all(got[h][n_kv - 2:] == 0)


def test_rope_with_host_positions(be, oracle):
    rng = np.random.default_rng(6)
    x = rng.standard_normal((3, 4, 128)).astype(np.float32)
    pos = np.array([0, 17, 511], dtype=np.int32)
    got = run(be, "Rope", [(x, B.FP32, (128, 4, 3), None, B.NODE_DYNAMIC), (pos, B.INT32, (3,), None, B.NODE_IO)], (128, 4, 3), n_dim=128).reshape(3, 4, 128)
    assert np.array_equal(bits(got), bits(oracle.rope(x, pos, 10000.0)))   # cos/sin come from the host libm


def test_getrow_f32_and_q8_0(be, oracle):
    rng = np.random.default_rng(7)
    table = rng.standard_normal((50, 256)).astype(np.float32)
    ids = np.array([3, 49, 0, 3], dtype=np.int32)
    got = run(be, "GetRow", [(table, B.FP32, (256, 50), None, B.NODE_CONSTANT), (ids, B.INT32, (4,), None, B.NODE_IO)], (256, 4)).reshape(4, 256)
    assert np.array_equal(bits(got), bits(table[ids]))
    tq = quants.quantize(table, quants.Q8_0)
    got = run(be, "GetRow", [(tq, B.Q8_0, (256, 50), None, B.NODE_CONSTANT), (ids, B.INT32, (4,), None, B.NODE_IO)], (256, 4)).reshape(4, 256)
    assert np.array_equal(bits(got), bits(quants.dequantize(tq, quants.Q8_0)[ids]))


def test_getrow_q4_0_and_f16_tables(be):
    """Embedding tables the CPU backend cannot gather (it aborts on Q4_0 rows, backend/host/operator/view.cpp:65-77):
    rows decode to value = (nibble - 8) * d in the element order of the dot product (low nibbles = elements 0..15), F16
    rows widen exactly. A model with such a table runs end to end as well."""
    rng = np.random.default_rng(17)
    table = (rng.standard_normal((40, 256)) * 0.1).astype(np.float32)
    ids = np.array([39, 0, 7, 7, 12], dtype=np.int32)
    tq = quants.quantize(table, quants.Q4_0)
    got = run(be, "GetRow", [(tq, B.Q4_0, (256, 40), None, B.NODE_CONSTANT), (ids, B.INT32, (5,), None, B.NODE_IO)], (256, 5)).reshape(5, 256)
    assert np.array_equal(bits(got), bits(quants.dequantize(tq, quants.Q4_0).reshape(40, 256)[ids]))
    th = table.astype(np.float16)
    got = run(be, "GetRow", [(th.view(np.uint16), B.FP16, (256, 40), None, B.NODE_CONSTANT), (ids, B.INT32, (5,), None, B.NODE_IO)], (256, 5)).reshape(5, 256)
    assert np.array_equal(bits(got), bits(th.astype(np.float32)[ids]))


@pytest.mark.parametrize("qt", [quants.Q4_K, quants.Q6_K])
def test_getrow_k_quant_tables(be, qt):
    """Embedding tables in K-quant formats (stock Q4_K_M files keep token_embd that way): rows decode as (d * sc) * q - dmin * m
    (Q4_K) and q * (d * sc) (Q6_K), one f32 operation at a time - the numpy decoder's order."""
    rng = np.random.default_rng(19)
    table = (rng.standard_normal((24, 512)) * 0.1).astype(np.float32)
    ids = np.array([23, 0, 5, 5, 11], dtype=np.int32)
    tq = quants.quantize(table, qt)
    got = run(be, "GetRow", [(tq, qt, (512, 24), None, B.NODE_CONSTANT), (ids, B.INT32, (5,), None, B.NODE_IO)], (512, 5)).reshape(5, 512)
    assert np.array_equal(bits(got), bits(quants.dequantize(tq, qt).reshape(24, 512)[ids]))


def test_copy_into_strided_f16_cache_and_view(be, oracle):
    """KV append as the graph does it: View at a byte offset, Copy f32 -> f16 into a transposed destination."""
    rng = np.random.default_rng(8)
    n_ctx, d, t, past = 16, 64, 3, 5
    v = rng.standard_normal((t, d)).astype(np.float32)
    cache = np.zeros(d * n_ctx, dtype=np.uint16)
    pc = be.upload(cache)
    vd = B.OpDesc(); vd.op_type, vd.num_input = B.OP["View"], 1
    vd.input[0] = B.make_tensor(pc, B.FP16, (d * n_ctx,)); vd.output = B.make_tensor(None, B.FP16, (t, d), (2, 2 * n_ctx)); vd.view_offset = 2 * past
    be.submit(vd)
    assert vd.output.data == pc + 2 * past
    # source = V transposed view of [d, t] f32: elements (t, d), strides (d*4, 4)
    pv = be.upload(v)
    cd = B.OpDesc(); cd.op_type, cd.num_input = B.OP["Copy"], 2
    cd.input[0] = B.make_tensor(pv, B.FP32, (t, d), (4 * d, 4)); cd.input[1] = vd.output; cd.output = B.make_tensor(None, B.FP16, (t, d))
    be.submit(cd); be.sync()
    assert cd.output.data == vd.output.data
    got = be.download(pc, (d, n_ctx), np.uint16)
    want = np.zeros((d, n_ctx), dtype=np.uint16)
    want[:, past:past + t] = oracle.quantize_f16(v).reshape(t, d).T
    assert np.array_equal(got, want)


def test_matmul_f16_strided_scores(be, oracle):
    """attn_score as the graph issues it: K view [hd, n_kv, H] with strides (2, d*2, hd*2) times Q [hd, 1, H] f32."""
    rng = np.random.default_rng(9)
    hd, heads, n_kv = 128, 2, 9
    d = hd * heads
    kc = oracle.quantize_f16(rng.standard_normal(n_kv * d).astype(np.float32))
    q = rng.standard_normal((heads, 1, hd)).astype(np.float32)
    got = run(be, "MatMul", [(kc, B.FP16, (hd, n_kv, heads), (2, d * 2, hd * 2), B.NODE_CACHE), (q, B.FP32, (hd, 1, heads), None, B.NODE_DYNAMIC)],
              (n_kv, 1, heads)).reshape(heads, n_kv)
    k2 = kc.reshape(n_kv, heads, hd)
    for h in range(heads):
        qh = oracle.quantize_f16(q[h, 0])
        want = np.array([oracle.dot("f16_f16", np.ascontiguousarray(k2[j, h]), qh, hd) for j in range(n_kv)], dtype=np.float32)
        assert close(got[h], want, rel=2e-6)


def test_alloc_free_reuse_and_callback(be):
    a = be.alloc_memory(1000); b = be.alloc_memory(5000)
    assert a % 256 == 0 and b % 256 == 0 and a != b
    be.dealloc_memory(a, 1000)
    assert be.alloc_memory(900) == a
    fired = []
    x = np.ones(64, dtype=np.float32)
    d = B.OpDesc(); d.op_type, d.num_input = B.OP["Silu"], 1
    px = be.upload(x); po = be.alloc_memory(256)
    d.input[0] = B.make_tensor(px, B.FP32, (64,)); d.output = B.make_tensor(po, B.FP32, (64,))
    be.submit(d, callback=lambda: fired.append(1))
    import time
    for _ in range(200):
        if fired:
            break
        time.sleep(0.01)
    assert fired == [1]
    be.sync()
    assert be.get_max_memory_capacity() > 100 << 30 and be.get_avail_memory_capacity() > 0


def _attention_oracle(oracle, q16, k16, vt16, pos0, n_head, hd, n_ctx, n_total=0):
    """The reference attention sub-graph composed from oracle primitives, one (token, head) at a time. Every row
    spans all n_total positions of the step; the causal mask (-inf) zeroes the ones after the token itself."""
    t, d = q16.shape
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    out = np.zeros((t, d), dtype=np.float32)
    n_kv = n_total if n_total else pos0 + t
    for i in range(t):
        mask = np.where(np.arange(n_kv) <= pos0 + i, np.float32(0), np.float32(-np.inf)).astype(np.float32)
        for h in range(n_head):
            qh = np.ascontiguousarray(q16[i, h * hd:(h + 1) * hd])
            sc = np.array([oracle.dot("f16_f16", np.ascontiguousarray(k16[j, h * hd:(h + 1) * hd]), qh, hd) for j in range(n_kv)], dtype=np.float32)
            pr = oracle.quantize_f16(oracle.softmax_masked(sc, mask, scale))
            for e in range(hd):
                out[i, h * hd + e] = oracle.dot("f16_f16", np.ascontiguousarray(vt16[h * hd + e, :n_kv]), pr, n_kv)
    return out


@pytest.mark.parametrize("pos0,t,n_total", [(0, 1, 0), (0, 4, 0), (4, 4, 0), (6, 1, 0), (30, 3, 0), (31, 2, 0), (63, 2, 0), (100, 1, 0),
                                            (0, 4, 8), (4, 3, 9), (28, 4, 37), (60, 4, 70), (0, 8, 8)])
@pytest.mark.parametrize("spread", [0.5, 4.0, 30.0])
def test_fused_attention_bits(be, oracle, pos0, t, n_total, spread):
    """Fused scores / softmax / PV against the oracle on wide-range values, across the 32-element boundaries of
    both dot products (n_kv = 1 .. 101)."""
    rng = np.random.default_rng(pos0 * 7 + t + int(spread * 10))
    n_head, hd, n_ctx = 2, 128, 128
    d = n_head * hd
    wide = lambda n: (rng.standard_normal(n) * rng.choice([0.05, 1.0, spread], size=n)).astype(np.float32)
    q16 = oracle.quantize_f16(wide(t * d)).reshape(t, d)
    k16 = oracle.quantize_f16(wide(n_ctx * d)).reshape(n_ctx, d)
    vt16 = oracle.quantize_f16(wide(n_ctx * d)).reshape(d, n_ctx)
    got = be.attention(q16, k16, vt16, pos0, n_head, hd, n_ctx, n_total)
    want = _attention_oracle(oracle, q16, k16, vt16, pos0, n_head, hd, n_ctx, n_total)
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("pos0,t,n_total,n_ctx", [(255, 1, 0, 512), (256, 2, 0, 512), (300, 1, 0, 512), (511, 1, 0, 512), (700, 2, 703, 1024), (1023, 1, 0, 1024),
                                                  (0, 1, 0, 2048), (5, 3, 0, 2048), (1500, 2, 0, 2048), (3000, 3, 3010, 4096), (4094, 2, 0, 4096), (4095, 1, 0, 4096)])
def test_fused_attention_long_rows(be, oracle, pos0, t, n_total, n_ctx):
    """Rows longer than the CTA (more than 256 positions: several positions per thread, many 32-position PV steps) up to
    a full context, against the oracle. Contexts above 1024 positions take the three-kernel path (scores, softmax and PV
    spread over the chip), at short and at full rows."""
    rng = np.random.default_rng(pos0 + n_ctx)
    n_head, hd = 1, 128
    d = n_head * hd
    wide = lambda n: (rng.standard_normal(n) * rng.choice([0.05, 1.0, 4.0], size=n)).astype(np.float32)
    q16 = oracle.quantize_f16(wide(t * d)).reshape(t, d)
    k16 = oracle.quantize_f16(wide(n_ctx * d)).reshape(n_ctx, d)
    vt16 = oracle.quantize_f16(wide(n_ctx * d)).reshape(d, n_ctx)
    got = be.attention(q16, k16, vt16, pos0, n_head, hd, n_ctx, n_total)
    want = _attention_oracle(oracle, q16, k16, vt16, pos0, n_head, hd, n_ctx, n_total)
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("pos0,t,n_total", [(0, 11, 0), (250, 16, 0), (1200, 9, 1215), (31, 8, 40), (2030, 18, 2048)])
def test_attention_of_a_prompt_shares_k_and_v_rows(be, oracle, pos0, t, n_total):
    """Eight and more tokens above 1024 positions of context: tiles of eight tokens share the K rows (scores) and the V^T rows
    (PV); every token's result must still be the oracle's bits - ragged last tiles, tiles that straddle 32- and 256-position
    boundaries, rows that end at the context's end."""
    rng = np.random.default_rng(pos0 + t)
    n_head, hd, n_ctx = 2, 128, 2048
    d = n_head * hd
    wide = lambda n: (rng.standard_normal(n) * rng.choice([0.05, 1.0, 4.0], size=n)).astype(np.float32)
    q16 = oracle.quantize_f16(wide(t * d)).reshape(t, d)
    k16 = oracle.quantize_f16(wide(n_ctx * d)).reshape(n_ctx, d)
    vt16 = oracle.quantize_f16(wide(n_ctx * d)).reshape(d, n_ctx)
    got = be.attention(q16, k16, vt16, pos0, n_head, hd, n_ctx, n_total)
    want = _attention_oracle(oracle, q16, k16, vt16, pos0, n_head, hd, n_ctx, n_total)
    assert np.array_equal(bits(got), bits(want))


def test_lookup_tables_identical_for_every_key(be, oracle):
    silu, ex = be.read_tables()
    want_silu, want_exp = oracle.tables()
    assert np.array_equal(bits(silu), bits(want_silu))
    assert np.array_equal(bits(ex), bits(want_exp))
