"""GPU: spyb_matmul_noalloc - the MatMul entry point that allocates nothing (its scratch for the re-tiled weights is a
fixed array inside the library image) - against the existing entry point, spyb_submit(MatMul), on the same inputs.
Two calls in a row share the scratch array: the second must not see anything of the first. The file is collected last
and passes on its own as well as after every other test."""
import numpy as np
import pytest

from spy_b200 import backend as B
from spy_b200 import quants

pytestmark = pytest.mark.gpu


def _submit_matmul(be, pw, qt, n, k, px, t, po):
    d = B.OpDesc(); d.op_type, d.num_input = B.OP["MatMul"], 2
    d.input[0] = B.make_tensor(pw, qt, (k, n), None, B.NODE_DYNAMIC)
    d.input[1] = B.make_tensor(px, B.FP32, (k, t))
    d.output = B.make_tensor(po, B.FP32, (n, t))
    be.submit(d); be.sync()


@pytest.mark.parametrize("qt", [quants.Q4_0, quants.Q8_0])
def test_two_calls_in_a_row_match_submit(qt):
    be = B.B200Backend(0)
    rng = np.random.default_rng(123 + qt)
    cases = [(4096, 4096, 1), (1024, 11008, 3)]      # second call: different shape over the same scratch array
    bufs = []
    for n, k, t in cases:
        w = quants.quantize((rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)), qt)
        x = rng.standard_normal((t, k)).astype(np.float32)
        pw, px = be.upload(w), be.upload(x)
        po_ref, po_new = be.alloc_memory(n * t * 4), be.alloc_memory(n * t * 4)
        bufs.append((n, k, t, w, x, pw, px, po_ref, po_new))
    for n, k, t, w, x, pw, px, po_ref, po_new in bufs:
        _submit_matmul(be, pw, qt, n, k, px, t, po_ref)
    # the two no-allocation calls back to back on the backend's stream, one synchronisation at the end
    for n, k, t, w, x, pw, px, po_ref, po_new in bufs:
        be.matmul_noalloc(qt, pw, n, k, px, t, po_new)
    be.sync()
    for n, k, t, w, x, pw, px, po_ref, po_new in bufs:
        want = be.download(po_ref, (t, n), np.float32)
        got = be.download(po_new, (t, n), np.float32)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        assert np.isfinite(got).all() and np.abs(got).max() > 0
    be.close()


def test_rejects_what_does_not_fit():
    be = B.B200Backend(0)
    p = be.alloc_memory(1 << 20)
    with pytest.raises(B.SpybError) as e:      # 32000 x 4096 Q4_0 re-tiles to 73.7 MB > 32 MiB
        be.matmul_noalloc(quants.Q4_0, p, 32000, 4096, p, 1, p)
    assert e.value.status == B.UNSUPPORTED
    with pytest.raises(B.SpybError):           # rows not a multiple of 4
        be.matmul_noalloc(quants.Q4_0, p, 6, 64, p, 1, p)
    with pytest.raises(B.SpybError):           # K-quants have no exact kernel
        be.matmul_noalloc(quants.Q4_K, p, 8, 256, p, 1, p)
    be.close()
