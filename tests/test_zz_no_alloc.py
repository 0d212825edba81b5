"""GPU: spyb_matmul_noalloc - the MatMul entry point that allocates nothing (its scratch for the re-tiled weights is a
fixed array inside the library image) - against the existing entry point, spyb_submit(MatMul), on the same inputs.
Two calls in a row share the scratch array: the second must not see anything of the first. The file is collected last
and passes on its own as well as after every other test."""
import numpy as np
import pytest

from spy_b200 import backend as B
from spy_b200 import quants

pytestmark = pytest.mark.gpu


def _device_free_bytes():
    import torch
    return torch.cuda.mem_get_info(0)[0]


def _submit_matmul(be, pw, qt, n, k, px, t, po):
    d = B.OpDesc(); d.op_type, d.num_input = B.OP["MatMul"], 2
    d.input[0] = B.make_tensor(pw, qt, (k, n), None, B.NODE_DYNAMIC)
    d.input[1] = B.make_tensor(px, B.FP32, (k, t))
    d.output = B.make_tensor(po, B.FP32, (n, t))
    be.submit(d); be.sync()


@pytest.mark.parametrize("qt", [quants.Q4_0, quants.Q8_0])
def test_two_calls_in_a_row_match_submit(qt, oracle):
    be = B.B200Backend(0)
    _device_free_bytes()                             # (the first query sets the measuring library up)
    rng = np.random.default_rng(123 + qt)
    # second call: a different shape over the same scratch array; third: k / 32 = 129 is not a multiple of 8, so the
    # zero padding of its rows lies over bytes the larger calls left behind
    cases = [(4096, 4096, 1), (1024, 11008, 3), (1024, 4128, 2)]
    bufs = []
    for n, k, t in cases:
        w = quants.quantize((rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)), qt)
        x = rng.standard_normal((t, k)).astype(np.float32)
        pw, px = be.upload(w), be.upload(x)
        po_ref, po_new = be.alloc_memory(n * t * 4), be.alloc_memory(n * t * 4)
        bufs.append((n, k, t, w, x, pw, px, po_ref, po_new))
    for n, k, t, w, x, pw, px, po_ref, po_new in bufs:
        _submit_matmul(be, pw, qt, n, k, px, t, po_ref)
    # The first call on a device is the set-up call (it looks the scratch array's address up, which is also when the
    # driver makes the library image's 32 MiB array resident); it is made once before anything is measured.
    n, k, t, w, x, pw, px, po_ref, po_new = bufs[0]
    be.matmul_noalloc(qt, pw, n, k, px, t, po_new)
    be.sync()
    # the no-allocation calls back to back on the backend's stream, one synchronisation at the end; neither the arena
    # behind spyb_alloc nor the device's free memory may move while they run
    arena_before, dev_before = be.get_avail_memory_capacity(), _device_free_bytes()
    for n, k, t, w, x, pw, px, po_ref, po_new in bufs:
        be.matmul_noalloc(qt, pw, n, k, px, t, po_new)
    be.sync()
    assert be.get_avail_memory_capacity() == arena_before and _device_free_bytes() == dev_before
    for n, k, t, w, x, pw, px, po_ref, po_new in bufs:
        want = be.download(po_ref, (t, n), np.float32)
        got = be.download(po_new, (t, n), np.float32)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        assert np.isfinite(got).all() and np.abs(got).max() > 0
        if n * k <= 1024 * 11008:      # and bit for bit against the CPU oracle (the larger matrix is covered through spyb_submit)
            cpu = oracle.matmul(qt, w, k, n, x)
            assert np.array_equal(got.view(np.uint32), np.asarray(cpu, dtype=np.float32).reshape(t, n).view(np.uint32))
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
    with pytest.raises(B.SpybError) as e:      # a view that is not 16-byte aligned would fault inside the kernel: refused on the host
        be.matmul_noalloc(quants.Q4_0, p, 8, 64, p + 4, 1, p)
    assert e.value.status == B.UNSUPPORTED
    with pytest.raises(B.SpybError):
        be.matmul_noalloc(quants.Q4_0, p, 8, 64, p, 1, p + 2)
    be.close()
