"""CPU, world size 2 over gloo: the tensor-parallel partition of a layer (spy_b200/tp_plan.py, the contract the
device loader follows) reproduces the unsharded layer when the two partial vectors are all-reduced.
The arithmetic here is float64 numpy on dequantized Q4_0 weights: this checks the host-side sharding logic
(which rows / which K blocks go where, who carries the residual), not kernel arithmetic."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from spy_b200 import quants, tp_plan

D, H, F = 256, 2, 512


def _weights():
    rng = np.random.default_rng(17)
    w = {}
    for name, shape in [("q", (D, D)), ("k", (D, D)), ("v", (D, D)), ("o", (D, D)), ("up", (F, D)), ("gate", (F, D)), ("down", (D, F))]:
        f = rng.standard_normal(shape).astype(np.float32) * 0.05
        w[name] = quants.dequantize_q4_0(quants.quantize_q4_0(f)).reshape(shape).astype(np.float64)
    return w, rng.standard_normal(D)


def _layer(w, x, sh):
    """One layer on the shard `sh` (attention reduced to a per-head mixing that needs q, k, v of the same head, so
    that a wrong head split shows): returns the two partial vectors that are summed over ranks."""
    hd = D // H
    rows = np.array(sh.qkv_rows)
    q, k, v = w["q"][rows] @ x, w["k"][rows] @ x, w["v"][rows] @ x
    att = np.concatenate([(q[i:i + hd] @ k[i:i + hd]) * v[i:i + hd] for i in range(0, len(rows), hd)])
    cols = np.arange(sh.wo_blocks.start * 32, sh.wo_blocks.stop * 32)
    assert np.array_equal(cols, rows)                      # Wo's input columns are the rank's head outputs
    part1 = w["o"][:, cols] @ att + (x if sh.carries_residual else 0.0)
    return part1, rows


def _ffn(w, h, sh):
    rows = np.array(sh.ffn_rows)
    up, gate = w["up"][rows] @ h, w["gate"][rows] @ h
    act = up * (gate / (1.0 + np.exp(-gate)))
    cols = np.arange(sh.down_blocks.start * 32, sh.down_blocks.stop * 32)
    assert np.array_equal(cols, rows)
    return w["down"][:, cols] @ act + (h if sh.carries_residual else 0.0)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    w, x = _weights()
    sh = tp_plan.layer_shard(D, H, F, world, rank)
    p1, _ = _layer(w, x, sh)
    t = torch.from_numpy(p1.copy()); dist.all_reduce(t); h = t.numpy()
    t2 = torch.from_numpy(_ffn(w, h, sh).copy()); dist.all_reduce(t2)
    if rank == 0:
        np.save(out, t2.numpy())
    dist.destroy_process_group()


def test_two_rank_partition_reproduces_the_layer(tmp_path):
    out = str(tmp_path / "tp2.npy")
    mp.spawn(_worker, args=(2, 29611, out), nprocs=2, join=True)
    w, x = _weights()
    full = tp_plan.layer_shard(D, H, F, 1, 0)
    h, _ = _layer(w, x, full)
    want = _ffn(w, h, full)
    got = np.load(out)
    assert np.allclose(got, want, rtol=1e-10, atol=1e-12)


def test_partition_covers_everything_once_and_rejects_bad_splits():
    for tp in (1, 2, 4, 8):
        shards = [tp_plan.layer_shard(4096, 32, 11008, tp, r) for r in range(tp)]
        assert sorted(i for s in shards for i in s.qkv_rows) == list(range(4096))
        assert sorted(i for s in shards for i in s.ffn_rows) == list(range(11008))
        assert sorted(i for s in shards for i in s.wo_blocks) == list(range(128))
        assert sorted(i for s in shards for i in s.down_blocks) == list(range(344))
        assert sum(s.carries_residual for s in shards) == 1
    with pytest.raises(ValueError):
        tp_plan.layer_shard(4096, 32, 11008, 3, 0)      # 32 heads do not split in three
    with pytest.raises(ValueError):
        tp_plan.layer_shard(4096, 32, 11008, 16, 0)     # 11008 / 16 = 688 is not a whole number of 32-blocks... (688 = 21.5 * 32)
    with pytest.raises(ValueError):
        tp_plan.layer_shard(4096, 32, 11008, 2, 2)
