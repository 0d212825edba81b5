"""CPU, world size 2 over gloo: the tensor-parallel partition of a layer - the library's own shard arithmetic
(spyb_tp_layer_shard through spy_b200/tp_plan.py) - reproduces the unsharded layer when the attention output and the FFN
activation are all-gathered and Wo / W_down run replicated. The arithmetic here is float64 numpy on dequantized Q4_0
weights: this checks the host-side sharding logic (which rows go where, what is gathered), not kernel arithmetic."""
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


def _attention_share(w, x, sh):
    """This rank's elements of the attention output (attention reduced to a per-head mixing that needs q, k, v of the
    same head, so that a wrong head split shows)."""
    hd = D // H
    rows = np.array(sh.qkv_rows)
    q, k, v = w["q"][rows] @ x, w["k"][rows] @ x, w["v"][rows] @ x
    return np.concatenate([(q[i:i + hd] @ k[i:i + hd]) * v[i:i + hd] for i in range(0, len(rows), hd)])


def _ffn_share(w, h, sh):
    rows = np.array(sh.ffn_rows)
    up, gate = w["up"][rows] @ h, w["gate"][rows] @ h
    return up * (gate / (1.0 + np.exp(-gate)))


def _gather(share, world):
    parts = [torch.zeros(len(share), dtype=torch.float64) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(share.copy()))
    return torch.cat(parts).numpy()


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    w, x = _weights()
    sh = tp_plan.layer_shard(D, H, F, world, rank)
    att = _gather(_attention_share(w, x, sh), world)          # shares are contiguous rank ranges: concatenation = the vector
    h = w["o"] @ att + x                                      # replicated
    act = _gather(_ffn_share(w, h, sh), world)
    y = w["down"] @ act + h                                   # replicated
    if rank == 0:
        np.save(out, y)
    dist.destroy_process_group()


def test_two_rank_partition_reproduces_the_layer(tmp_path):
    out = str(tmp_path / "tp2.npy")
    mp.spawn(_worker, args=(2, 29611, out), nprocs=2, join=True)
    w, x = _weights()
    full = tp_plan.layer_shard(D, H, F, 1, 0)
    h = w["o"] @ _attention_share(w, x, full) + x
    want = w["down"] @ _ffn_share(w, h, full) + h
    got = np.load(out)
    assert np.allclose(got, want, rtol=1e-12, atol=1e-13)


def test_partition_covers_everything_once_and_rejects_bad_splits():
    for tp in (1, 2, 4, 8):
        shards = [tp_plan.layer_shard(4096, 32, 11008, tp, r) for r in range(tp)]
        assert sorted(i for s in shards for i in s.qkv_rows) == list(range(4096))
        assert sorted(i for s in shards for i in s.ffn_rows) == list(range(11008))
        assert all(len(s.qkv_rows) % 128 == 0 and len(s.ffn_rows) % 32 == 0 for s in shards)     # whole heads, whole blocks
        assert [s.qkv_rows.start for s in shards] == sorted(s.qkv_rows.start for s in shards)    # rank order = element order
    for tp in (2, 4, 8):                                      # the 13B shapes the tensor-parallel configuration is specified on
        shards = [tp_plan.layer_shard(5120, 40, 13824, tp, r) for r in range(tp)]
        assert sorted(i for s in shards for i in s.ffn_rows) == list(range(13824))
    with pytest.raises(ValueError):
        tp_plan.layer_shard(4096, 32, 11008, 3, 0)      # 32 heads do not split in three
    with pytest.raises(ValueError):
        tp_plan.layer_shard(4096, 32, 11008, 16, 0)     # 11008 / 16 = 688 is not a whole number of 32-blocks
    with pytest.raises(ValueError):
        tp_plan.layer_shard(4096, 32, 11008, 2, 2)
