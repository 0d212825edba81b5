"""Tensor-parallel partition of one LLaMa layer. The arithmetic is the library's own (spyb_tp_layer_shard, the function
spyb_model_load_gguf cuts its shards with), bound here so that it can be checked without a GPU: rank r of N owns the heads
[r*H/N, (r+1)*H/N) - those rows of Wq, Wk, Wv, their KV cache and attention - and the FFN columns [r*F/N, (r+1)*F/N) - those
rows of W_up / W_gate. The attention output and the FFN activation are all-gathered; Wo, W_down, the norms, the residual
stream, the embeddings and the head are replicated, so no floating-point sum is ever split across ranks.

The reference has no tensor parallelism (backend/distributor: graph_divider is empty)."""
import ctypes as C
from dataclasses import dataclass

from . import backend


@dataclass(frozen=True)
class LayerShard:
    rank: int
    tp: int
    qkv_rows: range        # rows of each of Wq, Wk, Wv held by this rank = its elements of the gathered attention output
    ffn_rows: range        # rows of W_up and W_gate = its elements of the gathered FFN activation


def layer_shard(d_model: int, n_head: int, n_ff: int, tp: int, rank: int) -> LayerShard:
    out = (C.c_int64 * 4)()
    if backend.lib().spyb_tp_layer_shard(d_model, n_head, n_ff, tp, rank, out) != backend.SUCCESS:
        raise ValueError(f"tp_size {tp} / rank {rank} does not give whole heads and whole 32-element FFN blocks")
    return LayerShard(rank, tp, range(out[0], out[0] + out[1]), range(out[2], out[2] + out[3]))
