"""Tensor-parallel partition of one LLaMa layer, as `spyb_model_load_gguf` cuts it at upload
(spy_b200/csrc/spyb_model.cu): rank r of N owns the heads [r*H/N, (r+1)*H/N) - i.e. those rows of Wq, Wk, Wv
and the matching input columns of Wo (whole 32-element blocks: head_dim is a multiple of 32) - and the FFN
columns [r*F/N, (r+1)*F/N): those rows of W_up / W_gate and the matching input columns of W_down.
Norms, the residual stream, embeddings and the head are replicated; the two partial [d] vectors of a layer
are summed over ranks (all-reduce), rank 0 carrying the residual.

The reference has no tensor parallelism (backend/distributor: graph_divider is empty); this plan is the
contract between the loader and the model step plan, kept here so that it can be checked without a GPU."""
from dataclasses import dataclass


@dataclass(frozen=True)
class LayerShard:
    rank: int
    tp: int
    qkv_rows: range        # rows of each of Wq, Wk, Wv (and columns of Wo) held by this rank
    wo_blocks: range       # 32-element blocks of every Wo row
    ffn_rows: range        # rows of W_up and W_gate
    down_blocks: range     # 32-element blocks of every W_down row
    carries_residual: bool


def check_divisible(d_model: int, n_head: int, n_ff: int, tp: int) -> None:
    if tp < 1 or n_head % tp or n_ff % tp or (n_ff // tp) % 32 or d_model % n_head:
        raise ValueError(f"tp_size {tp} does not divide heads / FFN blocks")
    if (d_model // n_head) % 32:
        raise ValueError("head_dim must be a multiple of the 32-element quantization block")


def layer_shard(d_model: int, n_head: int, n_ff: int, tp: int, rank: int) -> LayerShard:
    check_divisible(d_model, n_head, n_ff, tp)
    if not 0 <= rank < tp:
        raise ValueError("rank out of range")
    dl, fl = d_model // tp, n_ff // tp
    return LayerShard(rank, tp, range(rank * dl, (rank + 1) * dl), range(rank * dl // 32, (rank + 1) * dl // 32),
                      range(rank * fl, (rank + 1) * fl), range(rank * fl // 32, (rank + 1) * fl // 32), rank == 0)
