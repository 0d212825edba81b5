"""Worker of the tensor-parallel GPU check (launched by tests/test_gpu_tp.py through torch.distributed.run):
every rank holds one shard of a LLaMa-shaped model, rank 0 also holds the whole model, and the tensor-parallel
logits are compared with the single-GPU ones. The exchange is an all-gather (Wo and W_down run replicated on the
gathered vectors), so no f32 sum is split across ranks: the gate is identical bits, not a tolerance. The "deep" case
(16 layers, d_model 1024) is the one where a tensor-parallel scheme that summed partial results across ranks would be
amplified out of the tolerance by the re-quantization in front of every MatMul."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch
    import torch.distributed as dist
    from spy_b200 import backend as B
    from spy_b200 import gguf_io

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group(backend="gloo", rank=rank, world_size=world)
    torch.cuda.set_device(local)
    path = sys.argv[1]
    deep = len(sys.argv) > 2 and sys.argv[2] == "deep"
    cfg = (gguf_io.LlamaConfig(n_layer=16, d_model=1024, n_head=8, n_ff=2816, n_vocab=2048, weight_std=0.03) if deep else
           gguf_io.LlamaConfig(n_layer=3, d_model=512, n_head=4, n_ff=1024, n_vocab=512, weight_std=0.05))
    if rank == 0:
        gguf_io.make_llama_gguf(path, cfg, seed=5)
    dist.barrier()
    prompt = np.random.default_rng(3).integers(3, cfg.n_vocab, size=9)

    be = B.B200Backend(local, tp_size=world, tp_rank=rank)
    m = B.LlamaModel(be, path, n_ctx=64)
    uid = [B.nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    m.init_tp(uid[0])
    if os.environ.get("SPYB_TP_NCCL_ONLY") is None:   # all-gather through peer memory inside the kernels (else: NCCL all-gathers)
        handles = [None] * world
        dist.all_gather_object(handles, m.tp_export())
        m.tp_import(handles)
    ids, logits = m.generate(prompt, 12)
    # a prompt long enough for the tensor-core GEMM path: every rank runs its heads and FFN rows for all tokens, the attention
    # output and the FFN activation are all-gathered once per layer
    long_prompt = np.random.default_rng(4).integers(3, cfg.n_vocab, size=41)
    long_logits = m.eval(long_prompt, 0).copy()
    # batches of sequences on the sharded model (every step one pass of the GEMM path, the sequences as its tokens): 3 and 18
    # sequences, each with its own 9-token prompt, decoded in lockstep
    batches = {}
    for nb in (3, 18):
        m.set_sequences(nb)
        prompts = [np.random.default_rng(100 + c).integers(3, cfg.n_vocab, size=9) for c in range(nb)]
        firsts = []
        for c in range(nb):
            m.select_sequence(c)
            firsts.append(int(np.argmax(m.eval(prompts[c], 0))))
        b_ids, b_logits = m.decode_batch(firsts, 9, 5, want_logits=True)
        batches[nb] = (prompts, firsts, b_ids.copy(), b_logits.copy())
    ok = True
    if rank == 0:
        b1 = B.B200Backend(local)
        m1 = B.LlamaModel(b1, path, n_ctx=64)
        ids1, logits1 = m1.generate(prompt, 12)
        err = float(np.abs(logits - logits1).max())
        same_bits = bool(np.array_equal(np.asarray(logits, dtype=np.float32).view(np.uint32), np.asarray(logits1, dtype=np.float32).view(np.uint32)))
        long_same = bool(np.array_equal(long_logits.view(np.uint32), m1.eval(long_prompt, 0).view(np.uint32)))
        batch_same = True
        for nb, (prompts, firsts, b_ids, b_logits) in batches.items():
            for c in range(nb):
                i1, l1 = m1.generate(prompts[c], 6)
                batch_same = batch_same and int(i1[0]) == firsts[c] and bool(np.array_equal(i1[1:], b_ids[:, c]))
                batch_same = batch_same and bool(np.array_equal(l1[1:].view(np.uint32), b_logits[:, c].view(np.uint32)))
        ok = bool(np.array_equal(ids, ids1)) and same_bits and long_same and batch_same
        print(f"TP{world} vs TP1 ({'deep' if deep else 'small'} model): max|dlogit| = {err:.3e}, bits identical = {same_bits}, "
              f"ids identical = {np.array_equal(ids, ids1)}, 41-token prompt bits identical = {long_same}, batches of 3 and 18 sequences bits identical = {batch_same} -> {'OK' if ok else 'FAIL'}", flush=True)
        m1.close(); b1.close()
    m.close(); be.close()
    flag = torch.tensor([0 if ok else 1])
    dist.all_reduce(flag)
    dist.destroy_process_group()
    sys.exit(int(flag.item() != 0))


if __name__ == "__main__":
    main()
