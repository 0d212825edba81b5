#!/usr/bin/env python
"""Decode-throughput benchmark of the LLaMa token loop on the sm_100a backend.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one single-token decode step (one execute() of the graph, batch 1) of a synthetic
LLaMa2-7B-architecture model with Q4_0 weights (seeded N(0, 0.02), norms = 1, F32 embeddings),
context 512, after an 8-token seeded prompt. With N > 1 the model is sharded tensor-parallel over
N GPUs (launched by torchrun, one rank per GPU: heads and FFN columns per rank, the attention output and the
FFN activation all-gathered over NVLink, Wo and W_down replicated - the results are the single-GPU bits),
so scaling is "strong". Rank 0 prints one JSON line.

  value          tokens/s with everything resident in HBM: CUDA-graph replay, greedy argmax and next
                 embedding on the device, timed with CUDA events on the launching stream.
  e2e            the same loop through spyb_model_eval: token id from pinned host memory in, the
                 32000 logits back to the host and the argmax there, every step.
  roofline       the dominant kernel (FFN up|gate mat-vec, 45 % of the weight bytes) timed alone over
                 all layers' weights (1.6 GB per sweep, far larger than L2) against the measured HBM peak;
                 "kernels" lists the other mat-vec launches of a step the same way.
  cpu_baseline   the reference's own CPU backend (oracle/_ref, compiled from the reference sources)
                 on the host cores, same GGUF and prompt, a few decode steps.

--impl reference times only that CPU arm and prints the same line with "impl": "reference".
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED, PROMPT_SEED, N_PROMPT, N_CTX = 1234, 4321, 8, 512
REPS = 5         # repetitions of the timed region; the median is reported
WORKLOAD = "llama2-7b-arch Q4_0 bs1 decode, ctx 512, prompt 8 (synthetic GGUF, seed 1234)"
ARCH, WTYPE_NAME = "7b", "q4_0"

# --config N selects another configuration of the baseline list (the default, 1, is the one the metric is quoted on):
#   3: 7B architecture, Q4_K_M-style mixed K-quants, prompt of 512 ids (parity for K-quants is against the CPU restatement: tests/)
#   4: 7B architecture, Q8_0 weights, f16 KV cache, context 4096, prompt of 3968 ids, decode at the end of the context
#   5: 13B architecture, Q4_0, prompt of 128 ids, decode 128 (the configuration tensor parallelism is specified on)
CONFIGS = {
    1: dict(arch="7b", wtype="q4_0", seed=1234, n_prompt=8, n_ctx=512, workload=WORKLOAD),
    2: dict(arch="7b", wtype="q4_0", seed=99, n_prompt=0, n_ctx=0,
            workload="MatMul operator sweep: Q4_0 / Q4_K / Q8_0 weights N(0, 0.02) x f32 activations N(0, 1), shapes 4096x4096, 11008x4096, "
                     "4096x11008, 32000x4096 (rows x K), batch 1 / 4 / 16 (seed 99)"),
    3: dict(arch="7b", wtype="q4_k_m", seed=1236, n_prompt=512, n_ctx=1024,
            workload="llama2-7b-arch Q4_K_M-style (Q6_K for attn_v, ffn_down, output; Q4_K elsewhere) bs1, prompt 512 + decode, ctx 1024 (synthetic GGUF, seed 1236)"),
    4: dict(arch="7b", wtype="q8_0", seed=1237, n_prompt=3968, n_ctx=4096,
            workload="llama2-7b-arch Q8_0 bs1 decode, f16 KV, ctx 4096, prompt 3968 (synthetic GGUF, seed 1237)"),
    5: dict(arch="13b", wtype="q4_0", seed=1238, n_prompt=128, n_ctx=512,
            workload="llama2-13b-arch Q4_0 bs1 decode, ctx 512, prompt 128 (synthetic GGUF, seed 1238)"),
}


def select_config(n):
    global SEED, N_PROMPT, N_CTX, WORKLOAD, ARCH, WTYPE_NAME
    c = CONFIGS[n]
    SEED, N_PROMPT, N_CTX, WORKLOAD, ARCH, WTYPE_NAME = c["seed"], c["n_prompt"], c["n_ctx"], c["workload"], c["arch"], c["wtype"]


def run_operator_sweep(args):
    """--config 2: every (weight type, shape, batch) of the operator sweep through spyb_submit(MatMul) on device-resident
    operands; device time from events on the backend's stream around back-to-back submits that walk over enough copies of
    the weights to exceed the L2 cache. Algorithmic bytes = quantized weights + f32 activations in + f32 results out."""
    import numpy as np
    from spy_b200 import backend as B, quants
    be = B.B200Backend(0)
    peak, peak_kind = measured_peak()
    rng = np.random.default_rng(99)
    shapes = [(4096, 4096), (11008, 4096), (4096, 11008), (32000, 4096)]
    types = [("q4_0", quants.Q4_0, 18 / 32), ("q4_k", quants.Q4_K, 144 / 256), ("q8_0", quants.Q8_0, 34 / 32)]
    sampler = ClockSampler(0); sampler.start()
    cases, launches = [], 0
    for n, k in shapes:
        wf = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
        for tname, qt, bpw in types:
            w = quants.quantize(wf, qt)
            w_bytes = int(n * k * bpw)
            copies = max(2, -(-300_000_000 // w_bytes))
            pws = [be.upload_constant(f"sweep_{tname}_{n}_{k}_{c}", w, qt, (k, n)) for c in range(copies)]
            for t in (1, 4, 16):
                x = rng.standard_normal((t, k)).astype(np.float32)
                px = be.upload(x); po = be.alloc_memory(n * t * 4)
                descs = []
                for pw in pws:
                    d = B.OpDesc(); d.op_type, d.num_input = B.OP["MatMul"], 2
                    d.input[0] = B.make_tensor(pw, qt, (k, n), None, B.NODE_CONSTANT)
                    d.input[1] = B.make_tensor(px, B.FP32, (k, t))
                    d.output = B.make_tensor(po, B.FP32, (n, t))
                    descs.append(d)
                reps = max(args.steps, 2 * copies)
                be.submit_timed(descs, max(args.warmup, copies))
                ms = be.submit_timed(descs, reps)
                us = ms * 1e3 / reps
                alg = w_bytes + 4 * k * t + 4 * n * t
                cases.append({"type": tname, "rows": n, "k": k, "batch": t, "us": us, "gbs": alg / us / 1e3, "frac": alg / us / 1e3 / peak, "bytes": alg, "weight_copies": copies})
                launches += reps
                be.dealloc_memory(px, x.nbytes); be.dealloc_memory(po, n * t * 4)
    clocks = sampler.stop()
    be.close()
    geo = float(np.exp(np.mean([np.log(c["gbs"]) for c in cases])))
    dom = max((c for c in cases if c["batch"] == 1), key=lambda c: c["gbs"])
    line = {"metric": "MatMul operator sweep, geometric mean of achieved GB/s", "value": geo, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": float(np.mean([c["us"] for c in cases])) / 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 block dots, f32 accumulate", "data": "synthetic",
            "config": {"workload": WORKLOAD, "l2": "every case walks over copies of its weights that total 300 MB and more (L2: 126 MB)",
                       "timing": "CUDA events on the backend's stream around back-to-back spyb_submit(MatMul) calls"},
            "roofline": {"bound": "hbm", "kernel": f"MatMul {dom['type']} {dom['rows']}x{dom['k']} batch 1 (best single-column case)", "achieved": dom["gbs"], "peak": peak,
                         "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": dom["frac"], "traffic": None},
            "cpu_baseline": None, "e2e": None, "gpu_launches": launches, "clocks": clocks, "sweep": cases}
    print(json.dumps(line))


def model_path():
    d = "/dev/shm" if os.path.isdir("/dev/shm") and os.access("/dev/shm", os.W_OK) else "/tmp"
    return os.path.join(d, f"spyb_llama{ARCH}_{WTYPE_NAME}_seed{SEED}.gguf")


def ensure_model(path, device):
    from spy_b200 import gguf_io, quants
    if os.path.exists(path) and os.path.getsize(path) > 4_000_000_000:
        return
    arch = gguf_io.LLAMA2_13B if ARCH == "13b" else gguf_io.LLAMA2_7B
    if WTYPE_NAME == "q4_k_m":
        cfg = gguf_io.LlamaConfig(**arch, wtype=quants.Q4_K, overrides={"attn_v": quants.Q6_K, "ffn_down": quants.Q6_K, "output": quants.Q6_K})
    else:
        cfg = gguf_io.LlamaConfig(**arch, wtype=quants.Q8_0 if WTYPE_NAME == "q8_0" else quants.Q4_0)
    tmp = path + f".tmp{os.getpid()}"
    gguf_io.make_llama_gguf_cuda(tmp, cfg, seed=SEED, device=device)
    os.replace(tmp, path)


def prompt_ids(n_vocab=32000):
    return np.random.default_rng(PROMPT_SEED).integers(3, n_vocab, size=N_PROMPT).astype(np.int32)


def physical_cores():
    try:
        allowed = os.sched_getaffinity(0)
        cores, phys, core, cpu = set(), None, None, None
        for line in open("/proc/cpuinfo"):
            if line.startswith("processor"):
                cpu = int(line.split(":")[1])
            elif line.startswith("physical id"):
                phys = int(line.split(":")[1])
            elif line.startswith("core id"):
                core = int(line.split(":")[1])
            elif not line.strip():
                if cpu in allowed and phys is not None and core is not None:
                    cores.add((phys, core))
                phys = core = cpu = None
        n = len(cores) if cores else len(allowed)
    except Exception:
        n = os.cpu_count() or 1
    return max(1, min(n, 64))


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs (read-only queries)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=3)
        except Exception:
            self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def bf16_peak_tflops():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p)).get("bf16_tflops", 1590.0))
    return 1590.0


N_PARITY = 32   # generated tokens of the parity record: the 8-token prompt, then 32 greedy tokens


def cpu_reference_run(path, steps, warmup, threads, want_logits=False, n_vocab=None):
    """Reference CPU backend: prefill of the prompt, then warmup + steps single-token decode steps."""
    from oracle import spy_ref
    if not spy_ref.available():
        return None
    n = 1 + warmup + steps
    ids, logits, ms = spy_ref.generate(path, prompt_ids(), n, n_ctx=N_CTX, threads=threads, warmup=False, want_logits=want_logits, n_vocab=n_vocab)
    dec = ms[1 + warmup:]
    return {"tokens_per_s": float(len(dec) / (dec.sum() / 1e3)), "ms_per_step": float(dec.mean()), "ids": ids, "logits": logits,
            "prefill_ms": float(ms[0])}


def parity_record(ids, logits, want_ids, want_logits):
    """The stated gates: greedy ids identical; per-step logits within max-abs 2e-2 and rel 1e-2 (relative to the step's
    largest |logit|); plus the smallest gap between the two largest logits of a step (what a flipped id would need)."""
    ids, want_ids = np.asarray(ids), np.asarray(want_ids)
    logits, want_logits = np.asarray(logits, dtype=np.float32), np.asarray(want_logits, dtype=np.float32)
    n = min(len(ids), len(want_ids))
    d = np.abs(logits[:n] - want_logits[:n]).max(axis=1)
    scale = np.abs(want_logits[:n]).max(axis=1)
    top2 = np.sort(want_logits[:n], axis=1)[:, -2:]
    rec = {"n_ids": int(n), "ids_identical": bool(np.array_equal(ids[:n], want_ids[:n])), "max_abs_dlogit": float(d.max()),
           "max_rel_dlogit": float((d / np.maximum(scale, 1e-30)).max()), "min_top2_gap": float((top2[:, 1] - top2[:, 0]).min()),
           "bits_identical": bool(np.array_equal(logits[:n].view(np.uint32), want_logits[:n].view(np.uint32)))}
    rec["within_tolerance"] = bool(rec["ids_identical"] and rec["max_abs_dlogit"] <= 2e-2 and rec["max_rel_dlogit"] <= 1e-2)
    return rec


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    path = model_path()
    if not os.path.exists(path):
        import torch
        if not torch.cuda.is_available():
            print(json.dumps({"impl": "reference", "unavailable": "the synthetic 7B GGUF is generated on the GPU and no CUDA device is visible"}))
            return
        ensure_model(path, "cuda:0")
    threads = physical_cores()
    steps = max(1, min(args.steps, N_CTX - N_PROMPT - args.warmup - 1))
    r = cpu_reference_run(path, steps, args.warmup, threads)
    if r is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libspy_ref.so (the reference's CPU path) was not built"}))
        return
    line = {"impl": "reference", "metric": "decode tokens/s", "value": r["tokens_per_s"], "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8 block dots, f32 accumulate", "data": "synthetic",
            "config": {"workload": WORKLOAD, "threads": threads},
            "cpu_baseline": {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": threads, "kind": "reference",
                             "sample": f"{steps} decode steps after an 8-token prefill, -t {threads}"},
            "e2e": {"value": r["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=1, choices=sorted(CONFIGS), help="configuration of the baseline list (default 1: the one the metric is quoted on)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--profile-step", type=int, default=0, metavar="LAYERS",
                    help="load only the first LAYERS blocks of the model, evaluate the prompt, decode 4 tokens and exit: the small case for an ncu capture of the single-token step kernel")
    ap.add_argument("--no-batch", action="store_true", help="skip the batch-of-sequences record")
    ap.add_argument("--profile-prefill", type=int, default=0, metavar="LAYERS",
                    help="load only the first LAYERS blocks of the model, evaluate a 448-token prompt twice and exit: the small case for an ncu capture of the prompt kernels")
    ap.add_argument("--profile-kernel", type=int, default=-1, metavar="KIND",
                    help="load the model, run two sweeps of one mat-vec kind over all layers (0 qkv, 1 attn_out, 2 ffn_up_gate, 3 ffn_down, 4 head) and exit: the small case for an ncu capture")
    args = ap.parse_args()
    select_config(args.config)
    if args.config != 1:
        args.no_cpu_baseline = True     # the CPU arm needs minutes to hours for these prompts; parity for them is in tests/
    if args.impl == "reference" and args.config == 2:
        print(json.dumps({"impl": "reference", "unavailable": "the operator sweep is timed on the GPU arm only; its parity against the CPU operators is in tests/test_gpu_ops.py"}))
        return
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.config == 2:
        run_operator_sweep(args)
        return

    import torch
    from spy_b200 import backend as B

    if args.profile_step > 0 or args.profile_prefill > 0:
        os.environ["SPYB_MAX_LAYERS"] = str(max(args.profile_step, args.profile_prefill))
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (launch with torch.distributed.run), got WORLD_SIZE={world}")
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend="gloo", rank=rank, world_size=world)
    torch.cuda.set_device(local)

    def barrier():
        if dist is not None:
            dist.barrier()

    path = model_path()
    if rank == 0:
        ensure_model(path, f"cuda:{local}")
    barrier()

    be = B.B200Backend(local, tp_size=world, tp_rank=rank, use_pdl=not args.no_pdl, use_graph=not args.no_graph)
    model = B.LlamaModel(be, path, n_ctx=N_CTX)
    if world > 1:
        uid = [B.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        model.init_tp(uid[0])
        if os.environ.get("SPYB_TP_NCCL_ONLY") is None:   # decode steps exchange through peer memory inside the kernels
            handles = [None] * world
            dist.all_gather_object(handles, model.tp_export())
            model.tp_import(handles)
    info = model.info
    prompt = prompt_ids(info.n_vocab)
    if args.profile_step > 0:
        first = model.eval(prompt, 0)
        ids, _ = model.decode(int(np.argmax(first)), N_PROMPT, 4)
        print(json.dumps({"profile_step_layers": args.profile_step, "ms_per_step": model.last_ms / 4, "ids": [int(i) for i in ids]}))
        model.close(); be.close()
        return
    if args.profile_prefill > 0:
        n_pre = max(N_PROMPT, min(512, N_CTX - 64))
        pre_ids = np.random.default_rng(PROMPT_SEED + 1).integers(3, info.n_vocab, size=n_pre).astype(np.int32)
        model.eval(pre_ids, 0)
        model.eval(pre_ids, 0)
        print(json.dumps({"profile_prefill_layers": args.profile_prefill, "tokens": int(n_pre), "ms": model.last_ms, "launches": int(model.last_launches)}))
        model.close(); be.close()
        return
    if args.profile_kernel >= 0:
        import ctypes as C
        nbytes = C.c_uint64()
        ms = be._l.spyb_model_bench_kernel(model.h, args.profile_kernel, 2, C.byref(nbytes))
        print(json.dumps({"profile_kernel": args.profile_kernel, "us_per_launch": ms * 1e3, "bytes_per_launch": int(nbytes.value)}))
        model.close(); be.close()
        return

    closed = False
    steps, warmup = args.steps, max(3, args.warmup)
    room = N_CTX - N_PROMPT - 1
    if warmup + steps > room:
        steps = room - warmup

    # ---- prompt evaluation (prefill): one eval call over a 512-token prompt (or the configuration's own, if longer) ----
    n_pre = max(N_PROMPT, min(512, N_CTX - 64))
    pre_ids = np.random.default_rng(PROMPT_SEED + 1).integers(3, info.n_vocab, size=n_pre).astype(np.int32)
    model.eval(pre_ids[:8], 0)                                # warm: the short-prompt path ...
    model.eval(pre_ids, 0)                                    # ... and the long-prompt path (first use of its kernels, buffers and, sharded, NCCL connections)
    barrier(); be.sync()
    pre_logits = model.eval(pre_ids, 0).copy()
    t_pre = torch.tensor([model.last_ms], dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t_pre, op=dist.ReduceOp.MAX)
    layer_weights = int(info.n_layer) * (4 * int(info.d_model) ** 2 + 3 * int(info.d_model) * int(info.n_ff))   # elements of the layers' matrices (all ranks together)
    pre_tflops = 2.0 * layer_weights * n_pre / (float(t_pre[0]) / 1e3) / 1e12
    prefill = {"tokens": int(n_pre), "ms": float(t_pre[0]), "tokens_per_s": float(n_pre / (float(t_pre[0]) / 1e3)),
               "launches": int(model.last_launches),
               "tflops": pre_tflops, "frac_of_bf16_peak": pre_tflops / (bf16_peak_tflops() * world),
               "tflops_note": "algorithmic: 2 x layer weights x tokens / time, against the measured dense bf16 peak of the GPUs used; the tensor cores issue 8 x "
                              "that (one MMA column per accumulator of a token: block-diagonal B operand), times 2 (Q4_0) or 4 (Q8_0) for the e4m3 split of "
                              "8-bit values, and the f32 chains after them set the time",
               "note": "one spyb_model_eval over the prompt (device time, CUDA events): chunks of up to 512 tokens through the tcgen05 GEMM kernel when the "
                       "widths fit its tiles (sharded models: each rank its heads and FFN rows, one NCCL all-gather of the attention output and of the FFN activation per layer)"}
    barrier()

    # ---- device-resident arm ---------------------------------------------------------------
    first = model.eval(prompt, 0)
    tok0 = int(np.argmax(first))
    model.decode(tok0, N_PROMPT, warmup)                      # warm-up (captures the graph on first use)
    barrier(); torch.cuda.synchronize(); be.sync()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ids_warm, _ = model.decode(tok0, N_PROMPT, warmup)        # re-run the warm-up region so the timed tokens follow it
    barrier(); be.sync()
    last_tok = int(ids_warm[-1])
    reps_ms = []
    for _ in range(REPS):                                     # the same `steps` positions every time: identical work per repetition
        barrier()
        ids, _ = model.decode(last_tok, N_PROMPT + warmup, steps)
        t = torch.tensor([model.last_ms], dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)          # device time of the slowest rank
        reps_ms.append(float(t[0]))
    ms_dev = float(np.median(reps_ms))
    launches = model.last_launches
    be.sync(); barrier()

    # ---- end-to-end arm: host token in, host logits out, argmax on the host, every step -----
    tok = last_tok
    model.eval(np.array([tok], dtype=np.int32), N_PROMPT + warmup)   # warm
    barrier(); be.sync()
    ev_ms = 0.0
    t0 = time.perf_counter()
    e2e_ids = []
    for s in range(steps):
        logits = model.eval(np.array([tok], dtype=np.int32), N_PROMPT + warmup + s)
        ev_ms += model.last_ms
        tok = int(np.argmax(logits))
        e2e_ids.append(tok)
    be.sync(); barrier()
    ms_e2e_wall = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop() if rank == 0 else None

    times = torch.tensor([ms_e2e_wall], dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_e2e = float(times[0])

    # ---- parity of the tensor-parallel run against the unsharded model, on the benchmarked model (rank 0 loads both)
    parity_tp = None
    if world > 1:
        ids_tp, logits_tp = model.decode(last_tok, N_PROMPT + warmup, min(steps, N_PARITY), want_logits=True)
        if rank == 0:
            be1 = B.B200Backend(local, tp_size=1, tp_rank=0, use_pdl=not args.no_pdl, use_graph=not args.no_graph)
            m1 = B.LlamaModel(be1, path, n_ctx=N_CTX)
            f1 = m1.eval(prompt, 0)
            w1, _ = m1.decode(int(np.argmax(f1)), N_PROMPT, warmup)
            ids_1, logits_1 = m1.decode(int(w1[-1]), N_PROMPT + warmup, min(steps, N_PARITY), want_logits=True)
            parity_tp = parity_record(ids_tp, logits_tp, ids_1, logits_1)
            parity_tp["against"] = "the same model unsharded on one GPU, same prompt and positions"
            parity_tp["warmup_ids_identical"] = bool(np.array_equal(w1, ids_warm) and int(np.argmax(f1)) == tok0)
            # and the long prompt: the sharded GEMM path (NCCL all-gathers of whole chunks) against the unsharded one
            pre_1 = m1.eval(pre_ids, 0)
            prefill["parity_tp"] = {"bits_identical": bool(np.array_equal(pre_1.view(np.uint32), pre_logits.view(np.uint32))),
                                    "max_abs_dlogit": float(np.abs(pre_1 - pre_logits).max()), "against": "the same model unsharded on one GPU, same prompt"}
            m1.close(); be1.close()
        barrier()

    # ---- a batch of independent sequences that share the weights (the batch > 1 cases of the configurations): sequence 0
    # has the benchmark's prompt, so its ids can be compared with the single-sequence run; aggregate tokens/s over all sequences
    n_batch = {1: 8, 4: 8, 5: 32}.get(args.config, 0)
    batch_rec = None
    if n_batch > 0 and not args.no_batch:
        try:
            n_cmp = min(16, room)
            ref_ids, _ = model.decode(tok0, N_PROMPT, n_cmp)
            model.set_sequences(n_batch)
            rng_b = np.random.default_rng(PROMPT_SEED + 7)
            firsts = []
            for c in range(n_batch):
                model.select_sequence(c)
                pc = prompt if c == 0 else rng_b.integers(3, info.n_vocab, size=N_PROMPT).astype(np.int32)
                firsts.append(int(np.argmax(model.eval(pc, 0))))
            b_steps = min(32, room)
            model.decode_batch(firsts, N_PROMPT, min(4, room))          # warm
            b_ids, _ = model.decode_batch(firsts, N_PROMPT, b_steps)
            batch_rec = {"sequences": n_batch, "steps": b_steps, "ms_per_step": model.last_ms / b_steps,
                         "tokens_per_s": n_batch * b_steps / (model.last_ms / 1e3), "launches": int(model.last_launches),
                         "sequence0_ids_match_single_sequence_run": bool(np.array_equal(b_ids[:n_cmp, 0], ref_ids[:n_cmp])),
                         "note": "greedy decoding of the sequences in lockstep (spyb_model_decode_batch): per step the layer weights are streamed once per group of 4 sequences "
                                 "through the mat-vec kernels (fewer than 16 sequences on one GPU), or once for all of them through the tcgen05 GEMM kernels (16 and more, "
                                 "and every batch of a tensor-parallel model: each rank on its rows, NCCL all-gathers of the whole vectors); device time of rank 0"}
            model.select_sequence(0)
        except Exception as e:  # noqa: BLE001
            batch_rec = {"error": str(e)[:300]}
    barrier()

    # ---- dominant kernel alone, over every layer's weights ----------------------------------
    roof = None
    if rank == 0:
        peak, peak_kind = measured_peak()
        kb = bench_kernels(model, be)
        dom = kb["ffn_up_gate"]
        # traffic: dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this workload's FFN
        # matrices, taken from an earlier ncu capture (the line says so in traffic_source)
        roof = {"bound": "hbm", "kernel": "matvec_rows_kernel<Q4_0, 1 column, 2 lanes per row> (fused FFN up|gate, RMSNorm+Q8_0 prologue, SiLU-mul epilogue)",
                "achieved": dom["gbs"], "peak": peak,
                "peak_kind": f"of {peak_kind} ({'MEASURED_PEAKS.json copy bandwidth' if peak_kind == 'measured' else 'fallback 6650 GB/s'})",
                "unit": "GB/s", "frac": dom["gbs"] / peak, "traffic": 50836224 if (dom["bytes"] == 50724864 and WTYPE_NAME == "q4_0") else None,
                "traffic_source": "ncu capture of this kernel on this matrix, summarised in profiles/matvec_rows_q4_0_ffn_up_gate_7b.md (not re-measured by this run)" if dom["bytes"] == 50724864 else None,
                "timing": "CUDA events on the launching stream around 320 back-to-back launches (10 sweeps over the 32 layers' matrices, 1.6 GB per sweep)",
                "bytes_per_launch": dom["bytes"], "us_per_launch": dom["us"], "kernels": kb}

    if rank == 0:
        weight_b, kv_b = info.weight_bytes, info.kv_bytes_per_token
        p_avg = N_PROMPT + warmup + (steps - 1) / 2.0
        bytes_per_token = weight_b + kv_b * p_avg + kv_b           # weights once + KV read + KV written, on this GPU
        tok_s = steps / (ms_dev / 1e3)
        peak, peak_kind = measured_peak()
        line = {"metric": "decode tokens/s", "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup,
                "ms_per_step": ms_dev / steps, "ms_per_step_reps": {"min": min(reps_ms) / steps, "median": ms_dev / steps, "max": max(reps_ms) / steps, "n": REPS},
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "int8 block dots, f32 accumulate", "data": "synthetic",
                "config": {"workload": WORKLOAD, "parallelism": f"tp{world}", "tp_exchange": None if world == 1 else ("all-gather by NCCL" if os.environ.get("SPYB_TP_NCCL_ONLY") else "all-gather fused into the kernels over peer memory"), "l2": "weights 3.7 GB per step, far larger than the 126 MB L2",
                           "pdl": not args.no_pdl, "cuda_graph": not args.no_graph},
                "hbm_gbs_per_gpu": bytes_per_token * tok_s / 1e9, "hbm_frac_of_peak": bytes_per_token * tok_s / 1e9 / peak,
                "hbm_peak_gbs": peak, "bytes_per_token_per_gpu": bytes_per_token,
                "e2e": {"value": steps / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": int(info.n_vocab) * 4,
                        "device_ms_per_step": ev_ms / steps},
                "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "prefill": prefill,
                "ids_match_e2e": bool(np.array_equal(ids, np.array(e2e_ids)))}
        if batch_rec is not None:
            line["batch"] = batch_rec
        if parity_tp is not None:
            line["parity_tp"] = parity_tp
        if not args.no_cpu_baseline and world == 1:
            # the reference's CPU backend on the whole parity sequence (8-token prompt, 32 greedy tokens, logits of every
            # step): its decode steps are the timed CPU baseline, its ids and logits the parity record
            threads = physical_cores()
            r = cpu_reference_run(path, N_PARITY - 2, 1, threads, want_logits=True, n_vocab=int(info.n_vocab))
            if r is not None:
                g_first = model.eval(prompt, 0)
                g_ids, g_logits = model.decode(int(np.argmax(g_first)), N_PROMPT, N_PARITY - 1, want_logits=True)
                g_ids = np.concatenate([[int(np.argmax(g_first))], g_ids])
                g_logits = np.concatenate([g_first[None, :], g_logits])
                line["parity"] = parity_record(g_ids, g_logits, r["ids"], r["logits"])
                line["parity"]["against"] = f"the reference's CPU backend (-t {threads}) on the same GGUF and prompt: prompt step + {N_PARITY - 1} decode steps"
                line["cpu_baseline"] = {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": threads, "kind": "reference",
                                        "sample": f"{N_PARITY - 2} decode steps after the 8-token prefill and 1 warm-up step, -t {threads}",
                                        "prefill_ms": r["prefill_ms"], "greedy_ids_identical": line["parity"]["ids_identical"]}
                line["vs_cpu_reference"] = {"value": tok_s / r["tokens_per_s"], "e2e": line["e2e"]["value"] / r["tokens_per_s"],
                                            "note": f"tokens/s over the reference's CPU backend at -t {threads} (physical cores of this box) in the same job"}
                # the prompt path: the reference CPU backend evaluates the same long prompt once (its logits after the prompt)
                try:
                    from oracle import spy_ref
                    p_ids, p_logits, p_ms = spy_ref.generate(path, pre_ids, 1, n_ctx=N_CTX, threads=threads, warmup=False, want_logits=True, n_vocab=int(info.n_vocab))
                    line["prefill"]["parity"] = parity_record([int(np.argmax(pre_logits))], pre_logits[None, :], p_ids[:1], np.asarray(p_logits)[:1])
                    line["prefill"]["cpu_reference_tokens_per_s"] = float(n_pre / (float(p_ms[0]) / 1e3))
                except Exception as e:  # noqa: BLE001
                    line["prefill"]["parity"] = {"error": str(e)[:200]}
            else:
                line["cpu_baseline"] = None
            # the reference's own token loop (scheduler, graph, sampler) on this library through the spy::Backend adapter
            try:
                from oracle import spy_ref
                if spy_ref.b200_available():
                    model.close(); be.close(); closed = True   # the adapter creates its own backend and uploads the weights itself
                    a_ids, _, a_ms = spy_ref.generate(path, prompt, 12, n_ctx=N_CTX, want_logits=False, device_backend=True)
                    line["adapter_e2e"] = {"value": float(10 / (a_ms[2:].sum() / 1e3)), "unit": "tokens/s",
                                           "sample": "10 decode steps of the reference's generate loop on backend gpu:b200 (operator-by-operator submit)",
                                           "ids_identical_to_cpu": bool(r is not None and np.array_equal(a_ids, r["ids"][:12]))}
                    p_ids, _, p_ms = spy_ref.generate(path, prompt, 34, n_ctx=N_CTX, want_logits=False, device_backend=True, plan=True)
                    line["adapter_plan_e2e"] = {"value": float(32 / (p_ms[2:].sum() / 1e3)), "unit": "tokens/s",
                                                "sample": "32 decode steps of the reference's generate loop on backend gpu:b200 in plan mode (its scheduler walks the graph, the steps run on the fused step plan)",
                                                "ids_identical_to_cpu": bool(r is not None and np.array_equal(p_ids[:32], r["ids"][:32]))}
            except Exception as e:   # the adapter build is optional
                line["adapter_e2e"] = {"unavailable": str(e)[:200]}
        print(json.dumps(line))
    if not closed:
        model.close()
        be.close()
    if dist is not None:
        dist.destroy_process_group()


def bench_kernels(model, be):
    """Each mat-vec kind launched alone, back to back over all layers (weights come from HBM each time)."""
    import ctypes as C
    l = be._l
    out = {}
    for kind, name in enumerate(["qkv", "attn_out", "ffn_up_gate", "ffn_down", "head"]):
        nbytes = C.c_uint64()
        l.spyb_model_bench_kernel(model.h, kind, 2, C.byref(nbytes))          # warm
        us = l.spyb_model_bench_kernel(model.h, kind, 10, C.byref(nbytes)) * 1e3
        if us > 0:
            out[name] = {"us": us, "bytes": int(nbytes.value), "gbs": nbytes.value / us / 1e3}
    return out


if __name__ == "__main__":
    main()
