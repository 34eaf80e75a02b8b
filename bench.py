#!/usr/bin/env python
"""Benchmark of the activation-checkpointed transformer training step.

    python bench.py --gpus N --steps K --warmup W [--workload c4] [--impl reference]

One "step" = zero_grad + forward + cross entropy + backward with per-block recompute +
(N > 1: fp32 gradient all-reduce overlapped with the backward) + AdamW, on one batch of
synthetic token ids. Prints ONE JSON line (rank 0). Workloads:
  c1  tiny Llama fp32 (4 layers, d 128, batch 8 x 256)            -- the CPU-parity case
  c2  GPT-2-small shape, bf16, batch 16 x 1024
  c3  Qwen2.5-0.5B-shape QLoRA (Q8_0 frozen base, LoRA r=16), bf16, batch 8 x 2048
  c4  Llama-1B shape, bf16, global batch 64 x 4096 (default; sharded by batch over N GPUs)
  c5  one checkpointed Llama block (d 2048, 16 heads of 128, SwiGLU 5632), bf16, batch 4, --seq S:
      a step = the recompute + backward of the block (its forward runs untimed before it)
Keys of the JSON line: metric/value (tokens/s, whole job, inputs resident on the device),
e2e (same through the public step API with host token buffers), roofline (tcgen05 GEMM:
achieved TFLOP/s from CUDA events around every launch in the timed region), cpu_baseline
(the unmodified reference's CPU path on a bounded sample, rank 0 at N=1), clocks, peak
activation memory with and without checkpointing (reported in `config`).

`--impl reference` times the reference's own CPU implementation (oracle/_ref/ref_harness,
built by oracle/Makefile from the reference's sources) on a bounded sample of the same
workload and prints the same line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SAMPLE_LAYERS = 2  # depth of the CPU baseline sample (see run_reference)

WORKLOADS = {
    "c1": dict(family="llama", dtype="fp32", vocab=4096, d=128, layers=4, heads=4, kv_heads=0, dff=512, nctx=256,
               theta=10000.0, rope_all=0, qlora=0, batch=8, seq=256,
               name="tiny Llama fp32 (4L d128 H4 dff512 V4096), batch 8 x 256"),
    "c2": dict(family="gpt2", dtype="bf16", vocab=50257, d=768, layers=12, heads=12, nctx=1024, batch=16, seq=1024,
               name="GPT-2-small shape (12L d768 H12 dff3072 V50257), bf16, batch 16 x 1024"),
    "c3": dict(family="llama", dtype="bf16", vocab=151936, d=896, layers=24, heads=14, kv_heads=2, dff=4864,
               nctx=2048, theta=1e6, rope_all=1, qlora=1, rank=16, alpha=32, batch=8, seq=2048,
               name="Qwen2.5-0.5B-shape QLoRA (24L d896 Hq14/Hkv2 dff4864 V151936, Q8_0 base, LoRA r16 q/v), "
                    "bf16, batch 8 x 2048"),
    "c4": dict(family="llama", dtype="bf16", vocab=32000, d=2048, layers=16, heads=32, kv_heads=8, dff=8192,
               nctx=4096, theta=500000.0, rope_all=1, qlora=0, batch=64, seq=4096,
               name="Llama-1B shape (16L d2048 Hq32/Hkv8 dff8192 V32000), bf16 + fp32 master/AdamW, "
                    "global batch 64 x 4096"),
    "c5": dict(family="block", dtype="bf16", d=2048, heads=16, kv_heads=16, dff=5632, theta=10000.0, batch=4, seq=4096,
               layers=1, vocab=0,
               name="one checkpointed Llama block (d2048, 16 heads of 128, dff5632), bf16, batch 4: recompute + backward"),
}


def model_spec(w, ckpt):
    if w["family"] == "gpt2":
        return dict(family="gpt2", vocab=w["vocab"], d=w["d"], layers=w["layers"], heads=w["heads"], nctx=w["nctx"],
                    seed=0, ckpt=int(ckpt))
    s = dict(family="llama", vocab=w["vocab"], d=w["d"], layers=w["layers"], heads=w["heads"],
             kv_heads=w["kv_heads"], dff=w["dff"], nctx=w["nctx"], theta=w["theta"], rope_all=w["rope_all"], tie=1,
             seed=0, ckpt=int(ckpt))
    if w.get("qlora"):
        s.update(qlora=1, rank=w["rank"], alpha=w["alpha"])
    return s


def flops_per_token(w):
    """Algorithmic dense FLOPs per token: forward block, attention (causal average), head."""
    d, L, V, S = w["d"], w["layers"], w["vocab"], w["seq"]
    H = w["heads"]
    Hkv = w.get("kv_heads") or H
    dk = d // H
    dq, dkv = H * dk, Hkv * dk
    if w["family"] == "gpt2":
        f_blk = 2 * (d * 3 * d + d * d + 2 * d * 4 * d)
    else:
        f_blk = 2 * (d * dq + 2 * d * dkv + dq * d + 3 * d * w["dff"])
    f_attn = 4 * (S / 2) * dq
    f_head = 2 * d * V
    return f_blk, f_attn, f_head


def last_projection_flops(w):
    """FLOPs per token of a block's last projection (down / c_proj). Its value is dead when the
    block is re-run for the backward pass, so the recompute does not execute it."""
    d = w["d"]
    return 2 * d * (4 * d if w["family"] == "gpt2" else w["dff"])


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        # the first samples precede the load; the median over the region is what counts
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def ref_harness_args(w, sample_tokens):
    fam = {"gpt2": "gpt2"}.get(w["family"], "llama")
    a = {"family": fam, "vocab": w["vocab"], "d": w["d"], "layers": w["layers"], "heads": w["heads"],
         "batch": 1, "seq": sample_tokens, "seed": 0, "data-seed": 0, "ckpt": 1, "adamw": 1}
    if fam == "gpt2":
        a["nctx"] = w["nctx"]
    else:
        a["dff"] = w["dff"]
        a["theta"] = w["theta"]
        if w.get("qlora"):
            a.update(family="qlora", rank=w["rank"], alpha=w["alpha"])
            a["kv-heads"] = w["kv_heads"]
        elif w.get("kv_heads"):
            a["family"] = "llamagqa"
            a["kv-heads"] = w["kv_heads"]
    return a


def step_flops_per_token(w):
    """Dense FLOPs one checkpointed training step of the reference executes per token (forward +
    full recompute + backward); used to scale the reference's timed sample to the full model."""
    f_blk, f_attn, f_head = flops_per_token(w)
    return w["layers"] * 4 * (f_blk + f_attn) + 3 * f_head


def run_reference(w, steps, warmup, sample_tokens):
    """Times the unmodified reference's CPU path on a bounded sample of the workload: one sequence of
    `sample_tokens` tokens through the first SAMPLE_LAYERS blocks (+ embedding, final norm, head, AdamW)
    of the same model. Its tokens/s is scaled to the full model by the ratio of dense FLOPs per token
    (a full-depth step of even 16 tokens costs the reference minutes: its per-step weight transposes
    and serial AdamW over 1.2 G parameters do not shrink with the token count)."""
    harness = ROOT / "oracle" / "_ref" / "ref_harness"
    if not harness.exists():
        return None, f"{harness} missing (built by `make -C oracle` from the reference's sources)"
    sw = dict(w)
    sw["layers"] = min(w["layers"], SAMPLE_LAYERS)
    sw["seq"] = sample_tokens
    args = ref_harness_args(sw, sample_tokens)
    argv = [str(harness), "bench"]
    for k, v in args.items():
        argv += [f"--{k}", str(v)]
    argv += ["--steps", str(steps + warmup), "--warmup", str(warmup)]
    t0 = time.time()
    res = subprocess.run(argv, capture_output=True, text=True)
    if res.returncode != 0:
        return None, f"reference harness failed: {res.stderr[-300:]}"
    line = [l for l in res.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    out["wall_s_total"] = time.time() - t0
    ratio = step_flops_per_token(sw) / step_flops_per_token(w)
    out["tokens_per_s_sample"] = out["tokens_per_s"]
    out["tokens_per_s"] = out["tokens_per_s"] * ratio
    out["sample"] = (f"{steps} timed step(s) of {sample_tokens} tokens (1 sequence) through {sw['layers']} of the "
                     f"{w['layers']} blocks + embedding, head and AdamW of the same model on the reference's CPU fp32 "
                     f"path with per-block checkpointing: {out['tokens_per_s_sample']:.3f} tokens/s measured, scaled by "
                     f"{ratio:.4f} (dense FLOPs per token, sample model / full model at seq {w['seq']})")
    return out, None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=os.environ.get("PK_BENCH_WORKLOAD", "c4"), choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="override the global batch (sequences)")
    ap.add_argument("--layers", type=int, default=0, help="override the number of blocks (small profiling cases)")
    ap.add_argument("--seq", type=int, default=0, help="override the sequence length (c5 sweep)")
    ap.add_argument("--accum", type=int, default=0,
                    help="micro-batches per step (gradient accumulation; exchange on the last one only); "
                         "0 = micro-batches of at most 65536 tokens per GPU")
    ap.add_argument("--comm", default="pk", choices=["pk", "torch"],
                    help="gradient exchange at N > 1: inside the library over libpk's collective group (pk, default) "
                         "or torch.distributed all-reduces from the Python segment hook (torch)")
    ap.add_argument("--nccl-max-ctas", type=int, default=int(os.environ.get("PK_NCCL_MAX_CTAS", "0")),
                    help="--comm pk: cap on the CTAs NCCL's kernels take from the kernels they overlap (0: NCCL's default)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-sample-tokens", type=int, default=0)
    ap.add_argument("--skip-nockpt", action="store_true", help="do not measure the un-checkpointed step")
    args = ap.parse_args()

    w = dict(WORKLOADS[args.workload])
    if args.batch:
        w["batch"] = args.batch
    if args.seq:
        w["seq"] = args.seq
        w["name"] += f" [seq {args.seq}]"
    if args.layers:
        w["layers"] = args.layers
        w["name"] += f" [reduced to {args.layers} block(s)]"
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    sample_tokens = args.cpu_sample_tokens or {"c1": 2048, "c2": 64, "c3": 32, "c4": 32, "c5": 32}[args.workload]
    if args.workload == "c1":
        sample_tokens = 256  # per sequence; the harness batches 8 of them below

    base = {"metric": "train tokens/s with per-block activation recompute", "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": f"{args.workload}: {w['name']}", "global_batch": w["batch"], "seq_len": w["seq"],
                       "parallelism": f"dp{args.gpus}", "l2": "inputs and activations exceed L2 (126 MB)"}}

    # ------------------------------------------------------------------ reference arm
    if args.impl == "reference":
        if rank != 0:
            return 0
        if args.workload == "c5":
            print(json.dumps({"impl": "reference", "unavailable": "the reference harness has no single-block mode; "
                              "c5 is checked against a PyTorch fp32 restatement in tests/test_block_gpu.py"}))
            return 0
        if args.workload == "c1":
            # bounded: at most 3 full-size steps (each ~20 s of CPU work)
            out, err = run_reference_c1(w, min(args.steps, 3), min(max(args.warmup, 0), 1))
        else:
            out, err = run_reference(w, min(args.steps, 3), min(max(args.warmup, 0), 1), sample_tokens)
        if out is None:
            print(json.dumps({"impl": "reference", "unavailable": err}))
            return 0
        line = dict(base)
        # the CPU arm is bounded: it never times more than 3 steps after at most 1 warm-up step
        line.update({"steps": min(args.steps, 3), "warmup": min(max(args.warmup, 0), 1)})
        line.update({"impl": "reference", "value": out["tokens_per_s"], "ms_per_step": out["step_s"] * 1e3,
                     "dtype": "f32", "gpu_launches": 0,
                     "cpu_baseline": {"value": out["tokens_per_s"], "unit": "tokens/s", "cores": 1, "kind": "reference",
                                      "sample": out["sample"], "host_threads": os.cpu_count(),
                                      "note": "the reference's GEMM (~95% of its step) is single-threaded by "
                                              "construction; OpenMP covers elementwise ops only"},
                     "e2e": {"value": out["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                             "d2h_bytes_per_step": 0}})
        print(json.dumps(line))
        return 0

    # ------------------------------------------------------------------ our arm
    import numpy as np
    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU execution path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from paperkiln_b200 import model as mt
    from paperkiln_b200._capi import libpk

    pk = libpk()
    mt.init(local_rank, mt.BF16 if w["dtype"] == "bf16" else mt.FP32)
    # One explicit (non-default) stream carries everything: the library's kernels, the CUDA events of
    # the timed regions, and -- as torch's current stream -- the point NCCL's all-reduces wait on
    # and are waited for. (Handing the library the default stream's null handle would make it fall
    # back to a private non-blocking stream that nothing else is ordered against.)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    mt.set_stream(stream.cuda_stream)
    if w["family"] == "block":
        rc = run_block(args, w, mt, pk, stream, base, world, rank, torch, np)
        if world > 1:
            dist.destroy_process_group()
        return rc

    B, S = w["batch"], w["seq"]
    if B % world:
        raise SystemExit(f"global batch {B} does not divide over {world} ranks")
    Bl = B // world
    n_local = Bl * S
    tokens_global = B * S
    if args.accum <= 0:
        # One optimizer step over the global batch, run as micro-batches of at most 65536 tokens
        # per GPU whose gradients accumulate in place (the reference trainer's `accum` loop,
        # tools/mtstudio.cpp:456-474). Measured on c4 at one GPU: 4 x 16 sequences is 6.5 %
        # faster than 1 x 64 (higher sustained SM clock under the power cap, 12 GiB instead of
        # 48 GiB of activations).
        args.accum = 1
        while n_local // args.accum > 65536 and Bl % (args.accum * 2) == 0:
            args.accum *= 2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # synthetic token stream: ids = rng % vocab, targets = ids shifted by one; rank r takes
    # sequences [r*B/g, (r+1)*B/g) of every global batch
    n_batches = args.warmup + args.steps + 1
    rng = np.random.RandomState(1234)
    host_ids, host_tg = [], []
    for _ in range(n_batches):
        stream_ids = rng.randint(0, w["vocab"], size=tokens_global + 1).astype(np.int32)
        lo = rank * n_local
        ids = torch.from_numpy(stream_ids[lo:lo + n_local].copy()).pin_memory()
        tg = torch.from_numpy(stream_ids[lo + 1:lo + n_local + 1].copy()).pin_memory()
        host_ids.append(ids)
        host_tg.append(tg)

    def build(ckpt):
        m = mt.Model(**model_spec(w, ckpt))
        m.set_adamw()
        return m

    class _Buf:
        def __init__(self, ptr, n):
            self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}

    def make_step(m):
        reducer = None
        in_library = world > 1 and args.comm == "pk"
        if in_library:
            # The exchange runs inside the library: each block's gradient range is all-reduced over
            # libpk's collective group (NCCL) as that block's backward is enqueued. Rank 0 draws the
            # communicator id; it travels over the launcher's process group.
            idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
            if rank == 0:
                idt.copy_(torch.frombuffer(bytearray(mt.Model.dp_unique_id()), dtype=torch.uint8))
            dist.broadcast(idt, 0)
            m.dp_init(idt.cpu().numpy().tobytes(), rank, world, args.nccl_max_ctas)
        elif world > 1:
            from paperkiln_b200.dp import BucketAllReducer
            # block i's gradients are one contiguous fp32 range of the flat gradient buffer
            reducer = BucketAllReducer([torch.as_tensor(_Buf(p, n), device="cuda") for (p, n) in m.buckets()])
            mt.set_segment_hook(reducer.on_segment)  # fires as each block's backward is enqueued

        accum = args.accum
        if Bl % accum:
            raise SystemExit(f"{Bl} sequences per rank do not divide into {accum} micro-batches")
        n_micro = n_local // accum
        m.set_accumulate(accum > 1)

        def step(i):
            if accum == 1:
                loss = m.step_ptr(host_ids[i].data_ptr(), host_tg[i].data_ptr(), n_local, S, loss_scale=1.0 / world)
            else:
                # micro-batches of Bl/accum sequences; gradients add up in place and are
                # exchanged during the backward of the last micro-batch only
                m.zero_grad()
                loss = 0.0
                for k in range(accum):
                    if in_library:
                        m.dp_enable(k == accum - 1)
                    if reducer is not None:
                        reducer.enabled = k == accum - 1
                    off = k * n_micro * 4
                    loss += m.step_ptr(host_ids[i].data_ptr() + off, host_tg[i].data_ptr() + off, n_micro, S,
                                       loss_scale=1.0 / (world * accum)) / accum
            if in_library:
                m.dp_finish()     # remaining ranges, then the compute stream waits for all transfers
            if reducer is not None:
                reducer.finish()  # remaining buckets, then wait for all of them
            m.optimizer_step()
            return loss
        return step

    def timed(step_fn, indices):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        loss = None
        for i in indices:
            loss = step_fn(i)
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, loss

    # ---- checkpointed model: warm-up, then the two timed regions
    m = build(ckpt=True)
    step_fn = make_step(m)
    for i in range(args.warmup):
        step_fn(i)
    barrier()
    mt.reset_peak()
    # (1) e2e: a fresh host batch every step (H2D of ids and targets inside the region, loss read back)
    sampler = ClockSampler(local_rank)
    sampler.start()
    pk.pk_prof_reset()
    pk.pk_prof_enable(1)
    e2e_ms, loss = timed(step_fn, range(args.warmup, args.warmup + args.steps))
    pk.pk_prof_enable(0)
    clocks = sampler.stop()
    peak_ckpt = mt.mem_stats()["activation_peak"]
    peak_live = {f"{sz / 2 ** 20:.1f} MiB": n for sz, n in mt.peak_blocks().items() if sz * n >= (8 << 20)}
    import ctypes
    prof = {}
    for kind, name in ((0, "gemm_tc"), (1, "gemm_simt"), (2, "attn_fwd"), (3, "attn_bwd")):
        ms_, work_, n_ = ctypes.c_double(0), ctypes.c_double(0), ctypes.c_int64(0)
        pk.pk_prof_summary(kind, ctypes.byref(ms_), ctypes.byref(work_), ctypes.byref(n_))
        prof[name] = {"ms": ms_.value, "flops": work_.value, "launches": n_.value}
    # (2) value: the same batch every step -- its ids/targets are already on the device
    # (the library caches uploaded index arrays by content), so no input crosses PCIe
    last = args.warmup + args.steps
    step_fn(last)
    res_ms, _ = timed(step_fn, [last] * args.steps)
    stats = mt.mem_stats()
    m.close()
    mt.set_segment_hook(None)

    # ---- the same step without checkpointing, for the activation-memory comparison
    peak_plain, plain_ms = None, None
    if not args.skip_nockpt:
        try:
            mt.empty_cache()
            m2 = build(ckpt=False)
            step2 = make_step(m2)
            step2(0)
            barrier()
            mt.reset_peak()
            plain_ms, _ = timed(step2, [1, 2])
            plain_ms /= 2
            peak_plain = mt.mem_stats()["activation_peak"]
            m2.close()
            mt.set_segment_hook(None)
        except Exception as e:  # does not fit without checkpointing at this size
            peak_plain = f"unavailable: {str(e)[:120]}"
            mt.empty_cache()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak_tf = peaks.get("bf16_tflops_sustained", 1400.0)
    peak_src = "measured (MEASURED_PEAKS.json, sustained cuBLAS bf16)" if peaks else "fallback 1.4 PFLOP/s"
    g = prof["gemm_tc"]
    achieved = g["flops"] / (g["ms"] * 1e-3) / 1e12 if g["ms"] > 0 else 0.0
    f_blk, f_attn, f_head = flops_per_token(w)
    L = w["layers"]
    if w.get("qlora"):
        # frozen base: the weight-gradient GEMMs of the projections and of the (tied, frozen) head are
        # not executed -- forward + recompute + input gradient for a block, forward + input gradient
        # for the head; attention is as for a dense model. (The rank-16 LoRA products are left out.)
        step_flops = (L * (3 * f_blk + 4 * f_attn - last_projection_flops(w)) + 2 * f_head) * tokens_global
        model_flops = (L * (2 * f_blk + 3 * f_attn) + 2 * f_head) * tokens_global
    else:
        step_flops = (L * (4 * (f_blk + f_attn) - last_projection_flops(w)) + 3 * f_head) * tokens_global
        model_flops = 3 * (L * (f_blk + f_attn) + f_head) * tokens_global
    launches = sum(p["launches"] for p in prof.values())
    # DRAM bytes of one launch of the dominant GEMM shape (the down projection, M x d x dff):
    # dram__bytes_read + dram__bytes_write of an ncu capture at M = 16384 (575.3 + 60.0 MB for
    # d 2048, dff 8192), scaled to this run's rows per GPU -- traffic grows in proportion to M.
    traffic, traffic_note = None, None
    if args.workload == "c4":
        traffic = 635.3e6 * (n_local / max(1, args.accum) / 16384.0)
        traffic_note = ("down projection launch (rows x 2048 x 8192): ncu capture at 16384 rows scaled by rows; "
                        "algorithmic bytes of that launch are 369 MB per 16384 rows (the A operand is read about "
                        "twice: a row block's 8192-deep slab does not stay in L2 between its tiles; tensor pipe 90 % busy)")
    line = dict(base)
    line["value"] = tokens_global / (res_ms / args.steps * 1e-3)
    line["ms_per_step"] = res_ms / args.steps
    line["e2e"] = {"value": tokens_global / (e2e_ms / args.steps * 1e-3), "unit": "tokens/s",
                   "h2d_bytes_per_step": 2 * n_local * 4 * world, "d2h_bytes_per_step": 4 * world * max(1, args.accum),
                   "ms_per_step": e2e_ms / args.steps}
    if args.accum > 1:
        line["config"] = dict(line["config"], micro_batches_per_step=args.accum)
    line["loss"] = loss
    line["clocks"] = clocks
    line["gpu_launches"] = int(launches)
    line["roofline"] = {"bound": "tensor", "kernel": ("gemm_q8_kernel (tcgen05 Q8_0 dequantise-GEMM + LoRA) / gemm_tc2_kernel" if w.get("qlora") else
                                   "gemm_tc2_kernel / gemm_tc_kernel (tcgen05 bf16 GEMM; CTA pairs where the tiles suffice)"), "achieved": achieved,
                        "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf if peak_tf else None,
                        "peak_source": peak_src, "traffic": traffic, "traffic_note": traffic_note,
                        "share_of_step": g["ms"] / e2e_ms if e2e_ms else None, "launches_timed": g["launches"]}
    line["kernels"] = {k: {"ms_per_step": v["ms"] / args.steps,
                           "tflops": (v["flops"] / (v["ms"] * 1e-3) / 1e12) if v["ms"] > 0 else None,
                           "launches_per_step": v["launches"] / args.steps} for k, v in prof.items()}
    line["step_tflops_executed"] = step_flops / (res_ms / args.steps * 1e-3) / 1e12 / args.gpus
    line["mfu_model_flops"] = model_flops / (res_ms / args.steps * 1e-3) / 1e12 / args.gpus / (peaks.get("bf16_tflops", 1676.5))
    line["config"].update({
        "peak_activation_gib_checkpointed": peak_ckpt / 2 ** 30,
        "peak_activation_live_blocks": peak_live,
        "peak_activation_gib_plain": (peak_plain / 2 ** 30) if isinstance(peak_plain, int) else peak_plain,
        "ms_per_step_plain": plain_ms,
        "persistent_gib": stats["persistent_peak"] / 2 ** 30,
    })
    if not args.no_cpu_baseline and world == 1:
        hw = dict(w)
        if args.workload == "c1":
            out, err = run_reference_c1(hw)
        else:
            out, err = run_reference(hw, 1, 0, sample_tokens)
        if out is not None:
            line["cpu_baseline"] = {"value": out["tokens_per_s"], "unit": "tokens/s", "cores": 1, "kind": "reference",
                                    "sample": out["sample"], "host_threads": os.cpu_count()}
        else:
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 1, "kind": "reference", "sample": err}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def run_block(args, w, mt, pk, stream, base, world, rank, torch, np):
    """c5: recompute + backward of one checkpointed Llama block; inputs N(0,1), upstream gradient
    N(0, 1e-3), weights N(0, 0.02) from the library's seeds. Every rank runs an independent replica."""
    import ctypes
    B, S, d, H, F = w["batch"], w["seq"], w["d"], w["heads"], w["dff"]
    R = B * S
    rng = np.random.RandomState(99 + rank)
    x = rng.randn(R, d).astype(np.float32)
    dy = (rng.randn(R, d) * 1e-3).astype(np.float32)
    m = mt.Model(family="block", d=d, heads=H, kv_heads=w["kv_heads"], dff=F, theta=w["theta"], rope_all=1, seed=0, ckpt=1)
    m.block_set_input(x, dy, S)
    for _ in range(args.warmup):
        m.block_forward()
        m.block_backward()
    torch.cuda.synchronize()
    mt.reset_peak()
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
    bwd_ms, fwd_ms = 0.0, 0.0
    prof_total = {}
    for _ in range(args.steps):
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record(stream)
        m.block_forward()
        e1.record(stream)
        pk.pk_prof_reset()
        pk.pk_prof_enable(1)
        m.block_backward()
        pk.pk_prof_enable(0)
        e2.record(stream)
        torch.cuda.synchronize()
        fwd_ms += e0.elapsed_time(e1)
        bwd_ms += e1.elapsed_time(e2)
        for kind, name in ((0, "gemm_tc"), (1, "gemm_simt"), (2, "attn_fwd"), (3, "attn_bwd")):
            ms_, work_, n_ = ctypes.c_double(0), ctypes.c_double(0), ctypes.c_int64(0)
            pk.pk_prof_summary(kind, ctypes.byref(ms_), ctypes.byref(work_), ctypes.byref(n_))
            t = prof_total.setdefault(name, [0.0, 0.0, 0])
            t[0] += ms_.value
            t[1] += work_.value
            t[2] += n_.value
    clocks = sampler.stop()
    # e2e: host arrays in, block output gradient out, every step
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record(stream)
    for _ in range(args.steps):
        m.block_set_input(x, dy, S)
        m.block_forward()
        m.block_backward()
        dx = m.block_input_grad()
    t1.record(stream)
    torch.cuda.synchronize()
    e2e_ms = t0.elapsed_time(t1) / args.steps
    peak = mt.mem_stats()["activation_peak"]
    m.close()
    if rank != 0:
        return 0
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak_tf = peaks.get("bf16_tflops", 1676.5)
    step_ms = bwd_ms / args.steps
    dk = d // H
    f_blk = 2 * (4 * d * d + 3 * d * F)
    f_attn = 4 * (S / 2) * d
    flops = (3 * (f_blk + f_attn) - 2 * F * d) * R   # recompute (1x, without the dead last projection) + backward (2x)
    g = prof_total["gemm_tc"]
    line = dict(base)
    line["metric"] = "tokens/s through recompute + backward of one checkpointed block"
    line["scaling"] = "weak"
    line["value"] = R * world / (step_ms * 1e-3)
    line["ms_per_step"] = step_ms
    line["e2e"] = {"value": R * world / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * R * d * 4 * world,
                   "d2h_bytes_per_step": R * d * 4 * world, "ms_per_step": e2e_ms,
                   "note": "block_set_input (host fp32 x and dy) + forward + backward + input gradient read back"}
    line["clocks"] = clocks
    line["gpu_launches"] = int(sum(t[2] for t in prof_total.values()))
    achieved = g[1] / (g[0] * 1e-3) / 1e12 if g[0] > 0 else 0.0
    line["roofline"] = {"bound": "tensor", "kernel": ("gemm_q8_kernel (tcgen05 Q8_0 dequantise-GEMM + LoRA) / gemm_tc2_kernel" if w.get("qlora") else
                                   "gemm_tc2_kernel / gemm_tc_kernel (tcgen05 bf16 GEMM; CTA pairs where the tiles suffice)"), "achieved": achieved, "peak": peak_tf,
                        "unit": "TFLOP/s", "frac": achieved / peak_tf, "peak_source": "measured (MEASURED_PEAKS.json, burst cuBLAS bf16: "
                        "the block is timed alone)" if peaks else "fallback", "traffic": None,
                        "share_of_step": g[0] / bwd_ms if bwd_ms else None}
    line["kernels"] = {k: {"ms_per_step": v[0] / args.steps, "tflops": (v[1] / (v[0] * 1e-3) / 1e12) if v[0] > 0 else None,
                           "frac_of_peak": (v[1] / (v[0] * 1e-3) / 1e12 / peak_tf) if v[0] > 0 else None,
                           "launches_per_step": v[2] / args.steps} for k, v in prof_total.items()}
    line["step_tflops_executed"] = flops / (step_ms * 1e-3) / 1e12
    line["config"].update({"forward_ms_untimed": fwd_ms / args.steps, "peak_activation_gib_checkpointed": peak / 2 ** 30,
                           "head_dim": dk})
    print(json.dumps(line))
    return 0


def run_reference_c1(w, steps=1, warmup=0):
    """Config 1 is the reference's own CPU-runnable case: full-size steps (8 x 256 tokens)."""
    harness = ROOT / "oracle" / "_ref" / "ref_harness"
    if not harness.exists():
        return None, f"{harness} missing (built by `make -C oracle` from the reference's sources)"
    argv = [str(harness), "bench", "--family", "llama", "--vocab", "4096", "--d", "128", "--layers", "4", "--heads", "4",
            "--dff", "512", "--nctx", "256", "--batch", "8", "--seq", "256", "--ckpt", "1",
            "--steps", str(steps + warmup), "--warmup", str(warmup)]
    res = subprocess.run(argv, capture_output=True, text=True)
    if res.returncode != 0:
        return None, res.stderr[-300:]
    out = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    out["sample"] = f"{steps} full-size step(s) (8 x 256 tokens), reference CPU fp32 path with checkpointing + AdamW"
    return out, None


if __name__ == "__main__":
    sys.exit(main())
