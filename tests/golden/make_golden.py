"""Generates the golden fixtures in this directory by running the UNMODIFIED reference
(paperkiln CPU fp32 path, compiled by oracle/Makefile into oracle/_ref/ref_harness).

    make -C oracle            # needs the reference checkout, see oracle/Makefile
    python tests/golden/make_golden.py

Each fixture is a compressed .npz with the parameters the reference started from, the
token ids / targets, the loss, every parameter gradient, the parameters after one
AdamW step and (config 1) summary statistics of the full-size run. The tests never run
this script; they read the committed files.
"""
import json
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
HARNESS = ROOT / "oracle" / "_ref" / "ref_harness"

# name -> harness arguments. Small shapes in the spirit of the reference's own tests
# (tests/test_checkpointing.cpp:93-124: d=32, 4 layers, 4 heads, T=16, vocab 97).
STEP_CASES = {
    "llama_tiny_ckpt": dict(family="llama", vocab=97, d=32, layers=4, heads=4, dff=64, nctx=64, batch=2, seq=16,
                            seed=9, **{"data-seed": 77}, ckpt=1),
    "llama_tiny_plain": dict(family="llama", vocab=97, d=32, layers=4, heads=4, dff=64, nctx=64, batch=2, seq=16,
                             seed=9, **{"data-seed": 77}, ckpt=0),
    "llama_untied": dict(family="llama", vocab=61, d=64, layers=2, heads=2, dff=96, nctx=64, batch=3, seq=20,
                         seed=3, **{"data-seed": 5}, ckpt=1, tie=0),
    "gpt2_tiny_ckpt": dict(family="gpt2", vocab=97, d=32, layers=4, heads=4, nctx=64, batch=2, seq=16, seed=9,
                           **{"data-seed": 77}, ckpt=1),
    "flex_ln_gelu_learned": dict(family="flex", vocab=97, d=32, layers=2, heads=4, dff=128, nctx=64, batch=2, seq=16,
                                 seed=4, **{"data-seed": 11}, ckpt=1, norm="layernorm", act="gelu", pos="learned"),
    "flex_rms_swiglu_sin": dict(family="flex", vocab=97, d=32, layers=2, heads=4, dff=64, nctx=64, batch=2, seq=16,
                                seed=4, **{"data-seed": 11}, ckpt=1, norm="rmsnorm", act="swiglu", pos="sinusoidal"),
    "flex_ln_relu": dict(family="flex", vocab=97, d=32, layers=2, heads=4, dff=64, nctx=64, batch=2, seq=16, seed=4,
                         **{"data-seed": 11}, ckpt=0, norm="layernorm", act="relu", pos="learned"),
    "llamagqa_tiny": dict(family="llamagqa", vocab=97, d=64, layers=2, heads=4, **{"kv-heads": 2}, dff=96, batch=2,
                          seq=24, seed=2, **{"data-seed": 13}, ckpt=1),
    "qlora_tiny": dict(family="qlora", vocab=97, d=64, layers=2, heads=4, **{"kv-heads": 2}, dff=96, batch=2, seq=24,
                       seed=2, **{"data-seed": 13}, ckpt=1, rank=8, alpha=16),
}

# Reduced shapes of the bf16 configurations: the model width, head layout (head_dim 64), MLP width
# and rotary base of GPT-2 small, the Qwen2.5-0.5B-shape QLoRA model and the Llama-1B shape, with
# 2 layers, 2 short sequences and a 1024-word vocabulary so that the reference's CPU path finishes
# in minutes. At these widths the GPU build runs its tcgen05 GEMM and attention kernels, which the
# tiny cases above never reach. Stored as statistics and strided samples (the parameters are
# regenerated from the seeds by the GPU build, bit for bit).
REDUCED_CASES = {
    "c2_reduced": dict(family="gpt2", vocab=1024, d=768, layers=2, heads=12, nctx=256, batch=2, seq=192, seed=21,
                       **{"data-seed": 31}, ckpt=1),
    "c3_reduced": dict(family="qlora", vocab=1024, d=896, layers=2, heads=14, **{"kv-heads": 2}, dff=4864, batch=2,
                       seq=128, seed=22, **{"data-seed": 32}, ckpt=1, rank=16, alpha=32, theta=1000000),
    "c4_reduced": dict(family="llamagqa", vocab=1024, d=2048, layers=2, heads=32, **{"kv-heads": 8}, dff=8192, batch=2,
                       seq=128, seed=23, **{"data-seed": 33}, ckpt=1, theta=500000),
}
SAMPLE = 2048


def strided_sample(v, n=SAMPLE):
    return v.reshape(-1)[::max(1, v.size // n)][:n].copy()


def tensor_stats(stats, prefix, v):
    flat = v.reshape(-1).astype(np.float64)
    stats[f"{prefix}.l2"] = np.float64(np.sqrt((flat * flat).sum()))
    stats[f"{prefix}.sum"] = np.float64(flat.sum())
    stats[f"{prefix}.sample"] = strided_sample(v)


# Eight optimizer steps on one batch with gradient clipping (the reference's own multi-step device
# pin, tests/test_step_residency.cpp:142-158, runs 8 steps): per-step losses and the final weights.
TRAIN_CASES = {
    "llama_train8": dict(family="llama", vocab=97, d=32, layers=2, heads=4, dff=64, nctx=64, batch=2, seq=16, seed=9,
                         **{"data-seed": 77}, ckpt=1, steps=8, clip=1.0, lr=0.003),
    "gpt2_train8": dict(family="gpt2", vocab=97, d=32, layers=2, heads=4, nctx=64, batch=2, seq=16, seed=9,
                        **{"data-seed": 77}, ckpt=1, steps=8, clip=1.0, lr=0.003),
}


CONFIG1 = dict(family="llama", vocab=4096, d=128, layers=4, heads=4, dff=512, nctx=256, batch=8, seq=256, seed=0,
               **{"data-seed": 0})


def run_harness(cmd, args, out_dir):
    argv = [str(HARNESS), cmd]
    for k, v in args.items():
        argv += [f"--{k}", str(v)]
    argv += ["--out", str(out_dir)]
    res = subprocess.run(argv, capture_output=True, text=True, check=True)
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    return json.loads(lines[-1]) if lines else {}


def load_dir(d: Path):
    return {p.stem: np.load(p) for p in sorted(d.glob("*.npy"))}


def main():
    if not HARNESS.exists():
        sys.exit(f"{HARNESS} not found: run `make -C oracle` first")
    for name, args in STEP_CASES.items():
        with tempfile.TemporaryDirectory() as tmp:
            info = run_harness("step", args, tmp)
            arrays = load_dir(Path(tmp))
            arrays["meta_json"] = np.frombuffer(json.dumps({"args": args, "result": info}).encode(), dtype=np.uint8)
            np.savez_compressed(HERE / f"{name}.npz", **arrays)
            print(name, info.get("loss"), f"{(HERE / (name + '.npz')).stat().st_size / 1024:.0f} KiB")
    for cmd in ("ops", "quant"):
        with tempfile.TemporaryDirectory() as tmp:
            run_harness(cmd, {}, tmp)
            np.savez_compressed(HERE / f"{cmd}.npz", **load_dir(Path(tmp)))
            print(cmd, f"{(HERE / (cmd + '.npz')).stat().st_size / 1024:.0f} KiB")
    # Config 1 at full size: keep scalars and per-parameter statistics, not 2 x 6 MB of
    # tensors. The GPU test regenerates the same parameters from the same seeds, checks
    # them against these statistics, and compares loss / gradient norms / a strided
    # sample of every gradient.
    stats = {}
    for ckpt in (0, 1):
        with tempfile.TemporaryDirectory() as tmp:
            info = run_harness("step", dict(CONFIG1, ckpt=ckpt), tmp)
            arrays = load_dir(Path(tmp))
            tag = "ckpt" if ckpt else "plain"
            stats[f"{tag}.loss"] = np.float32(info["loss"])
            stats[f"{tag}.live_after_fwd"] = np.int64(info["live_after_fwd"])
            if ckpt:
                stats["ids"] = arrays["ids"]
                stats["targets"] = arrays["targets"]
            for k, v in arrays.items():
                if k.startswith("grad.") or (ckpt and (k.startswith("param.") or k.startswith("after."))):
                    flat = v.reshape(-1).astype(np.float64)
                    stats[f"{tag}.{k}.l2"] = np.float64(np.sqrt((flat * flat).sum()))
                    stats[f"{tag}.{k}.sum"] = np.float64(flat.sum())
                    stats[f"{tag}.{k}.sample"] = v.reshape(-1)[::max(1, v.size // 512)][:512].copy()
            print("config1", tag, info)
    stats["meta_json"] = np.frombuffer(json.dumps({"args": CONFIG1}).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "config1_llama_stats.npz", **stats)
    print("config1", f"{(HERE / 'config1_llama_stats.npz').stat().st_size / 1024:.0f} KiB")
    make_reduced()
    make_train()


def make_train():
    for name, args in TRAIN_CASES.items():
        with tempfile.TemporaryDirectory() as tmp:
            info = run_harness("step", args, tmp)
            arrays = load_dir(Path(tmp))
            keep = {k: v for k, v in arrays.items() if k in ("ids", "targets", "losses") or k.startswith(("param.", "after."))}
            keep["meta_json"] = np.frombuffer(json.dumps({"args": args, "result": info}).encode(), dtype=np.uint8)
            np.savez_compressed(HERE / f"{name}.npz", **keep)
            print(name, arrays["losses"].ravel(), f"{(HERE / (name + '.npz')).stat().st_size / 1024:.0f} KiB")


def make_reduced(only=None):
    for name, args in REDUCED_CASES.items():
        if only and name not in only:
            continue
        with tempfile.TemporaryDirectory() as tmp:
            info = run_harness("step", args, tmp)
            arrays = load_dir(Path(tmp))
            stats = {"loss": np.float32(info["loss"]), "ids": arrays["ids"], "targets": arrays["targets"]}
            for k, v in arrays.items():
                if k.startswith(("grad.", "param.", "after.")):
                    tensor_stats(stats, k, v)
            stats["meta_json"] = np.frombuffer(json.dumps({"args": args, "result": info}).encode(), dtype=np.uint8)
            np.savez_compressed(HERE / f"{name}.npz", **stats)
            print(name, info, f"{(HERE / (name + '.npz')).stat().st_size / 1024:.0f} KiB")


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] in ("reduced", "train"):   # only one group of cases
        if not HARNESS.exists():
            sys.exit(f"{HARNESS} not found: run `make -C oracle` first")
        make_reduced(sys.argv[2:]) if sys.argv[1] == "reduced" else make_train()
    else:
        main()
