"""Arithmetic of bench.py that the reported numbers rest on (no GPU needed): dense FLOPs per token
of the workloads, the reference-arm sample scaling, and the lines printed without a GPU."""
import importlib.util
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_mod", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_flops_per_token_match_the_hand_computed_figures():
    b = load_bench()
    # forward GFLOP per token = L (F_blk + F_attn) + F_head; checkpointed step = L 4 (F_blk + F_attn) + 3 F_head
    expect = {"c1": (0.0034, 0.0126), "c2": (0.266, 0.987), "c4": (2.346, 9.25)}
    for name, (fwd, step) in expect.items():
        w = b.WORKLOADS[name]
        f_blk, f_attn, f_head = b.flops_per_token(w)
        fwd_gf = (w["layers"] * (f_blk + f_attn) + f_head) / 1e9
        step_gf = b.step_flops_per_token(w) / 1e9
        assert abs(fwd_gf - fwd) <= 0.01 * fwd + 1e-4, (name, fwd_gf)
        assert abs(step_gf - step) <= 0.01 * step + 1e-4, (name, step_gf)


def test_reference_sample_scaling_is_a_flop_ratio():
    b = load_bench()
    w = dict(b.WORKLOADS["c4"])
    sw = dict(w)
    sw["layers"] = b.SAMPLE_LAYERS
    sw["seq"] = 32
    ratio = b.step_flops_per_token(sw) / b.step_flops_per_token(w)
    assert 0.1 < ratio < 0.2   # 2 of 16 blocks + the full head


def test_block_workload_reference_arm_says_unavailable():
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "c5"],
                         capture_output=True, text=True, timeout=120)
    assert res.returncode == 0
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line
