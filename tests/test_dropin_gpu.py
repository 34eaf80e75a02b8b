"""Drop-in proof, GPU part: the reference's own tests -- tests/test_checkpointing.cpp (checkpointed
== plain, half the live variables), test_llama.cpp (shapes, finite differences, a training run),
test_batching.cpp (stacked == per-sequence, exact isolation, accumulation), test_flex.cpp (flex
defaults == GPT-2) and test_lora_quant.cpp (block-64 quantisation bound, LoRA identity, merged
weight, QLoRA training) -- compiled unchanged against this library's headers, run on the GPU in
fp32 with MICROTORCH_DEVICE=cuda; and its python/bindings.cpp, compiled unchanged, driving a GPT-2
training step whose loss is compared with the reference's golden."""
import json
import os
import shutil
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
DROPIN = ROOT / "oracle" / "_ref" / "dropin"
GOLDEN = ROOT / "tests" / "golden"


def _env():
    env = dict(os.environ)
    env.update(MICROTORCH_DEVICE="cuda", MICROTORCH_DTYPE="fp32")
    return env


@pytest.mark.parametrize("name", ["test_checkpointing", "test_llama", "test_batching", "test_flex", "test_lora_quant"])
def test_reference_test_passes_on_the_gpu(name):
    exe = DROPIN / name
    if not exe.exists():
        pytest.skip(f"{exe} not built (needs a reference checkout at build time)")
    # line-buffered stdout: what the program printed before an uncaught exception must not be lost
    cmd = (["stdbuf", "-oL"] if shutil.which("stdbuf") else []) + [str(exe)]
    res = subprocess.run(cmd, capture_output=True, text=True, env=_env(), timeout=900)
    tail = (res.stdout[-2500:] + "\n" + res.stderr[-2500:]).strip()
    assert "CHECK failed" not in res.stderr and "FAIL" not in res.stdout, tail
    if name == "test_batching":
        # Its GPT-2 and Llama lanes are this path and must pass all five receipts each (stacked ==
        # per-sequence logits twice, loss, gradients, exact isolation). The program then moves on
        # to the reference's Kimi / surprise-routed research models, which this library declares
        # but does not provide: it must stop there, with that message, and nowhere earlier.
        lines = res.stdout.splitlines()
        assert sum(l.startswith("  [gpt2]") for l in lines) == 5, tail
        assert sum(l.startswith("  [llama]") for l in lines) == 5, tail
        assert res.returncode != 0 and "KimiLinearAttention::forward: not provided" in res.stderr, tail
        return
    assert res.returncode == 0, f"{name} exited {res.returncode}\n{tail}"


def test_reference_python_bindings_drive_a_training_step():
    if not list(DROPIN.glob("_microtorch*.so")):
        pytest.skip("the pybind module was not built (needs a reference checkout at build time)")
    z = np.load(GOLDEN / "gpt2_tiny_ckpt.npz")
    a = json.loads(bytes(z["meta_json"]).decode())["args"]
    grad_sq = sum(float((z[k].astype(np.float64) ** 2).sum()) for k in z.files if k.startswith("grad."))
    code = f"""
import sys, json
import numpy as np
sys.path.insert(0, {str(DROPIN)!r})
import _microtorch as m
z = np.load({str(GOLDEN / 'gpt2_tiny_ckpt.npz')!r})
cfg = m.nn.GPT2Config()
cfg.vocab, cfg.n_ctx, cfg.d, cfg.n_layers, cfg.n_heads = {a['vocab']}, {a['nctx']}, {a['d']}, {a['layers']}, {a['heads']}
model = m.nn.GPT2(cfg, {a['seed']})
sd = model.state_dict()
for k, v in sd.items():
    assert np.array_equal(v, z['param.' + k]), k        # the reference's initial weights, bit for bit
ids, targets = [int(i) for i in z['ids']], [int(i) for i in z['targets']]
params = model.parameters()
opt = m.nn.AdamW(params)
sched = m.nn.CosineWarmupLR(opt, 2, 10)
logits = model.forward(ids, {a['seq']})
assert logits.shape == (len(ids), cfg.vocab)
loss = m.ops.cross_entropy(logits, targets)
m.backward(loss)
sq = sum(float((p.grad.astype(np.float64) ** 2).sum()) for p in params)
total = m.ops.clip_grad_norm(params, 1e9)
opt.step(); sched.step()
after = model.state_dict()
worst = max(float(np.abs(after[k] - z['after.' + k]).max()) for k in after)
s = m.ops.softmax(m.tensor(np.arange(12, dtype=np.float32).reshape(3, 4)))
print(json.dumps(dict(loss=float(loss.data[0, 0]), sq=sq, total=float(total), worst=worst, lr=opt.lr,
                      rowsum=float(s.data.sum()))))
"""
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=_env(), cwd="/tmp", timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    out = json.loads(res.stdout.strip().splitlines()[-1])
    ref_loss = float(z["losses"][0, 0])
    assert abs(out["loss"] - ref_loss) <= 1e-4 * abs(ref_loss), (out, ref_loss)
    assert abs(out["sq"] - grad_sq) <= 2e-4 * grad_sq, (out["sq"], grad_sq)
    assert abs(out["total"] - np.sqrt(grad_sq)) <= 2e-4 * np.sqrt(grad_sq)
    assert out["worst"] <= 2.1e-3                      # one AdamW step from the reference's weights
    assert abs(out["lr"] - 0.5e-3) < 1e-9              # warm-up: step 1 of 2 from the base rate 1e-3
    assert abs(out["rowsum"] - 3.0) < 1e-5
