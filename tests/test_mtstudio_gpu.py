"""The mtstudio-compatible driver on the GPU: the reference trainer's loop (tools/mtstudio.cpp:448-518
-- zero_grad, `accum` micro-batches of `batch` stacked sequences, backward pre-scaled by 1/accum,
clip, AdamW) with per-block activation checkpointing, emitting the reference's JSONL events
(:181-192, 482-486, 561-566): model, step (loss, grad_norm), eval (val_loss), export, done; then a
resumed run picks up at the saved step."""
import json
import os
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
EXE = ROOT / "paperkiln_b200" / "mtstudio"


def run_spec(tmp_path, spec):
    p = tmp_path / "spec.json"
    p.write_text(json.dumps(spec))
    env = dict(os.environ, MICROTORCH_DEVICE="cuda")
    res = subprocess.run([str(EXE), "run", str(p)], capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-1500:]
    return [json.loads(l) for l in res.stdout.splitlines() if l.startswith("{")]


@pytest.mark.parametrize("preset,dtype", [("llama-tiny", "fp32"), ("gpt2-nano", "bf16")])
def test_training_run_emits_the_reference_event_stream(tmp_path, preset, dtype):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    out = tmp_path / "out"
    # a corpus with structure to learn: a cycle of 40 words, so the next word is a function of the current one
    words = [f"w{i}" for i in range(40)]
    corpus = tmp_path / "corpus.txt"
    corpus.write_text(" ".join(words[i % 40] for i in range(30000)))
    spec = {"name": "r", "arch": {"preset": preset}, "data": {"corpus": str(corpus), "vocab_cap": 256, "T": 64},
            "train": {"steps": 12, "lr": 3e-3, "eval_every": 4, "checkpoint_every": 6, "batch": 4, "accum": 2,
                      "checkpoint_activations": True, "dtype": dtype},
            "export": {"formats": ["safetensors", "gguf"]}, "out_dir": str(out)}
    ev = run_spec(tmp_path, spec)
    kinds = [e["event"] for e in ev]
    assert kinds[0] == "model" and kinds[-1] == "done"
    model = ev[0]
    assert model["checkpoint_activations"] is True and model["batch"] == 4 and model["accum"] == 2 and model["vocab"] == 41
    assert model["position"] == ("rope" if preset.startswith("llama") else "learned")
    steps = [e for e in ev if e["event"] == "step"]
    assert [e["step"] for e in steps] == list(range(1, 13))
    assert all(e["loss"] > 0 and e["grad_norm"] > 0 for e in steps)
    assert steps[-1]["loss"] < 0.8 * steps[0]["loss"]
    assert [e["step"] for e in ev if e["event"] == "eval"] == [4, 8, 12]
    exports = {e["format"]: e for e in ev if e["event"] in ("export", "export_skipped")}
    assert Path(exports["safetensors"]["path"]).exists()
    if preset.startswith("llama"):
        assert Path(exports["gguf"]["path"]).exists()
    else:
        assert exports["gguf"]["event"] == "export_skipped"
    assert ev[-1]["final_step"] == 12 and ev[-1]["early_stopped"] is False
    assert (out / "events.jsonl").read_text().count("\n") == len(ev)
    assert (out / "model.safetensors").exists() and (out / "state.txt").read_text().strip() == "12"
    result = json.loads((out / "result.json").read_text())
    assert result["final_step"] == 12 and result["checkpoint_activations"] is True and result["tokens_per_second"] > 0
    # a longer run over the same directory resumes at step 12, weights and AdamW moments restored
    spec["train"]["steps"] = 14
    ev2 = run_spec(tmp_path, spec)
    assert ev2[1] == {"event": "resume", "step": 12}
    assert [e["step"] for e in ev2 if e["event"] == "step"] == [13, 14]
    assert ev2[2]["loss"] < steps[0]["loss"]
