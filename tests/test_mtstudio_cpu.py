"""The mtstudio-compatible driver (paperkiln_b200/host/examples/mtstudio.cpp) without a GPU: it
reads the reference's run-spec keys (tools/mtstudio.cpp:83-169 there) -- `plan` resolves a spec
and touches no device -- and refuses what it does not provide with a message."""
import json
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
EXE = ROOT / "paperkiln_b200" / "mtstudio"


def plan(tmp_path, spec, mode="plan"):
    p = tmp_path / "spec.json"
    p.write_text(spec if isinstance(spec, str) else json.dumps(spec))
    return subprocess.run([str(EXE), mode, str(p)], capture_output=True, text=True, timeout=60)


def test_plan_resolves_presets_custom_dims_and_training_keys(tmp_path):
    if not EXE.exists():
        pytest.skip("package not built")
    spec = """{
      // comments are accepted, as by the reference's reader
      "name": "t1", "arch": {"preset": "llama-tiny", "custom": {"layers": 3, "d_ff": 256}},
      "data": {"vocab_cap": 300, "T": 32, "synthetic_tokens": 5000},
      "train": {"steps": 7, "batch": 4, "accum": 2, "checkpoint_activations": true, "seed": 11},
      "out_dir": "%s"
    }""" % (tmp_path / "out")
    res = plan(tmp_path, spec)
    assert res.returncode == 0, res.stderr
    line = res.stdout.strip()
    for part in ("family=llama", "d=128", "layers=3", "heads=4", "T=32", "d_ff=256", "vocab=300", "steps=7", "batch=4",
                 "accum=2", "checkpoint_activations=1"):
        assert part in line, (part, line)
    # gpt2 presets resolve to the flex family (whose defaults are the GPT-2 block), default d_ff = 4 d
    res = plan(tmp_path, {"arch": {"preset": "gpt2-small"}, "data": {"vocab_cap": 100}})
    assert res.returncode == 0 and "family=flex" in res.stdout and "d=256" in res.stdout and "d_ff=1024" in res.stdout
    # flavour knobs: rope means the llama block
    res = plan(tmp_path, {"arch": {"custom": {"d": 64, "heads": 2, "position": "rope"}}, "data": {"vocab_cap": 100}})
    assert res.returncode == 0 and "family=llama" in res.stdout and "d_ff=192" in res.stdout


def test_corpus_and_word_vocabulary(tmp_path):
    if not EXE.exists():
        pytest.skip("package not built")
    corpus = tmp_path / "c.txt"
    corpus.write_text(" ".join(["the cat sat on the mat and the dog sat too"] * 200))
    res = plan(tmp_path, {"arch": {"preset": "gpt2-nano"}, "data": {"corpus": str(corpus), "T": 16, "vocab_cap": 6}})
    assert res.returncode == 0, res.stderr
    assert "vocab=6" in res.stdout and "tokens=2200" in res.stdout


@pytest.mark.parametrize("spec,msg", [
    ({"arch": {"preset": "kimi-tiny"}}, "not provided"),
    ({"arch": {"custom": {"attention": "srd"}}}, "outside this library"),
    ({"train": {"optimizer": "muon"}}, "adamw"),
    ({"arch": {"custom": {"position": "rope", "norm": "layernorm"}}}, "llama block"),
    ("{\"name\": }", "spec:"),
])
def test_what_is_not_provided_is_refused_with_a_message(tmp_path, spec, msg):
    if not EXE.exists():
        pytest.skip("package not built")
    res = plan(tmp_path, spec)
    assert res.returncode == 1 and msg in res.stderr, res.stderr
