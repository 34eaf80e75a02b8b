"""Drop-in proof, CPU part: the reference's own python/bindings.cpp and five of its hot-path
tests compile UNCHANGED against this repository's headers and link against libmicrotorch.so
(`make -C oracle dropin`, run by __graft_entry__.build() when a reference checkout is at hand),
and the pybind module imports. Skipped where there is neither a reference checkout nor the
prebuilt binaries (they travel with the tree; the sources do not)."""
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
DROPIN = ROOT / "oracle" / "_ref" / "dropin"
TESTS = ["test_checkpointing", "test_llama", "test_batching", "test_flex", "test_lora_quant"]


def _reference():
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as g
    return g.reference_checkout()


def test_reference_sources_compile_against_this_library():
    ref = _reference()
    if ref is None:
        if not DROPIN.exists():
            pytest.skip("no reference checkout and no prebuilt drop-in binaries")
    else:
        res = subprocess.run(["make", "-C", str(ROOT / "oracle"), f"REF={ref}", f"PYTHON={sys.executable}", "dropin"],
                             capture_output=True, text=True)
        assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    for t in TESTS:
        assert (DROPIN / t).exists(), f"{t} was not built"
    assert list(DROPIN.glob("_microtorch*.so")), "the pybind module was not built"


def test_bindings_module_imports_and_lists_the_bound_surface():
    if not list(DROPIN.glob("_microtorch*.so")):
        pytest.skip("the pybind module was not built (no reference checkout)")
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "import _microtorch as m\n"
        "names = ['tensor', 'backward', 'zero_grad', 'load_safetensors', 'save_safetensors']\n"
        "assert all(hasattr(m, n) for n in names)\n"
        "ops = ['matmul', 'add', 'sub', 'mul', 'add_bias', 'gelu', 'silu', 'softmax', 'mean', 'scale', 'transpose',\n"
        "       'layernorm', 'rmsnorm', 'embedding', 'cross_entropy', 'dropout', 'clip_grad_norm', 'kimi_attention']\n"
        "assert all(hasattr(m.ops, n) for n in ops)\n"
        "layers = ['Module', 'Linear', 'LayerNorm', 'Dropout', 'CausalSelfAttention', 'KimiLinearAttention', 'GPT2Config',\n"
        "          'GPT2', 'SGD', 'AdamW', 'CosineWarmupLR', 'StepLR']\n"
        "assert all(hasattr(m.nn, n) for n in layers)\n"
        "print('ok')\n" % str(DROPIN))
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd="/tmp")
    assert res.returncode == 0 and "ok" in res.stdout, res.stdout + res.stderr
