"""Host-side protocol of the collective group (pk_comm_*, include/pk.h) on CPU ranks: the file
backend moves host buffers between processes, so ordering, the time limit, abort and use after
abort are exercised without a GPU and without faulting anything. A rank that is late is waited
for; a rank that never joins makes the others time out with PK_ERR_TIMEOUT, after which their
communicator is dead (PK_ERR_COMM) and is torn down cleanly."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
WORKER = ROOT / "tests" / "comm_worker.py"


def run_ranks(tmp_path, world, scenario):
    d = tmp_path / "exchange"
    d.mkdir()
    procs = []
    for r in range(world):
        out = tmp_path / f"out{r}.json"
        procs.append((out, subprocess.Popen([sys.executable, str(WORKER), str(d), str(r), str(world), scenario, str(out)],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    results = []
    for out, p in procs:
        log, _ = p.communicate(timeout=120)
        assert p.returncode == 0, log
        results.append(json.loads(out.read_text()))
    return results


@pytest.mark.parametrize("world", [2, 3])
def test_sums_are_exact_and_identical_on_every_rank(tmp_path, world):
    for res in run_ranks(tmp_path, world, "sum"):
        assert len(res["rounds"]) == 3 and all(r["ok"] and r["rc"] == [0, 0, 0] for r in res["rounds"]), res


def test_a_late_rank_is_waited_for(tmp_path):
    results = run_ranks(tmp_path, 2, "late")
    for res in results:
        assert all(r["ok"] for r in res["rounds"]), res
    # rank 0 sat in its wait while rank 1 slept
    assert results[0]["rounds"][1]["wait_s"] > 0.3


def test_an_absent_rank_runs_the_others_into_the_time_limit(tmp_path):
    results = run_ranks(tmp_path, 3, "absent")
    assert results[2].get("left_early")
    for res in results[:2]:
        assert res["rounds"][0]["ok"]
        second = res["rounds"][1]
        assert second["rc"][2] == 4 and not second["ok"], res          # PK_ERR_TIMEOUT
        assert 0.4 < second["wait_s"] < 5.0, second                    # the 0.5 s limit, not a hang
        after = res["after_timeout"]
        assert after["alive"] == 0 and after["next_rc"] == 6 and after["abort_rc"] == 0, after   # PK_ERR_COMM
        assert "did not join" in after["msg"] or "aborted" in after["msg"]


def test_nccl_entry_points_fail_cleanly_without_a_gpu():
    """pk_comm_unique_id / pk_comm_init need NCCL and a GPU; without them they return an error
    code and a message instead of crashing."""
    import ctypes
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    sys.path.insert(0, str(ROOT))
    from paperkiln_b200._capi import libpk
    pk = libpk()
    buf = (ctypes.c_char * 128)()
    assert pk.pk_comm_unique_id(buf, 16) == 1      # PK_ERR_INVALID: the id needs 128 bytes
    comm = ctypes.c_void_p()
    assert pk.pk_comm_init_file(b"/nonexistent/dir", 0, 1, ctypes.byref(comm)) == 1
    assert pk.pk_comm_init(buf, 2, 2, 0, ctypes.byref(comm)) == 1   # rank out of range
