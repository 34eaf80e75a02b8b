"""One CPU rank of the collective group's file backend (pk_comm_init_file): run as a child
process by tests/test_comm_cpu.py.

    python tests/comm_worker.py <dir> <rank> <world> <scenario> <out.json>

scenarios
  sum     three rounds of two collectives each (started back to back, then waited for), sums checked
  late    rank 1 sleeps 0.6 s before joining the second round; everybody still gets the sums
  absent  the last rank never joins the second round: the others run into the 0.5 s limit,
          see PK_ERR_TIMEOUT, find the communicator dead (PK_ERR_COMM) and leave cleanly
"""
import ctypes
import json
import sys
import time
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from paperkiln_b200._capi import libpk  # noqa: E402

PK_ERR_TIMEOUT, PK_ERR_COMM = 4, 6


def main():
    d, rank, world, scenario, out = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4], sys.argv[5]
    pk = libpk()
    comm = ctypes.c_void_p()
    assert pk.pk_comm_init_file(d.encode(), rank, world, ctypes.byref(comm)) == 0, pk.pk_last_error()
    assert pk.pk_comm_set_timeout(comm, 0.5 if scenario == "absent" else 20.0) == 0
    res = {"rank": rank, "rounds": []}

    def one_round(r):
        a = (np.arange(1000, dtype=np.float32) + 1000.0 * rank + r).copy()
        b = np.full(7, 0.25 * (rank + 1) + r, dtype=np.float32)
        rc1 = pk.pk_allreduce_async(comm, a.ctypes.data_as(ctypes.c_void_p), a.size, None)
        rc2 = pk.pk_allreduce_async(comm, b.ctypes.data_as(ctypes.c_void_p), b.size, None)
        t0 = time.perf_counter()
        rcw = pk.pk_comm_wait(comm, None)
        dt = time.perf_counter() - t0
        exp_a = sum(np.arange(1000, dtype=np.float32) + 1000.0 * k + r for k in range(world))
        exp_b = np.full(7, sum(np.float32(0.25 * (k + 1) + r) for k in range(world)), dtype=np.float32)
        ok = rcw == 0 and bool(np.array_equal(a, exp_a)) and bool(np.array_equal(b, exp_b))
        res["rounds"].append({"rc": [rc1, rc2, rcw], "ok": ok, "wait_s": dt})
        return rcw

    one_round(0)
    if scenario == "late" and rank == 1:
        time.sleep(0.6)
    if scenario == "absent" and rank == world - 1:
        res["left_early"] = True
    else:
        rc = one_round(1)
        if scenario == "absent":
            alive = ctypes.c_int(-1)
            pk.pk_comm_info(comm, None, None, None, ctypes.byref(alive))
            x = np.ones(4, dtype=np.float32)
            res["after_timeout"] = {"rc": rc, "alive": alive.value,
                                    "next_rc": pk.pk_allreduce_async(comm, x.ctypes.data_as(ctypes.c_void_p), 4, None),
                                    "abort_rc": pk.pk_comm_abort(comm), "msg": pk.pk_last_error().decode()}
        else:
            one_round(2)
    assert pk.pk_comm_destroy(comm) == 0
    Path(out).write_text(json.dumps(res))


if __name__ == "__main__":
    main()
