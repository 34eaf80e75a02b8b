"""Data-parallel path on CPU ranks (gloo, world size 2): batch sharding + per-block gradient
buckets all-reduced in the order the checkpointed backward releases them reproduce the
full-batch gradients. Gradients come from the numpy oracle (the checker), the bucket
logic is the shipped paperkiln_b200.dp code that bench.py runs on GPUs with NCCL."""
import json
import os
import socket
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import pk_oracle as O
from paperkiln_b200 import dp

GOLDEN = Path(__file__).resolve().parent / "golden"


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _bucket_layout(names, shapes, n_layers):
    """Same packing order as the C driver: block 0 .. L-1, then the rest."""
    order, bounds = [], []
    for b in range(n_layers):
        first = len(order)
        order += [n for n in names if n.startswith(f"layers.{b}.")]
        bounds.append((first, len(order)))
    first = len(order)
    order += [n for n in names if not n.startswith("layers.")]
    bounds.append((first, len(order)))
    return order, bounds


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        z = np.load(GOLDEN / "llama_tiny_ckpt.npz")
        a = json.loads(bytes(z["meta_json"]).decode())["args"]
        params = {k[len("param."):]: z[k] for k in z.files if k.startswith("param.")}
        B, S = a["batch"], a["seq"]
        stream = np.concatenate([z["ids"], z["targets"][-1:]])
        ids, targets = dp.shard_tokens(stream, B, S, rank, world)
        orc = O.StepOracle("llama", params, heads=a["heads"], layers=a["layers"])
        loss, grads = orc.step(ids, targets, seq_len=S)
        names = sorted(params)
        order, bounds = _bucket_layout(names, None, a["layers"])
        # local gradients scaled by 1/world (the loss scale), packed into per-block buckets
        buckets = []
        for lo, hi in bounds:
            flat = np.concatenate([grads[n].ravel() for n in order[lo:hi]]) / world
            buckets.append(torch.from_numpy(flat.astype(np.float32)))
        red = dp.BucketAllReducer(buckets)
        launched = []
        for k in range(a["layers"]):  # segments finish in reverse block order
            red.on_segment(k)
            launched.append(red.order[-1])
        assert launched == list(range(a["layers"] - 1, -1, -1))
        red.finish()
        loss_t = torch.tensor([loss / world], dtype=torch.float64)
        dist.all_reduce(loss_t)
        if rank == 0:
            np.savez(Path(out_dir) / "dp.npz", loss=loss_t.numpy(), **{f"b{i}": b.numpy() for i, b in enumerate(buckets)})
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_rank_data_parallel_equals_full_batch(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    got = np.load(tmp_path / "dp.npz")
    z = np.load(GOLDEN / "llama_tiny_ckpt.npz")
    a = json.loads(bytes(z["meta_json"]).decode())["args"]
    params = {k[len("param."):]: z[k] for k in z.files if k.startswith("param.")}
    orc = O.StepOracle("llama", params, heads=a["heads"], layers=a["layers"])
    loss, grads = orc.step(z["ids"], z["targets"], seq_len=a["seq"])
    assert abs(float(got["loss"][0]) - loss) < 1e-5
    order, bounds = _bucket_layout(sorted(params), None, a["layers"])
    for i, (lo, hi) in enumerate(bounds):
        ref = np.concatenate([grads[n].ravel() for n in order[lo:hi]])
        assert float(np.abs(got[f"b{i}"] - ref).max()) < 1e-5
        # and against the reference's own full-batch gradients
        gold = np.concatenate([z["grad." + n].ravel() for n in order[lo:hi]])
        assert float(np.abs(got[f"b{i}"] - gold).max()) < 1e-4


def _accum_stream(vocab, n):
    return np.random.RandomState(4321).randint(0, vocab, size=n + 1).astype(np.int32)


def _worker_accum(rank, world, port, out_dir):
    """Two micro-batches per rank: gradients add up locally, the hook is muted for the first
    micro-batch and the buckets are exchanged once, during the last one."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        z = np.load(GOLDEN / "llama_tiny_ckpt.npz")
        a = json.loads(bytes(z["meta_json"]).decode())["args"]
        params = {k[len("param."):]: z[k] for k in z.files if k.startswith("param.")}
        B, S, accum = 4, a["seq"], 2
        ids, targets = dp.shard_tokens(_accum_stream(a["vocab"], B * S), B, S, rank, world)
        orc = O.StepOracle("llama", params, heads=a["heads"], layers=a["layers"])
        order, bounds = _bucket_layout(sorted(params), None, a["layers"])
        buckets = [torch.zeros(sum(params[n].size for n in order[lo:hi]), dtype=torch.float32) for lo, hi in bounds]
        red = dp.BucketAllReducer(buckets)
        n_micro = len(ids) // accum
        for k in range(accum):
            red.enabled = k == accum - 1
            sl = slice(k * n_micro, (k + 1) * n_micro)
            _, grads = orc.step(ids[sl], targets[sl], seq_len=S)
            for b, (lo, hi) in zip(buckets, bounds):
                flat = np.concatenate([grads[n].ravel() for n in order[lo:hi]]) / (world * accum)
                b += torch.from_numpy(flat.astype(np.float32))
            for seg in range(a["layers"]):
                red.on_segment(seg)
            assert len(red.order) == (a["layers"] if red.enabled else 0)
        red.finish()
        if rank == 0:
            np.savez(Path(out_dir) / "dp_accum.npz", **{f"b{i}": b.numpy() for i, b in enumerate(buckets)})
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_rank_accumulation_exchanges_once_and_equals_full_batch(tmp_path):
    world = 2
    mp.spawn(_worker_accum, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    got = np.load(tmp_path / "dp_accum.npz")
    z = np.load(GOLDEN / "llama_tiny_ckpt.npz")
    a = json.loads(bytes(z["meta_json"]).decode())["args"]
    params = {k[len("param."):]: z[k] for k in z.files if k.startswith("param.")}
    stream = _accum_stream(a["vocab"], 4 * a["seq"])
    orc = O.StepOracle("llama", params, heads=a["heads"], layers=a["layers"])
    _, grads = orc.step(stream[:-1], stream[1:], seq_len=a["seq"])
    order, bounds = _bucket_layout(sorted(params), None, a["layers"])
    for i, (lo, hi) in enumerate(bounds):
        ref = np.concatenate([grads[n].ravel() for n in order[lo:hi]])
        assert float(np.abs(got[f"b{i}"] - ref).max()) < 1e-5
