"""Worker of tests/test_dp_gpu.py: one rank of a batch-sharded data-parallel step over NCCL.

Every rank steps its shard of one global batch with the loss scaled by 1/world while the
gradients are all-reduced during the backward pass; rank 0 then steps the whole batch alone on
a second model of the same seed and compares: summed shard gradients == full-batch gradients
(the identity the reference asserts for accumulation, tests/test_batching.cpp:75-106), up to
fp32 summation order. Three variants:
    torch    per-block buckets all-reduced by torch.distributed from the Python segment hook
    pk       the exchange inside the library (mt_dp_*: libpk's collective group, no Python on the path)
    qlora    the same on a QLoRA model: only LoRA gradients exist, sent as one flat buffer
Usage (under torchrun): dp_worker.py [torch|pk|qlora]"""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


class _Buf:
    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def main():
    variant = sys.argv[1] if len(sys.argv) > 1 else "torch"
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from paperkiln_b200 import model as mt
    from paperkiln_b200.dp import BucketAllReducer, shard_tokens
    mt.init(local, mt.FP32)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    mt.set_stream(stream.cuda_stream)
    spec = dict(family="llama", vocab=512, d=128, layers=3, heads=4, kv_heads=2, dff=256, nctx=64, rope_all=1, seed=3, ckpt=1)
    if variant == "qlora":
        spec.update(qlora=1, rank=8, alpha=16)
    B, S = 8, 64
    ids_all = np.random.RandomState(5).randint(0, spec["vocab"], size=B * S + 1).astype(np.int32)
    ids, tg = shard_tokens(ids_all, B, S, rank, world)
    m = mt.Model(**spec)
    if variant == "torch":
        reducer = BucketAllReducer([torch.as_tensor(_Buf(p, n), device="cuda") for (p, n) in m.buckets()])
        mt.set_segment_hook(reducer.on_segment)
        loss = m.step(ids, tg, seq_len=S, loss_scale=1.0 / world)
        reducer.finish()
        launched = len(m.buckets())
    else:
        # rank 0 draws the communicator id; it travels as a byte tensor over the launcher's group
        idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            idt.copy_(torch.frombuffer(bytearray(mt.Model.dp_unique_id()), dtype=torch.uint8))
        dist.broadcast(idt, 0)
        m.dp_init(bytes(idt.cpu().numpy().tobytes()), rank, world)
        if variant == "pk":
            m.dp_set_flat_threshold(0)   # this small model would otherwise go out as one flat buffer
        loss = m.step(ids, tg, seq_len=S, loss_scale=1.0 / world)
        m.dp_finish()
        m.dp_wait_host()
        launched, single = m.dp_stats()
        if variant == "qlora" and not (single and launched == 1):
            print(f"qlora: expected one flat collective, got {launched} (single={single})")
            return 1
        if variant == "pk" and (single or launched != len(m.buckets())):
            print(f"pk: expected {len(m.buckets())} bucket collectives, got {launched} (single={single})")
            return 1
    torch.cuda.synchronize()
    grads = m.grads()
    t = torch.tensor([loss / world], device="cuda")
    dist.all_reduce(t)
    mean_loss = float(t.item())
    if variant == "torch":
        mt.set_segment_hook(None)
    else:
        m.dp_destroy()
    ok = True
    if rank == 0:
        full = mt.Model(**spec)
        full_loss = full.step(ids_all[:-1], ids_all[1:], seq_len=S)
        ref = full.grads()
        if abs(mean_loss - full_loss) > 1e-5 * abs(full_loss):
            print(f"loss: mean of shards {mean_loss} vs full batch {full_loss}")
            ok = False
        if variant == "qlora" and not all(("lora_A" in n or "lora_B" in n) for n in ref):
            print("qlora: a parameter other than the LoRA matrices is trainable:", sorted(ref))
            ok = False
        for n, g in ref.items():
            a = grads[n]
            scale = max(1e-6, float(np.abs(g).max()))
            if a is None or float(np.abs(a - g).max()) > 2e-5 * scale:
                print(f"{n}: max abs diff {None if a is None else float(np.abs(a - g).max()):.3e} (scale {scale:.3e})")
                ok = False
        print(f"dp_worker[{variant}]: world {world}, {launched} collective(s), loss {mean_loss:.6f} vs {full_loss:.6f}: "
              f"{'OK' if ok else 'MISMATCH'}")
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
