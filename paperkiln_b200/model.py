"""Python driver over libmicrotorch (the C++ tape + models) through its C entry points.

This is plumbing for tests and benchmarks: it builds a model from a spec, moves numpy
arrays across the C ABI and runs the checkpointed training step. All computation
happens in the CUDA kernels of libpk; nothing here has a CPU fallback.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Tuple

import numpy as np

from ._capi import libmt

FP32, BF16 = 0, 1


class MtError(RuntimeError):
    pass


def _check(rc: int, what: str):
    if rc != 0:
        raise MtError(f"{what}: {libmt().mt_last_error().decode(errors='replace')}")


def init(device: int = 0, dtype: int = FP32):
    _check(libmt().mt_init(device, dtype), "mt_init")


def set_stream(cuda_stream: Optional[int]):
    _check(libmt().mt_set_stream(ctypes.c_void_p(cuda_stream) if cuda_stream else None), "mt_set_stream")


def sync():
    _check(libmt().mt_sync(), "mt_sync")


def mem_stats() -> Dict[str, int]:
    out = (ctypes.c_uint64 * 6)()
    _check(libmt().mt_mem_stats(out), "mt_mem_stats")
    keys = ("activation_in_use", "activation_peak", "persistent_in_use", "persistent_peak", "reserved",
            "driver_allocs")
    return dict(zip(keys, (int(v) for v in out)))


def peak_blocks() -> Dict[int, int]:
    """{block bytes: number of blocks} of the activations that were live at the high-water mark."""
    sizes, counts, n = (ctypes.c_uint64 * 256)(), (ctypes.c_uint64 * 256)(), ctypes.c_int(0)
    _check(libmt().mt_mem_peak_blocks(sizes, counts, 256, ctypes.byref(n)), "mt_mem_peak_blocks")
    return {int(sizes[i]): int(counts[i]) for i in range(min(n.value, 256))}


def reset_peak():
    _check(libmt().mt_reset_peak(), "mt_reset_peak")


def empty_cache():
    _check(libmt().mt_empty_cache(), "mt_empty_cache")


def live_variables() -> int:
    n = ctypes.c_int64(0)
    _check(libmt().mt_live_variables(ctypes.byref(n)), "mt_live_variables")
    return n.value


_SEGMENT_CB = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_void_p)
_hook_keepalive = None


def set_segment_hook(fn):
    """fn(k) is called after the backward of the k-th checkpointed block was enqueued."""
    global _hook_keepalive
    if fn is None:
        _check(libmt().mt_set_segment_hook(None, None), "mt_set_segment_hook")
        _hook_keepalive = None
        return
    cb = _SEGMENT_CB(lambda k, _user: fn(k))
    _hook_keepalive = cb
    _check(libmt().mt_set_segment_hook(ctypes.cast(cb, ctypes.c_void_p), None), "mt_set_segment_hook")


def spec_string(**kw) -> str:
    return ";".join(f"{k}={v}" for k, v in kw.items())


class Model:
    """A model of one of the families llama | gpt2 | flex living on the GPU."""

    def __init__(self, **spec):
        self.spec = dict(spec)
        self._h = ctypes.c_void_p()
        _check(libmt().mt_model_create(spec_string(**spec).encode(), ctypes.byref(self._h)), "mt_model_create")
        n = ctypes.c_int64(0)
        _check(libmt().mt_model_num_params(self._h, ctypes.byref(n)), "mt_model_num_params")
        self.names: List[str] = []
        self.shapes: List[Tuple[int, int]] = []
        buf = ctypes.create_string_buffer(256)
        for i in range(n.value):
            r, c = ctypes.c_int64(0), ctypes.c_int64(0)
            _check(libmt().mt_model_param_info(self._h, i, buf, 256, ctypes.byref(r), ctypes.byref(c)),
                   "mt_model_param_info")
            self.names.append(buf.value.decode())
            self.shapes.append((r.value, c.value))
        self._index = {n_: i for i, n_ in enumerate(self.names)}

    def close(self):
        if self._h:
            libmt().mt_model_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- parameters / gradients as numpy ----
    def get_param(self, name: str) -> np.ndarray:
        i = self._index[name]
        out = np.empty(self.shapes[i], dtype=np.float32)
        _check(libmt().mt_model_param_get(self._h, i, out.ctypes.data_as(ctypes.c_void_p)), "mt_model_param_get")
        return out

    def set_param(self, name: str, value: np.ndarray):
        i = self._index[name]
        v = np.ascontiguousarray(value, dtype=np.float32).reshape(self.shapes[i])
        _check(libmt().mt_model_param_set(self._h, i, v.ctypes.data_as(ctypes.c_void_p)), "mt_model_param_set")

    def get_grad(self, name: str) -> Optional[np.ndarray]:
        i = self._index[name]
        out = np.empty(self.shapes[i], dtype=np.float32)
        has = ctypes.c_int(0)
        _check(libmt().mt_model_grad_get(self._h, i, out.ctypes.data_as(ctypes.c_void_p), ctypes.byref(has)),
               "mt_model_grad_get")
        return out if has.value else None

    def state_dict(self) -> Dict[str, np.ndarray]:
        return {n: self.get_param(n) for n in self.names}

    def load_state_dict(self, sd: Dict[str, np.ndarray]):
        for n in self.names:
            self.set_param(n, sd[n])

    def grads(self) -> Dict[str, Optional[np.ndarray]]:
        return {n: self.get_grad(n) for n in self.names}

    # ---- the step ----
    def set_checkpoint(self, on: bool):
        _check(libmt().mt_model_set_checkpoint(self._h, int(on)), "mt_model_set_checkpoint")

    # ---- a single block (family="block") ----
    def block_set_input(self, x: np.ndarray, dy: np.ndarray, seq_len: int):
        """x, dy: [rows, d] fp32 host arrays (block input and upstream gradient of its output)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        dy = np.ascontiguousarray(dy, dtype=np.float32)
        assert x.shape == dy.shape and x.ndim == 2
        self._block_shape = x.shape
        _check(libmt().mt_block_set_input(self._h, x.ctypes.data_as(ctypes.c_void_p), dy.ctypes.data_as(ctypes.c_void_p),
                                          x.shape[0], int(seq_len)), "mt_block_set_input")

    def block_forward(self):
        _check(libmt().mt_block_forward(self._h), "mt_block_forward")

    def block_backward(self):
        """Backward of the pending forward: recompute + backward when checkpointing is on."""
        _check(libmt().mt_block_backward(self._h), "mt_block_backward")

    def block_output(self) -> np.ndarray:
        out = np.empty(self._block_shape, dtype=np.float32)
        _check(libmt().mt_block_output(self._h, out.ctypes.data_as(ctypes.c_void_p)), "mt_block_output")
        return out

    def block_input_grad(self) -> np.ndarray:
        out = np.empty(self._block_shape, dtype=np.float32)
        _check(libmt().mt_block_input_grad(self._h, out.ctypes.data_as(ctypes.c_void_p)), "mt_block_input_grad")
        return out

    def set_loss_chunk(self, rows: int):
        """rows > 0: fused head + cross entropy over row chunks (default 16384); 0: separate ops."""
        _check(libmt().mt_model_set_loss_chunk(self._h, int(rows)), "mt_model_set_loss_chunk")

    def step(self, ids, targets, seq_len: int = 0, loss_scale: float = 1.0, backward: bool = True) -> float:
        """zero_grad + forward + cross entropy (+ backward). ids/targets: int32 arrays (host)."""
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        targets = np.ascontiguousarray(targets, dtype=np.int32)
        loss = ctypes.c_float(0.0)
        _check(libmt().mt_model_step(self._h, ids.ctypes.data_as(ctypes.c_void_p),
                                     targets.ctypes.data_as(ctypes.c_void_p), ids.size, seq_len,
                                     loss_scale, int(backward), ctypes.byref(loss)), "mt_model_step")
        return float(loss.value)

    def step_ptr(self, ids_ptr: int, targets_ptr: int, n: int, seq_len: int, loss_scale: float = 1.0) -> float:
        """Same as step() for int32 host buffers given by address (e.g. pinned memory)."""
        loss = ctypes.c_float(0.0)
        _check(libmt().mt_model_step(self._h, ctypes.c_void_p(ids_ptr), ctypes.c_void_p(targets_ptr), n, seq_len,
                                     loss_scale, 1, ctypes.byref(loss)), "mt_model_step")
        return float(loss.value)

    def live_after_forward(self) -> int:
        n = ctypes.c_int64(0)
        _check(libmt().mt_model_live_after_forward(self._h, ctypes.byref(n)), "mt_model_live_after_forward")
        return n.value

    def set_adamw(self, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01):
        _check(libmt().mt_model_set_adamw(self._h, lr, beta1, beta2, eps, weight_decay), "mt_model_set_adamw")

    def optimizer_step(self):
        _check(libmt().mt_model_optimizer_step(self._h), "mt_model_optimizer_step")

    # ---- gradient accumulation (tools/mtstudio.cpp:456-474 of the reference) ----
    def set_accumulate(self, on: bool):
        """With accumulation on, step() adds to the gradients instead of clearing them first."""
        _check(libmt().mt_model_set_accumulate(self._h, 1 if on else 0), "mt_model_set_accumulate")

    def zero_grad(self):
        _check(libmt().mt_model_zero_grad(self._h), "mt_model_zero_grad")

    # ---- optimizer state for checkpoint / resume ----
    def optimizer_steps(self) -> int:
        t = ctypes.c_int64(0)
        _check(libmt().mt_model_optimizer_steps_get(self._h, ctypes.byref(t)), "mt_model_optimizer_steps_get")
        return int(t.value)

    def optimizer_state(self) -> dict:
        """{"t": steps taken, "m": {name: array}, "v": {name: array}} on the host."""
        out = {"t": self.optimizer_steps(), "m": {}, "v": {}}
        for name, i in self._index.items():
            m = np.empty(self.shapes[i], dtype=np.float32)
            v = np.empty(self.shapes[i], dtype=np.float32)
            rc = libmt().mt_model_optimizer_state_get(self._h, i, m.ctypes.data_as(ctypes.c_void_p),
                                                      v.ctypes.data_as(ctypes.c_void_p))
            _check(rc, "mt_model_optimizer_state_get")
            out["m"][name], out["v"][name] = m, v
        return out

    def load_optimizer_state(self, state: dict):
        _check(libmt().mt_model_optimizer_steps_set(self._h, int(state["t"])), "mt_model_optimizer_steps_set")
        for name, i in self._index.items():
            m = np.ascontiguousarray(state["m"][name], dtype=np.float32).reshape(self.shapes[i])
            v = np.ascontiguousarray(state["v"][name], dtype=np.float32).reshape(self.shapes[i])
            rc = libmt().mt_model_optimizer_state_set(self._h, i, m.ctypes.data_as(ctypes.c_void_p),
                                                      v.ctypes.data_as(ctypes.c_void_p))
            _check(rc, "mt_model_optimizer_state_set")

    # ---- checkpoint files (safetensors, the reference's layout) ----
    def save(self, weights_path: str, optimizer_path: Optional[str] = None):
        _check(libmt().mt_model_save(self._h, weights_path.encode(), optimizer_path.encode() if optimizer_path else None),
               "mt_model_save")

    def load(self, weights_path: Optional[str], optimizer_path: Optional[str] = None):
        _check(libmt().mt_model_load(self._h, weights_path.encode() if weights_path else None,
                                     optimizer_path.encode() if optimizer_path else None), "mt_model_load")

    def load_base(self, weights_path: str):
        """QLoRA models: frozen base from a dense model's weights file, quantised on the device."""
        _check(libmt().mt_model_load_base(self._h, weights_path.encode()), "mt_model_load_base")

    def save_merged(self, weights_path: str):
        """QLoRA models: the equivalent dense model's weights file (base + merged LoRA)."""
        _check(libmt().mt_model_save_merged(self._h, weights_path.encode()), "mt_model_save_merged")

    def export_gguf(self, path: str, name: str = "microtorch-model", context_length: int = 2048):
        """GGUF v3 file of a llama-family model (adapters merged), the reference exporter's layout."""
        _check(libmt().mt_model_export_gguf(self._h, path.encode(), name.encode(), context_length),
               "mt_model_export_gguf")

    def clip_grad_norm(self, max_norm: float) -> float:
        n = ctypes.c_float(0.0)
        _check(libmt().mt_model_clip_grad_norm(self._h, max_norm, ctypes.byref(n)), "mt_model_clip_grad_norm")
        return float(n.value)

    # ---- data parallelism inside the library (mt_dp_*: NCCL through libpk's collective group) ----
    @staticmethod
    def dp_unique_id() -> bytes:
        """The 128-byte communicator id; rank 0 draws it and the launcher hands it to every rank."""
        buf = ctypes.create_string_buffer(128)
        _check(libmt().mt_dp_unique_id(buf, 128), "mt_dp_unique_id")
        return buf.raw

    def dp_init(self, unique_id: bytes, rank: int, world: int, max_ctas: int = 0):
        _check(libmt().mt_dp_init(self._h, unique_id, rank, world, max_ctas), "mt_dp_init")

    def dp_enable(self, on: bool):
        _check(libmt().mt_dp_enable(self._h, int(on)), "mt_dp_enable")

    def dp_finish(self):
        _check(libmt().mt_dp_finish(self._h), "mt_dp_finish")

    def dp_wait_host(self):
        _check(libmt().mt_dp_wait_host(self._h), "mt_dp_wait_host")

    def dp_set_timeout(self, seconds: float):
        _check(libmt().mt_dp_set_timeout(self._h, seconds), "mt_dp_set_timeout")

    def dp_set_flat_threshold(self, nbytes: int):
        _check(libmt().mt_dp_set_flat_threshold(self._h, nbytes), "mt_dp_set_flat_threshold")

    def dp_stats(self) -> Tuple[int, bool]:
        """(collectives started in the last finished step, whole gradient sent as one buffer)."""
        n, single = ctypes.c_int64(0), ctypes.c_int(0)
        _check(libmt().mt_dp_stats(self._h, ctypes.byref(n), ctypes.byref(single)), "mt_dp_stats")
        return int(n.value), bool(single.value)

    def dp_destroy(self):
        _check(libmt().mt_dp_destroy(self._h), "mt_dp_destroy")

    # ---- data-parallel gradient buckets ----
    def buckets(self) -> List[Tuple[int, int]]:
        """[(device pointer, fp32 element count)]: one per transformer block, then the rest."""
        n = ctypes.c_int64(0)
        _check(libmt().mt_model_num_buckets(self._h, ctypes.byref(n)), "mt_model_num_buckets")
        out = []
        for i in range(n.value):
            p, c = ctypes.c_void_p(), ctypes.c_int64(0)
            _check(libmt().mt_model_bucket(self._h, i, ctypes.byref(p), ctypes.byref(c)), "mt_model_bucket")
            out.append((int(p.value), int(c.value)))
        return out
