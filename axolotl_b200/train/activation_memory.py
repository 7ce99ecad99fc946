"""Activation-memory tools: checkpointing whose saved layer inputs live in pinned host memory or on disk,
a saved-tensor offloader for everything outside the checkpointed layers, selective checkpointing that
keeps the attention result, and host-resident frozen layers that are streamed in around their use.

What the reference builds from monkeypatches around ``torch.utils.checkpoint`` and TRL's offloader
(src/axolotl/monkeypatch/gradient_checkpointing/offload_cpu.py:38, offload_disk.py:43-532,
src/axolotl/monkeypatch/activation_offload_checkpoint.py:49-260,
src/axolotl/monkeypatch/selective_checkpointing.py:167-330,
src/axolotl/core/trainers/mixins/layer_offloading.py:52-304) is one small runtime here: copies run on a side
stream next to the compute stream, host buffers are pinned and recycled, and what comes back is bit-identical
to what went out, so an offloaded run reproduces the plain run's gradients exactly.
"""
from __future__ import annotations

import os
import tempfile
import threading
from concurrent.futures import ThreadPoolExecutor

import torch


class _Handle:
    __slots__ = ("shape", "dtype", "device", "host", "event", "gpu", "gpu_event", "prev", "path", "future", "nbytes")

    def __init__(self):
        self.host = self.event = self.gpu = self.gpu_event = self.prev = self.path = self.future = None


class HostStore:
    """Pinned host memory as the backing store; device<->host copies on a side stream.

    ``put`` returns immediately (the copy is ordered after the producer on the compute stream);
    ``get`` first requests the tensor that will be needed NEXT in the backward pass (the one that was put
    just before this one), then hands out its own tensor, which was requested one ``get`` earlier — so a
    layer's input travels back over PCIe/NVLink-C2C while the layer after it runs its backward pass."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self._pool: dict[tuple, list] = {}
        self._last = None
        self.bytes_out = 0

    def _host_buffer(self, shape, dtype):
        key = (tuple(shape), dtype)
        free = self._pool.get(key)
        if free:
            return free.pop()
        return torch.empty(shape, dtype=dtype, pin_memory=self.cuda)

    def put(self, t: torch.Tensor) -> _Handle:
        h = _Handle()
        h.shape, h.dtype, h.device, h.nbytes = t.shape, t.dtype, t.device, t.numel() * t.element_size()
        h.prev, self._last = self._last, h
        self.bytes_out += h.nbytes
        src = t.detach()
        if not src.is_contiguous():
            src = src.contiguous()
        h.host = self._host_buffer(src.shape, src.dtype)
        if self.cuda and src.is_cuda:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                h.host.copy_(src, non_blocking=True)
                h.event = torch.cuda.Event()
                h.event.record(self.stream)
            src.record_stream(self.stream)    # the device block stays alive until the copy has run
        else:
            h.host.copy_(src)
        return h

    def _request(self, h: _Handle):
        if h is None or h.gpu is not None or h.host is None:
            return
        if self.cuda and h.device.type == "cuda":
            with torch.cuda.stream(self.stream):
                if h.event is not None:
                    self.stream.wait_event(h.event)
                h.gpu = torch.empty(h.shape, dtype=h.dtype, device=h.device)
                h.gpu.copy_(h.host, non_blocking=True)
                h.gpu_event = torch.cuda.Event()
                h.gpu_event.record(self.stream)
        else:
            h.gpu = h.host.clone()

    def get(self, h: _Handle) -> torch.Tensor:
        self._request(h)
        self._request(h.prev)             # overlaps with the backward pass of the layer that called get
        if h.gpu_event is not None:
            torch.cuda.current_stream(self.device).wait_event(h.gpu_event)
            h.gpu.record_stream(torch.cuda.current_stream(self.device))
        out, h.gpu = h.gpu, None
        self._pool.setdefault((tuple(h.shape), h.dtype), []).append(h.host)
        h.host = None
        if self._last is h:
            self._last = h.prev
        return out

    def reset(self):
        self._last = None


class DiskStore(HostStore):
    """Same interface; the host copy is written to a file by a worker thread and read back on demand."""

    def __init__(self, device, directory=None, workers=2):
        super().__init__(device)
        self.dir = directory or tempfile.mkdtemp(prefix="axb_act_")
        os.makedirs(self.dir, exist_ok=True)
        self.exec = ThreadPoolExecutor(max_workers=workers)
        self._n = 0
        self._lock = threading.Lock()

    def put(self, t):
        h = super().put(t)
        with self._lock:
            self._n += 1
            h.path = os.path.join(self.dir, f"act_{os.getpid()}_{self._n}.bin")
        host, event = h.host, h.event

        def write():
            if event is not None:
                event.synchronize()
            host.view(torch.uint8).reshape(-1).numpy().tofile(h.path)
            return True

        h.future = self.exec.submit(write)
        return h

    def _request(self, h):
        if h is None or h.gpu is not None or h.path is None:
            return
        if h.future is not None:
            h.future.result()
            h.future = None
            # the pinned buffer can go back to the pool as soon as the file exists
            self._pool.setdefault((tuple(h.shape), h.dtype), []).append(h.host)
            h.host = None
        import numpy as np

        raw = torch.from_numpy(np.fromfile(h.path, dtype=np.uint8))
        host = self._host_buffer(h.shape, h.dtype)
        host.view(torch.uint8).reshape(-1).copy_(raw)
        os.remove(h.path)
        h.path, h.host, h.event = None, host, None
        super()._request(h)


def make_store(mode, device, directory=None):
    """``mode``: True / "legacy" / "hidden_states" -> pinned host memory, "disk" -> files."""
    if mode == "disk":
        return DiskStore(device, directory)
    return HostStore(device)


class _OffloadedCheckpoint(torch.autograd.Function):
    """Activation checkpoint of one decoder layer whose saved inputs go to ``store`` instead of staying on
    the device; the backward pass fetches them, re-runs the layer with gradients and back-propagates."""

    @staticmethod
    def forward(ctx, run_fn, store, n_tensors, _needs_grad, *args):
        ctx.run_fn, ctx.store, ctx.n = run_fn, store, n_tensors
        ctx.rest = args[n_tensors:]
        ctx.kept = []
        for t in args[:n_tensors]:
            if isinstance(t, torch.Tensor) and t.is_floating_point() and t.numel() >= 4096:
                ctx.kept.append(("h", store.put(t), t.requires_grad))
            else:
                ctx.kept.append(("t", t, isinstance(t, torch.Tensor) and t.requires_grad))
        ctx.cpu_rng = torch.get_rng_state()
        dev = next((t.device for t in args[:n_tensors] if isinstance(t, torch.Tensor)), None)
        ctx.cuda_rng = torch.cuda.get_rng_state(dev) if dev is not None and dev.type == "cuda" else None
        ctx.dev = dev
        with torch.no_grad():
            outs = run_fn(*args)
        ctx.out_is_tensor = [isinstance(o, torch.Tensor) for o in outs]
        return outs

    @staticmethod
    def backward(ctx, *grads):
        ins = []
        for kind, v, rg in ctx.kept:
            t = ctx.store.get(v) if kind == "h" else v
            if isinstance(t, torch.Tensor):
                t = t.detach()
                t.requires_grad_(rg or t.is_floating_point())
            ins.append(t)
        devs = [ctx.dev] if ctx.cuda_rng is not None else []
        with torch.random.fork_rng(devices=devs):
            torch.set_rng_state(ctx.cpu_rng)
            if ctx.cuda_rng is not None:
                torch.cuda.set_rng_state(ctx.cuda_rng, ctx.dev)
            with torch.enable_grad():
                outs = ctx.run_fn(*ins, *ctx.rest)
        pairs = [(o, g) for o, g in zip(outs, grads) if isinstance(o, torch.Tensor) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        in_grads = [t.grad if isinstance(t, torch.Tensor) else None for t in ins]
        return (None, None, None, None, *in_grads, *([None] * len(ctx.rest)))


def offloaded_checkpoint(run_fn, store, tensor_args, other_args=()):
    """``run_fn(*tensor_args, *other_args)`` -> tuple; ``tensor_args`` are the (possibly None) activations to
    offload, ``other_args`` anything that is not differentiated (positions, tables, metadata). The layer's
    parameters receive their gradients during the recomputation's backward pass; an empty tensor that
    requires grad keeps the node in the graph when no activation does (adapter training on frozen
    embeddings)."""
    anchor = torch.empty(0, requires_grad=True)
    return _OffloadedCheckpoint.apply(run_fn, store, len(tensor_args), anchor, *tensor_args, *other_args)


class OffloadSavedTensors:
    """Context manager: every large floating-point tensor that autograd saves inside the block is moved to
    the store and brought back when the backward pass needs it (parameters and tensors that require grad
    themselves are left alone). Used around the parts of the step that are not checkpointed layers."""

    def __init__(self, store, min_bytes=1 << 20):
        self.store, self.min_bytes = store, min_bytes
        self._ctx = None

    def _pack(self, t):
        skip = (not isinstance(t, torch.Tensor) or isinstance(t, torch.nn.Parameter) or not t.is_floating_point()
                or t.numel() * t.element_size() < self.min_bytes or (t.requires_grad and t.is_leaf)
                or getattr(t, "_axb_symm", None) is not None)
        if not skip and t.device.type == "cpu" and not isinstance(self.store, DiskStore):
            skip = True        # already in host memory
        if skip:
            return ("t", t)
        return ("h", self.store.put(t))

    def _unpack(self, packed):
        if packed[0] == "t":
            return packed[1]
        return self.store.get(packed[1])

    def __enter__(self):
        self._ctx = torch.autograd.graph.saved_tensors_hooks(self._pack, self._unpack)
        self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        return self._ctx.__exit__(*exc)


class LayerOffloader:
    """Frozen decoder-layer weights live in pinned host memory; a layer's weights are copied to the device on
    a side stream before the layer runs (forward, recomputation and backward) and dropped afterwards, with
    the next layer in the running direction requested one layer ahead. Trainable parameters stay put."""

    def __init__(self, model, device, ahead=1):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.layers = list(model.layers)
        self.ahead = ahead
        self.host, self.ready, self.resident, self.in_backward = [], {}, set(), set()
        for i, layer in enumerate(self.layers):
            entry = []
            for p in layer.parameters():
                if p.requires_grad or getattr(p, "_axb_shard", None) is not None:
                    continue
                h = torch.empty(p.shape, dtype=p.dtype, pin_memory=self.cuda)
                h.copy_(p.detach())
                entry.append((p, h))
                p.data = torch.empty(0, dtype=p.dtype, device=self.device)
            self.host.append(entry)
            layer.register_forward_pre_hook(lambda m, a, i=i: self._enter(i, +1))
            layer.register_forward_hook(lambda m, a, o, i=i: self._leave(i, False))
            layer.register_full_backward_pre_hook(lambda m, g, i=i: self._enter(i, -1))
        self.bytes_per_layer = [sum(h.numel() * h.element_size() for _, h in e) for e in self.host]

    def _fetch(self, i):
        if i < 0 or i >= len(self.layers) or i in self.resident:
            return
        self.resident.add(i)
        if self.cuda:
            with torch.cuda.stream(self.stream):
                for p, h in self.host[i]:
                    p.data = torch.empty(h.shape, dtype=h.dtype, device=self.device)
                    p.data.copy_(h, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
            self.ready[i] = ev
        else:
            for p, h in self.host[i]:
                p.data = h.clone()

    def _enter(self, i, direction):
        if direction < 0:
            if not self.in_backward:   # first layer of this backward pass: clean up when the pass is over
                torch.autograd.Variable._execution_engine.queue_callback(self._backward_done)
            self.in_backward.add(i)    # a recomputation inside the backward pass must not drop the weights
            # The backward pass of layer i+1 produced the gradients that triggered this call; its weights
            # are kept for one more layer, because nodes that only feed parameter gradients may still be
            # queued, and dropped when layer i-1 starts.
            if i + 2 < len(self.layers):
                self._leave(i + 2, True)
        self._fetch(i)
        ev = self.ready.pop(i, None)
        if ev is not None:
            cur = torch.cuda.current_stream(self.device)
            cur.wait_event(ev)
            for p, _ in self.host[i]:
                p.data.record_stream(cur)
        for k in range(1, self.ahead + 1):
            self._fetch(i + direction * k)

    def _leave(self, i, backward_done):
        if backward_done:
            self.in_backward.discard(i)
        elif i in self.in_backward:
            return
        if i not in self.resident:
            return
        self.resident.discard(i)
        self.ready.pop(i, None)
        for p, _ in self.host[i]:
            p.data = torch.empty(0, dtype=p.dtype, device=self.device)

    def _backward_done(self):
        for i in list(self.resident):
            self._leave(i, True)
        self.in_backward.clear()

    def materialize(self):
        """Puts every layer back on the device (saving, merging, evaluation without hooks)."""
        for i in range(len(self.layers)):
            self._fetch(i)
            ev = self.ready.pop(i, None)
            if ev is not None:
                ev.synchronize()
