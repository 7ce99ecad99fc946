"""Parallel runtime: glues the mesh, the sharded weights and the fused gradient/optimizer kernel
to the trainer. Two communication back ends share one interface:

* ``fused`` (CUDA, default): symmetric-memory buffers, weights gathered inside the GEMM kernel,
  gradients reduced + clipped + AdamW-updated + re-published by ONE kernel (``axb_rs_adamw_ag``).
* ``collective`` (any device; gloo on CPU, NCCL on GPU): weights replicated, flat gradient
  all-reduced with ``torch.distributed``; used for host-side plumbing tests and as a baseline.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import _lib
from ..utils.logging import get_logger
from .mesh import DeviceMesh, MeshSpec

LOG = get_logger(__name__)


class ParallelRuntime:
    def __init__(self, mesh: DeviceMesh, device, backend="fused"):
        self.mesh, self.device, self.backend = mesh, torch.device(device), backend
        self.rank = dist.get_rank()
        self.world_size = dist.get_world_size()
        self.dp_group = mesh.group("ep", "dp_replicate", "dp_shard") if mesh.size("ep", "dp_replicate", "dp_shard") > 1 else None
        self.dp_size = mesh.size("ep", "dp_replicate", "dp_shard")
        ranks = mesh.ranks("ep", "dp_replicate", "dp_shard")
        self.dp_rank = ranks.index(self.rank) if self.rank in ranks else 0
        self.shard_group = mesh.group("dp_shard")
        self.shard_size = mesh.size("dp_shard")
        self.fsdp = None
        self.sync = None
        self.opt = None
        self._symm = []
        self.cp = None
        self.tp = None
        self.ep = None
        self.reduce_group = self.dp_group   # group over which gradients are reduced
        self.reduce_size = self.dp_size
        self.mp_group = None                # tensor- or expert-parallel group
        self.dp_rest_group, self.dp_rest_size = self.dp_group, self.dp_size

    # ------------------------------------------------------------------ setup
    def shard_model(self, model):
        self.setup_ep(model)
        if self.backend != "fused" or self.shard_size <= 1:
            return
        from .fsdp import FSDPContext

        self.fsdp = FSDPContext(self.device, self.shard_group, self.shard_size, self.mesh.coord("dp_shard"),
                                reshard_after_forward=getattr(self, "reshard_after_forward", True))
        self.fsdp.shard_model(model)

    def symmetric_alloc(self, numel, dtype):
        """Allocator handed to FlatAdamW so gradients / masters / shadows live in peer-mapped memory."""
        from .symm import SymmBuffer

        buf = SymmBuffer(numel, dtype, self.device, self.reduce_group, use_multicast=os.environ.get("AXB_NO_MULTIMEM") != "1")
        self._symm.append(buf)
        t = buf.tensor
        t._axb_symm = buf
        return t

    def optimizer_alloc(self):
        if self.tp is not None or self.mesh.size("ep") > 1:
            return None
        if self.backend == "fused" and self.reduce_size > 1 and self.device.type == "cuda":
            return self.symmetric_alloc
        return None

    def moment_shard(self):
        """(rank, world) for FlatAdamW(moment_shard=...) when the fused reduce-scatter/AdamW/all-gather
        kernel steps the optimizer (each rank then stores 1/world of the AdamW moments), else None."""
        if self.tp is None and self.mesh.size("ep") == 1 and self.backend == "fused" and self.reduce_size > 1 \
                and self.device.type == "cuda":
            return (dist.get_rank(self.reduce_group), self.reduce_size)
        return None

    def attach_optimizer(self, opt):
        self.opt = opt
        if self.tp is None and self.mesh.size("ep") == 1 and self.backend == "fused" and self.reduce_size > 1 \
                and self.device.type == "cuda":
            from .symm import PeerSync

            self.sync = PeerSync(self.device, self.reduce_group)
            for g in opt.groups:
                if getattr(g["grad"], "_axb_symm", None) is None:
                    raise RuntimeError("FlatAdamW must be built with alloc=parallel.optimizer_alloc() for the fused backend")
            self._scratch = self.symmetric_alloc(64, torch.float32)
            self._gnorm = torch.zeros(1, dtype=torch.float32, device=self.device)
            dist.barrier(self.reduce_group)

    # ------------------------------------------------------------------ trainer interface
    def before_micro_batch(self, last):
        pass

    def after_optimizer_step(self):
        if self.fsdp is not None:
            self.fsdp.end_of_step()

    def barrier(self):
        if self.world_size > 1:
            dist.barrier()

    def mean_scalar(self, v):
        t = torch.tensor([float(v)], dtype=torch.float64, device=self.device)
        dist.all_reduce(t)
        return float(t.item()) / self.world_size

    def min_scalar(self, v):
        t = torch.tensor([float(v)], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return float(t.item())

    @torch.no_grad()
    def materialize_full_weights(self, model):
        """Replaces every sharded weight by its gathered full tensor (checkpoint saving / merging)."""
        if self.fsdp is None:
            return
        for m in list(self.fsdp.sharded):
            full = self.fsdp.gather_full_weight(m)
            m.weight = torch.nn.Parameter(full, requires_grad=False)
        self.fsdp.sharded = []

    def sum_scalar(self, v):
        t = torch.tensor([float(v)], dtype=torch.float64, device=self.device)
        dist.all_reduce(t)
        r = float(t.item())
        return int(r) if isinstance(v, int) else r

    # ------------------------------------------------------------------ expert parallel
    def setup_ep(self, model):
        """Shards the experts of every MoE block over the ep axis (call after adapters exist)."""
        n = self.mesh.size("ep")
        if n <= 1 or self.ep is not None:
            return
        from .ep import ExpertParallelGroup

        self.ep = ExpertParallelGroup(self.device, self.mesh.group("ep"), n, self.mesh.coord("ep"),
                                      model.config.num_experts)
        self.ep.shard_experts(model)
        self.mp_group = self.mesh.group("ep")
        self.dp_rest_group = self.mesh.group("dp_replicate", "dp_shard")
        self.dp_rest_size = self.mesh.size("dp_replicate", "dp_shard")

    # ------------------------------------------------------------------ context parallel
    def setup_cp(self):
        n = self.mesh.size("cp")
        if n <= 1 or self.cp is not None:
            return
        from .cp import CPContext

        self.cp = CPContext(self.device, self.mesh.group("cp"), n, self.mesh.coord("cp"))
        # gradients are SUMMED over cp ranks (each holds a slice of the same sequence) and averaged
        # over data-parallel ranks: reduce over dp x cp, scale by 1 / dp
        self.reduce_group = self.mesh.group("dp_shard", "cp") if self.mesh.size("dp_replicate") * self.mesh.size("ep") == 1 \
            else dist.group.WORLD
        self.reduce_size = self.dp_size * n

    # ------------------------------------------------------------------ tensor parallel
    def apply_tp(self, model):
        self.setup_cp()
        n = self.mesh.size("tp")
        if n <= 1:
            return
        from .tp import TPContext, apply_tensor_parallel

        cfg = model.config
        max_elems = getattr(self, "tp_max_tokens", 16384) * max(cfg.hidden_size, 1)
        self.tp = TPContext(self.device, self.mesh.group("tp"), n, self.mesh.coord("tp"), max_elems)
        apply_tensor_parallel(model, self.tp)
        self.mp_group = self.tp.group
        self.dp_rest_group = self.dp_group
        self.dp_rest_size = self.dp_size

    def _tp_step(self, opt, lr):
        """Model-parallel (TP or EP) x CP x DP: sum the gradients of replicated parameters over the
        model-parallel group, sum everything over the context-parallel group and over the remaining
        data-parallel ranks, scale by 1 / data_parallel_size; global norm = replicated part + sum over the model-parallel group of
        the sharded part. Everything stays on the device."""
        from ..ops.optim import grad_sumsq

        opt._fold_autograd_grads()
        tp_group = self.mp_group
        cp_group = self.mesh.group("cp") if self.cp is not None else None
        total = torch.zeros(1, dtype=torch.float32, device=self.device)
        for g in opt.groups:
            split = g["tp_split"]
            if split > 0:
                dist.all_reduce(g["grad"][:split], group=tp_group)
            if cp_group is not None:
                # every cp rank saw another slice of the same sequences: their gradients add up
                dist.all_reduce(g["grad"], group=cp_group)
            if self.dp_rest_size > 1:
                dist.all_reduce(g["grad"], group=self.dp_rest_group)
            grad_sumsq(g["grad"][:split], total) if split > 0 else None
            if split < g["grad"].numel():
                sh = grad_sumsq(g["grad"][split:])
                dist.all_reduce(sh, group=tp_group)
                total += sh
        opt.grad_scale = 1.0 / self.dp_size
        return opt.step(lr=lr, gnorm_sq=total)

    def optimizer_step(self, opt, lr):
        """Gradient synchronisation + clipping + optimizer update. Returns the squared global
        gradient norm (device scalar) or None."""
        if self.ep is not None and self.ep.take_overflow():
            return None      # rows were dropped in a layer call: no update from these gradients (the caller zeroes them)
        if self.tp is not None or self.ep is not None:
            return self._tp_step(opt, lr)
        if self.reduce_size <= 1:
            return opt.step(lr=lr)
        if self.backend == "fused" and self.sync is not None:
            return self._fused_step(opt, lr)
        # collective back end: sum the flat gradients, scale by 1 / dp, then a local fused AdamW
        for g in opt.flat_grads():
            dist.all_reduce(g, group=self.reduce_group)
        opt.grad_scale = 1.0 / self.dp_size
        return opt.step(lr=lr)

    def _fused_step(self, opt, lr):
        lib = _lib.cuda_lib()
        from .symm import WAIT_BUDGET_NS

        opt._fold_autograd_grads()
        opt.step_count += 1
        bc1 = 1.0 - opt.betas[0] ** opt.step_count
        bc2 = 1.0 - opt.betas[1] ** opt.step_count
        rank = dist.get_rank(self.reduce_group)
        sliced = 1 if opt.moment_shard is not None else 0
        groups = [g for g in opt.groups if g.get("active", True)]
        # One group: reduce + clip + update in a single launch. Several groups (weight decay on
        # matrices only, LoRA+, embedding LR, lr_groups): the clip factor needs the norm over ALL
        # groups, so every group is reduced first (pass 1 adds its squared norm to _gnorm) and
        # updated afterwards (pass 2 clips by the accumulated norm).
        passes = (0,) if len(groups) == 1 else (1, 2)
        if len(groups) > 1:
            self._gnorm.zero_()
        for mode in passes:
            for g in groups:
                gb, sb = g["grad"]._axb_symm, g["shadow"]._axb_symm
                if g.get("master_local"):
                    from .symm import _u64_array

                    m_ptrs, m_mc = _u64_array([g["master"].data_ptr()] * self.reduce_size), None
                    flags = sliced | 2
                else:
                    mb = g["master"]._axb_symm
                    m_ptrs, m_mc, flags = mb.ptrs_c, mb.multicast_ptr or None, sliced
                epoch = self.sync.next_epoch(0, 3)
                rc = lib.axb_rs_adamw_ag_pass(
                    gb.ptrs_c, m_ptrs, sb.ptrs_c, self.sync.buf.pad_ptrs_c, self._scratch._axb_symm.ptrs_c,
                    gb.multicast_ptr or None, m_mc, sb.multicast_ptr or None,
                    g["exp_avg"].data_ptr(), g["exp_avg_sq"].data_ptr(), g["grad"].numel(), rank, self.reduce_size,
                    epoch, lr * g["lr_scale"], opt.betas[0], opt.betas[1], opt.eps, g["weight_decay"], bc1, bc2,
                    float(opt.max_grad_norm or 0.0), 1.0 / self.dp_size,
                    self._gnorm.data_ptr(), _lib.status_word(self.device).data_ptr(), WAIT_BUDGET_NS, _lib.stream_ptr(),
                    flags, mode)
                _lib.check_rc(rc, "rs_adamw_ag")
        for g in opt.groups:   # inactive groups (LISA) keep their weights; their gradients are dropped
            if not g.get("active", True):
                g["grad"].zero_()
        opt.skip_zero_grad_once = True  # the kernel already cleared the gradient buffers
        return self._gnorm


def init_distributed(backend=None, timeout_s=None):
    """Process-group bring-up from the torchrun environment (RANK / WORLD_SIZE / MASTER_*)."""
    import datetime

    if dist.is_initialized():
        return
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    t = timeout_s or int(os.environ.get("AXOLOTL_NCCL_TIMEOUT", "1800"))
    kw = {}
    if backend == "nccl":
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(dev)
        kw["device_id"] = dev
    dist.init_process_group(backend, timeout=datetime.timedelta(seconds=t), **kw)


def create_runtime(*, device, dp_shard=None, dp_replicate=1, tp=1, cp=1, ep=1, backend=None):
    """Mesh + runtime for an already initialised process group (no model changes yet). Call
    ``apply_tp(model)`` before adapters are injected and ``shard_model(model)`` afterwards."""
    world = dist.get_world_size()
    spec = MeshSpec.from_cfg(world, tensor_parallel_size=tp, context_parallel_size=cp, dp_shard_size=dp_shard,
                             dp_replicate_size=dp_replicate, expert_parallel_size=ep)
    device = torch.device(device)
    if backend is None:
        backend = os.environ.get("AXB_COMM", "fused" if device.type == "cuda" else "collective")
    return ParallelRuntime(DeviceMesh(spec, dist.get_rank()), device, backend)


def build_parallel(model, *, device, dp_shard=None, dp_replicate=1, tp=1, cp=1, ep=1, backend=None,
                   reshard_after_forward=True):
    """Creates the mesh + runtime for an already initialised process group and shards the model."""
    if tp > 1 or cp > 1 or ep > 1:
        rt = create_runtime(device=device, dp_shard=dp_shard, dp_replicate=dp_replicate, tp=tp, cp=cp, ep=ep,
                            backend=backend)
        rt.reshard_after_forward = reshard_after_forward
        rt.apply_tp(model)
        rt.shard_model(model)
        return rt
    world = dist.get_world_size()
    spec = MeshSpec.from_cfg(world, tensor_parallel_size=tp, context_parallel_size=cp, dp_shard_size=dp_shard,
                             dp_replicate_size=dp_replicate, expert_parallel_size=ep)
    device = torch.device(device)
    if backend is None:
        backend = os.environ.get("AXB_COMM", "fused" if device.type == "cuda" else "collective")
    mesh = DeviceMesh(spec, dist.get_rank())
    rt = ParallelRuntime(mesh, device, backend)
    rt.reshard_after_forward = reshard_after_forward
    rt.setup_cp()
    rt.shard_model(model)
    return rt
