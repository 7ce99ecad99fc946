"""Optimizers beyond the fused AdamW kernel, as plain ``torch.optim`` classes: ADOPT, Lion, and
the torch built-ins by name. (Reference: src/axolotl/utils/optimizers/adopt.py:39-539 and the
optimizer dispatch in src/axolotl/core/builders/base.py:292-484.)"""
from __future__ import annotations

import torch


class ADOPT(torch.optim.Optimizer):
    """ADOPT (Taniguchi et al. 2024): the second moment is updated AFTER it normalises the
    gradient, the normalised gradient is clipped by step**0.25, momentum is applied afterwards."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.9999), eps=1e-6, weight_decay=0.0, decouple=True, clip_exp=0.25):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, decouple=decouple,
                                      clip_exp=clip_exp))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad.float()
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                if g["weight_decay"] and g["decouple"]:
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                elif g["weight_decay"]:
                    grad = grad.add(p.float(), alpha=g["weight_decay"])
                if st["step"] == 0:
                    st["exp_avg_sq"].addcmul_(grad, grad)
                    st["step"] = 1
                    continue
                denom = st["exp_avg_sq"].sqrt().clamp_(min=g["eps"])
                normed = grad / denom
                if g["clip_exp"] is not None:
                    c = st["step"] ** g["clip_exp"]
                    normed.clamp_(-c, c)
                st["exp_avg"].lerp_(normed, 1 - b1)
                p.add_(st["exp_avg"].to(p.dtype), alpha=-g["lr"])
                st["exp_avg_sq"].mul_(b2).addcmul_(grad, grad, value=1 - b2)
                st["step"] += 1
        return loss


class Lion(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-4, betas=(0.9, 0.99), weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                grad = p.grad.float()
                p.mul_(1 - g["lr"] * g["weight_decay"])
                update = st["exp_avg"].mul(b1).add_(grad, alpha=1 - b1).sign_()
                p.add_(update.to(p.dtype), alpha=-g["lr"])
                st["exp_avg"].mul_(b2).add_(grad, alpha=1 - b2)
        return loss


class SinkGD(torch.optim.Optimizer):
    """Stateless multi-normalised gradient descent: the gradient of every matrix is alternately
    normalised by its row norms and column norms (``n_iters`` Sinkhorn-like sweeps, scaled so the
    result has unit-RMS rows and columns) and applied with a plain SGD step; vectors and scalars
    fall back to AdamW. No momentum buffers for matrices, i.e. optimizer memory close to zero.
    Reference: src/axolotl/utils/optimizers/sinkgd.py:240-1088 (SinkGD / SR-Sinkhorn)."""

    def __init__(self, params, lr=1e-3, n_iters=5, weight_decay=0.0, betas=(0.9, 0.999), eps=1e-8, sink_eps=1e-8):
        super().__init__(params, dict(lr=lr, n_iters=n_iters, weight_decay=weight_decay, betas=betas, eps=eps,
                                      sink_eps=sink_eps))

    @staticmethod
    def sinkhorn_normalize(g, n_iters=5, eps=1e-8):
        m, n = g.shape
        x = g.float()
        for _ in range(n_iters):
            x = x / (x.norm(dim=1, keepdim=True) + eps) * (n ** 0.5)
            x = x / (x.norm(dim=0, keepdim=True) + eps) * (m ** 0.5)
        return x

    def _fused_step(self, p, grp):
        """Scale-vector formulation on the device: the sweeps only update a [m] and b [n]; the
        matrix is read once per half-sweep and written once by the final update."""
        from ..ops import _lib

        m, n = p.shape
        st = self.state[p]
        if "sink_a" not in st:
            st["sink_a"] = torch.empty(m, dtype=torch.float32, device=p.device)
            st["sink_b"] = torch.empty(n, dtype=torch.float32, device=p.device)
        _lib.check_rc(_lib.cuda_lib().axb_sinkgd_step(
            p.data_ptr(), 0 if p.dtype == torch.float32 else 1, p.grad.data_ptr(), st["sink_a"].data_ptr(),
            st["sink_b"].data_ptr(), m, n, int(grp["n_iters"]), float(grp["lr"]), float(grp["weight_decay"]),
            float(grp["sink_eps"]), _lib.stream_ptr()), "sinkgd_step")

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for grp in self.param_groups:
            for p in grp["params"]:
                if p.grad is None:
                    continue
                if (p.is_cuda and p.dim() == 2 and min(p.shape) > 1 and p.grad.dtype == torch.float32
                        and p.grad.is_contiguous() and p.is_contiguous() and p.dtype in (torch.float32, torch.bfloat16)):
                    self._fused_step(p, grp)
                    continue
                if grp["weight_decay"]:
                    p.mul_(1 - grp["lr"] * grp["weight_decay"])
                if p.dim() == 2 and min(p.shape) > 1:
                    upd = self.sinkhorn_normalize(p.grad, grp["n_iters"], grp["sink_eps"])
                    p.add_(upd.to(p.dtype), alpha=-grp["lr"])
                    continue
                st = self.state[p]
                if not st:
                    st["step"], st["m"], st["v"] = 0, torch.zeros_like(p, dtype=torch.float32), torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
                b1, b2 = grp["betas"]
                g = p.grad.float()
                st["m"].mul_(b1).add_(g, alpha=1 - b1)
                st["v"].mul_(b2).addcmul_(g, g, value=1 - b2)
                mh = st["m"] / (1 - b1 ** st["step"])
                vh = st["v"] / (1 - b2 ** st["step"])
                p.add_((mh / (vh.sqrt() + grp["eps"])).to(p.dtype), alpha=-grp["lr"])
        return loss


def _matmul_nt(a, b):
    """a @ b^T: the tcgen05 GEMM for bf16 CUDA operands with 16-byte rows, torch elsewhere."""
    if a.is_cuda and a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and b.shape[0] % 8 == 0:
        from ..ops.gemm import gemm

        return gemm(a.contiguous(), b.contiguous())
    return a @ b.t()


def newton_schulz_orthogonalize(G, steps=5):
    """Quintic Newton-Schulz iteration that drives the singular values of ``G`` towards 1 (the
    matrix sign / polar factor used by Muon); runs in bf16 on CUDA, fp32 on CPU."""
    a, b, c = 3.4445, -4.7750, 2.0315
    X = G.to(torch.bfloat16) if G.is_cuda else G.float()
    transposed = X.shape[0] > X.shape[1]
    if transposed:
        X = X.t().contiguous()
    X = X / (X.float().norm() + 1e-7).to(X.dtype)
    for _ in range(steps):
        A = _matmul_nt(X, X)                       # X X^T  (symmetric)
        B = b * A + c * _matmul_nt(A, A)           # b A + c A^2
        X = a * X + _matmul_nt(B, X.t().contiguous())
    return (X.t() if transposed else X).to(G.dtype)


class Muon(torch.optim.Optimizer):
    """Muon (momentum orthogonalised by Newton-Schulz) for the hidden matrices, AdamW for everything
    else (embeddings, lm_head, norms, biases, adapter vectors). Update of a matrix:
    ``W <- W (1 - lr wd) - lr * 0.2 sqrt(max(m, n)) * NS(nesterov momentum)`` (the RMS-matched scaling
    that lets Muon share AdamW's learning rate)."""

    def __init__(self, params, lr=1e-3, momentum=0.95, nesterov=True, ns_steps=5, weight_decay=0.0, betas=(0.9, 0.95),
                 eps=1e-8, adamw_names=("embed_tokens", "lm_head")):
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                                      weight_decay=weight_decay, betas=betas, eps=eps))
        self.adamw_ids = set()

    def mark_adamw(self, params):
        self.adamw_ids.update(id(p) for p in params)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for grp in self.param_groups:
            lr, wd = grp["lr"], grp["weight_decay"]
            for p in grp["params"]:
                if p.grad is None:
                    continue
                g = p.grad.float()
                st = self.state[p]
                if p.dim() == 2 and min(p.shape) > 1 and id(p) not in self.adamw_ids:
                    if not st:
                        st["momentum"] = torch.zeros_like(g)
                    buf = st["momentum"].mul_(grp["momentum"]).add_(g)
                    upd = g.add(buf, alpha=grp["momentum"]) if grp["nesterov"] else buf
                    o = newton_schulz_orthogonalize(upd, grp["ns_steps"]).float()
                    if wd:
                        p.mul_(1 - lr * wd)
                    p.add_(o.to(p.dtype), alpha=-lr * 0.2 * max(p.shape) ** 0.5)
                    continue
                if not st:
                    st["step"], st["m"], st["v"] = 0, torch.zeros_like(g), torch.zeros_like(g)
                st["step"] += 1
                b1, b2 = grp["betas"]
                st["m"].mul_(b1).add_(g, alpha=1 - b1)
                st["v"].mul_(b2).addcmul_(g, g, value=1 - b2)
                mh, vh = st["m"] / (1 - b1 ** st["step"]), st["v"] / (1 - b2 ** st["step"])
                if wd:
                    p.mul_(1 - lr * wd)
                p.add_((mh / (vh.sqrt() + grp["eps"])).to(p.dtype), alpha=-lr)
        return loss


class CAME(torch.optim.Optimizer):
    """CAME (confidence-guided adaptive memory-efficient optimisation, Luo et al. 2023): Adafactor-style
    factored second moments plus a factored "instability" statistic that damps updates the momentum
    disagrees with. Memory per matrix: one momentum tensor and four vectors."""

    def __init__(self, params, lr=2e-4, betas=(0.9, 0.999, 0.9999), eps=(1e-30, 1e-16), clip_threshold=1.0,
                 weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, clip_threshold=clip_threshold,
                                      weight_decay=weight_decay))

    @staticmethod
    def _approx(row, col):
        r = (row / row.mean(-1, keepdim=True)).rsqrt().unsqueeze(-1)
        return r * col.rsqrt().unsqueeze(-2)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for grp in self.param_groups:
            b1, b2, b3 = grp["betas"]
            e1, e2 = grp["eps"]
            for p in grp["params"]:
                if p.grad is None:
                    continue
                g = p.grad.float()
                st = self.state[p]
                factored = g.dim() >= 2
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(g)
                    if factored:
                        st["row"], st["col"] = g.new_zeros(g.shape[:-1]), g.new_zeros(g.shape[:-2] + g.shape[-1:])
                        st["res_row"], st["res_col"] = torch.zeros_like(st["row"]), torch.zeros_like(st["col"])
                    else:
                        st["sq"] = torch.zeros_like(g)
                st["step"] += 1
                upd = g * g + e1
                if factored:
                    st["row"].mul_(b2).add_(upd.mean(-1), alpha=1 - b2)
                    st["col"].mul_(b2).add_(upd.mean(-2), alpha=1 - b2)
                    u = self._approx(st["row"], st["col"]) * g
                else:
                    st["sq"].mul_(b2).add_(upd, alpha=1 - b2)
                    u = st["sq"].rsqrt() * g
                rms = u.norm() / (u.numel() ** 0.5)
                u = u / (rms / grp["clip_threshold"]).clamp(min=1.0)
                m = st["exp_avg"].mul_(b1).add_(u, alpha=1 - b1)
                if factored:
                    res = (u - m) ** 2 + e2
                    st["res_row"].mul_(b3).add_(res.mean(-1), alpha=1 - b3)
                    st["res_col"].mul_(b3).add_(res.mean(-2), alpha=1 - b3)
                    out = self._approx(st["res_row"], st["res_col"]) * m
                else:
                    out = m
                if grp["weight_decay"]:
                    p.mul_(1 - grp["lr"] * grp["weight_decay"])
                p.add_(out.to(p.dtype), alpha=-grp["lr"])
        return loss


def build_torch_optimizer(name, params, lr, betas, eps, cfg=None):
    name = name.lower()
    args = {}
    oa = (cfg or {}).get("optim_args")
    if isinstance(oa, dict):
        args = dict(oa)
    elif isinstance(oa, str) and oa:
        for kv in oa.split(","):
            k, _, v = kv.partition("=")
            try:
                args[k.strip()] = float(v)
            except ValueError:
                args[k.strip()] = v.strip()
    if name in ("sgd",):
        return torch.optim.SGD(params, lr=lr, momentum=args.pop("momentum", 0.0), **args)
    if name in ("adagrad",):
        return torch.optim.Adagrad(params, lr=lr, **args)
    if name in ("adafactor",):
        return torch.optim.Adafactor(params, lr=lr, **args)
    if name in ("rmsprop",):
        return torch.optim.RMSprop(params, lr=lr, **args)
    if name in ("adam",):
        return torch.optim.Adam(params, lr=lr, betas=betas, eps=eps, **args)
    if name in ("adopt_adamw", "adopt"):
        return ADOPT(params, lr=lr, betas=(betas[0], args.pop("beta2", 0.9999)), eps=args.pop("eps", 1e-6), **args)
    if name in ("lion_pytorch", "lion", "lion_32bit"):
        return Lion(params, lr=lr, betas=(betas[0], args.pop("beta2", 0.99)), **args)
    if name in ("sinkgd", "sinkgd_triton", "dist_sinkgd"):
        return SinkGD(params, lr=lr, n_iters=int(args.pop("n_iters", args.pop("num_iters", 5))), betas=betas, eps=eps, **args)
    if name in ("muon",):
        return Muon(params, lr=lr, momentum=args.pop("momentum", 0.95), ns_steps=int(args.pop("ns_steps", 5)),
                    betas=(betas[0], args.pop("beta2", 0.95)), eps=eps, **args)
    if name in ("came_pytorch", "came"):
        return CAME(params, lr=lr, betas=(betas[0], args.pop("beta2", 0.999), args.pop("beta3", 0.9999)), **args)
    raise ValueError(f"optimizer '{name}' is not available on axolotl_b200")
