"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _check_status():
    from axolotl_b200.ops import _lib
    _lib.check_status()


@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (1000, 776, 328), (128, 64, 64), (2048, 4096, 1024), (77, 24, 40)])
@pytest.mark.parametrize("bn", [None, 64, 128, 256])
def test_gemm_tn(M, N, K, bn):
    from axolotl_b200.ops.gemm import gemm
    torch.manual_seed(0)
    a = torch.randn(M, K, device=_dev(), dtype=torch.bfloat16)
    b = torch.randn(N, K, device=_dev(), dtype=torch.bfloat16)
    c = gemm(a, b, bn=bn)
    _check_status()
    ref = a.float() @ b.float().t()
    assert _rel_err(c, ref) < 5e-3


@pytest.mark.parametrize("ta,tb", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(512, 768, 640), (192, 136, 200)])
def test_gemm_transposed_operands(ta, tb, M, N, K):
    from axolotl_b200.ops.gemm import gemm
    torch.manual_seed(1)
    a = torch.randn((K, M) if ta else (M, K), device=_dev(), dtype=torch.bfloat16)
    b = torch.randn((K, N) if tb else (N, K), device=_dev(), dtype=torch.bfloat16)
    for bn in (64, 128, 256):
        c = gemm(a, b, trans_a=ta, trans_b=tb, bn=bn, out_dtype=torch.float32)
        _check_status()
        ref = (a.float().t() if ta else a.float()) @ (b.float() if tb else b.float().t())
        assert _rel_err(c, ref) < 5e-3, (ta, tb, bn)


@pytest.mark.parametrize("M,N,K", [(4096, 5000, 512), (2304, 8192 + 24, 256), (5000, 4096, 192)])
def test_pair_gemm_tma_store_epilogue_matches_row_stores(M, N, K):
    """Large bf16 GEMMs leave the CTA-pair kernel through staged TMA tile stores; ragged M / N edges are
    clipped by the tensor map. Same result as the per-thread row stores, bit for bit."""
    from axolotl_b200.ops import _lib
    from axolotl_b200.ops.gemm import _use_pair, gemm
    torch.manual_seed(21)
    lib = _lib.cuda_lib()
    assert _use_pair(M, N, 256)
    a = torch.randn(M, K, device=_dev(), dtype=torch.bfloat16)
    b = torch.randn(N, K, device=_dev(), dtype=torch.bfloat16)
    guard = torch.full((M + 8, N + 8), 7.0, device=_dev(), dtype=torch.bfloat16)
    out = guard[:M, :N]                       # a view with ld = N + 8: rows stay 16-byte aligned
    try:
        lib.axb_gemm_set_pair_tuning(0, 1, 0)
        gemm(a, b, out=out, bn=256)
        _check_status()
        lib.axb_gemm_set_pair_tuning(3, 0, 0)
        ref_rows = gemm(a, b, bn=256)
        _check_status()
    finally:
        lib.axb_gemm_set_pair_tuning(0, 1, 0)
    assert torch.equal(out, ref_rows)
    assert _rel_err(out, a.float() @ b.float().t()) < 5e-3
    assert bool((guard[M:, :] == 7.0).all()) and bool((guard[:, N:] == 7.0).all())   # nothing beyond the edges


def test_gemm_k_extension_and_epilogue():
    from axolotl_b200.ops.gemm import gemm
    torch.manual_seed(2)
    M, N, K, R = 640, 1024, 512, 48
    a = torch.randn(M, K, device=_dev(), dtype=torch.bfloat16)
    b = torch.randn(N, K, device=_dev(), dtype=torch.bfloat16)
    a2 = torch.randn(M, R, device=_dev(), dtype=torch.bfloat16)
    b2 = torch.randn(N, R, device=_dev(), dtype=torch.bfloat16)
    cin = torch.randn(M, N, device=_dev(), dtype=torch.bfloat16)
    c = gemm(a, b, a2=a2, b2=b2, alpha=0.5, beta=2.0, c_in=cin)
    _check_status()
    ref = 0.5 * (a.float() @ b.float().t() + a2.float() @ b2.float().t()) + 2.0 * cin.float()
    assert _rel_err(c, ref) < 5e-3
    # transposed-B form with an extension (the dX GEMM of a LoRA layer)
    w = torch.randn(K, N, device=_dev(), dtype=torch.bfloat16)   # stored [Kred, N]
    e = torch.randn(R, N, device=_dev(), dtype=torch.bfloat16)
    c2 = gemm(a, w, trans_b=True, a2=a2, b2=e)
    _check_status()
    ref2 = a.float() @ w.float() + a2.float() @ e.float()
    assert _rel_err(c2, ref2) < 5e-3


def test_gemm_splitk_accumulate():
    from axolotl_b200.ops.gemm import gemm
    torch.manual_seed(3)
    T, R, K = 4096, 48, 1024
    t = torch.randn(T, R, device=_dev(), dtype=torch.bfloat16)
    x = torch.randn(T, K, device=_dev(), dtype=torch.bfloat16)
    out = torch.ones(R, K, device=_dev(), dtype=torch.float32)
    gemm(t, x, trans_a=True, trans_b=True, out=out, accumulate=True, splits=8)
    _check_status()
    ref = 1.0 + t.float().t() @ x.float()
    assert _rel_err(out, ref) < 5e-3


def test_rmsnorm_fwd_bwd():
    from axolotl_b200.ops.functional import add_rmsnorm
    torch.manual_seed(4)
    T, H = 300, 1024
    x = torch.randn(T, H, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(T, H, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(H, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    y, h = add_rmsnorm(x, r, w, 1e-5)
    gy, gh = torch.randn_like(y), torch.randn_like(h)
    (y.float() * gy.float()).sum().add((h.float() * gh.float()).sum()).backward()
    xc, rc, wc = [t.detach().cpu().float().requires_grad_(True) for t in (x, r, w)]
    hc = (xc + rc).bfloat16().float() + 0 * (xc + rc)  # value rounded like the kernel
    hc = xc + rc
    yc = hc * torch.rsqrt(hc.pow(2).mean(-1, keepdim=True) + 1e-5) * wc
    (yc * gy.cpu().float()).sum().add((hc * gh.cpu().float()).sum()).backward()
    assert _rel_err(y.cpu(), yc) < 1e-2
    assert _rel_err(x.grad.cpu(), xc.grad) < 2e-2
    assert _rel_err(r.grad.cpu(), rc.grad) < 2e-2
    assert _rel_err(w.grad.cpu(), wc.grad) < 2e-2


@pytest.mark.parametrize("with_norm", [False, True])
def test_rope_fwd_bwd(with_norm):
    from axolotl_b200.ops.functional import rope_qk_
    torch.manual_seed(5)
    T, Hq, Hk, D = 200, 8, 2, 128
    base = torch.randn(T, (Hq + 2 * Hk) * D, device=_dev(), dtype=torch.bfloat16)
    pos = torch.arange(T, device=_dev(), dtype=torch.int32) % 77
    inv = (1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))).to(_dev())
    qn = torch.randn(D, device=_dev(), dtype=torch.bfloat16, requires_grad=True) if with_norm else None
    kn = torch.randn(D, device=_dev(), dtype=torch.bfloat16, requires_grad=True) if with_norm else None
    x = base.clone().requires_grad_(True)
    y = rope_qk_(x * 1.0, pos, inv, Hq, Hk, D, 1.0, qn, kn, 1e-6)
    g = torch.randn_like(y)
    (y.float() * g.float()).sum().backward()
    xc = base.cpu().clone().requires_grad_(True)
    qnc = qn.detach().cpu().requires_grad_(True) if with_norm else None
    knc = kn.detach().cpu().requires_grad_(True) if with_norm else None
    yc = rope_qk_(xc * 1.0, pos.cpu(), inv.cpu(), Hq, Hk, D, 1.0, qnc, knc, 1e-6)
    (yc.float() * g.cpu().float()).sum().backward()
    assert _rel_err(y.cpu(), yc) < 1e-2
    assert _rel_err(x.grad.cpu(), xc.grad) < 2e-2
    if with_norm:
        assert _rel_err(qn.grad.cpu(), qnc.grad) < 3e-2
        assert _rel_err(kn.grad.cpu(), knc.grad) < 3e-2


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
def test_glu(act):
    from axolotl_b200.ops.functional import glu
    torch.manual_seed(6)
    gu = torch.randn(130, 2 * 344 * 2, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    h = glu(gu, act)
    g = torch.randn_like(h)
    (h.float() * g.float()).sum().backward()
    guc = gu.detach().cpu().float().requires_grad_(True)
    hc = glu(guc, act)
    (hc * g.cpu().float()).sum().backward()
    assert _rel_err(h.cpu(), hc) < 1e-2
    assert _rel_err(gu.grad.cpu(), guc.grad) < 2e-2


def test_embedding():
    from axolotl_b200.ops.functional import embedding
    torch.manual_seed(7)
    tab = torch.randn(1000, 256, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, 1000, (3, 50), device=_dev())
    out = embedding(tab, ids)
    assert torch.equal(out, tab.detach()[ids])
    out.float().sum().backward()
    ref = torch.zeros(1000, 256)
    ref.index_add_(0, ids.cpu().reshape(-1), torch.ones(150, 256))
    assert _rel_err(tab.grad.cpu(), ref) < 1e-3


@pytest.mark.parametrize("D,Hq,Hk", [(128, 4, 2), (64, 4, 2), (128, 8, 8), (128, 8, 1)])
@pytest.mark.parametrize("lens", [[128], [200, 57, 300], [1, 129, 640, 31], [1024, 513]])
def test_flash_varlen_fwd_bwd(D, Hq, Hk, lens):
    from axolotl_b200.ops.functional import AttnMeta, flash_varlen
    torch.manual_seed(8)
    cu = [0]
    for l in lens:
        cu.append(cu[-1] + l)
    T = cu[-1]
    base = (torch.randn(T, (Hq + 2 * Hk) * D, dtype=torch.float32) * 0.5).bfloat16()
    meta = AttnMeta(cu, _dev())
    x = base.to(_dev()).requires_grad_(True)
    out = flash_varlen(x, meta, Hq, Hk, D)
    _check_status()
    g = (torch.randn(T, Hq * D) * 0.5).bfloat16()
    (out.float() * g.to(_dev()).float()).sum().backward()
    _check_status()
    xc = base.float().requires_grad_(True)
    meta_c = AttnMeta(cu, "cpu")
    outc = flash_varlen(xc, meta_c, Hq, Hk, D)
    (outc * g.float()).sum().backward()
    assert _rel_err(out.cpu(), outc) < 1e-2
    q_end, k_end = Hq * D, (Hq + Hk) * D
    gx, gc = x.grad.cpu().float(), xc.grad
    assert _rel_err(gx[:, :q_end], gc[:, :q_end]) < 2e-2, "dq"
    assert _rel_err(gx[:, q_end:k_end], gc[:, q_end:k_end]) < 2e-2, "dk"
    assert _rel_err(gx[:, k_end:], gc[:, k_end:]) < 2e-2, "dv"


@pytest.mark.parametrize("D,Dv,Hq,Hk,softcap,window,causal", [
    (256, 256, 4, 2, 0.0, 0, True), (256, 256, 2, 1, 20.0, 0, True), (256, 256, 2, 2, 0.0, 100, True),
    (192, 128, 4, 4, 0.0, 0, True), (192, 128, 4, 2, 0.0, 0, False), (256, 256, 2, 1, 0.0, 0, False)])
@pytest.mark.parametrize("lens", [[128], [200, 57, 300], [1, 129, 640, 31]])
def test_flash_wide_heads_fwd_bwd(D, Dv, Hq, Hk, softcap, window, causal, lens):
    """Head widths 256 (Gemma) and 192/128 (latent attention), tanh soft cap, sliding window, bidirectional
    documents: the wide tcgen05 kernels against per-document fp32 attention."""
    from axolotl_b200.ops.functional import AttnMeta, flash_varlen
    torch.manual_seed(18)
    cu = [0]
    for l in lens:
        cu.append(cu[-1] + l)
    T = cu[-1]
    width = Hq * D + Hk * D + Hk * Dv
    base = (torch.randn(T, width, dtype=torch.float32) * 0.5).bfloat16()
    meta = AttnMeta(cu, _dev(), causal, window or None)
    x = base.to(_dev()).requires_grad_(True)
    out = flash_varlen(x, meta, Hq, Hk, D, Dv=Dv, softcap=softcap)
    _check_status()
    g = (torch.randn(T, Hq * Dv) * 0.5).bfloat16()
    (out.float() * g.to(_dev()).float()).sum().backward()
    _check_status()
    xc = base.float().requires_grad_(True)
    outc = flash_varlen(xc, AttnMeta(cu, "cpu", causal, window or None), Hq, Hk, D, Dv=Dv, softcap=softcap)
    (outc * g.float()).sum().backward()
    assert _rel_err(out.cpu(), outc) < 1e-2
    q_end, k_end = Hq * D, (Hq + Hk) * D
    gx, gc = x.grad.cpu().float(), xc.grad
    assert _rel_err(gx[:, :q_end], gc[:, :q_end]) < 2e-2, "dq"
    assert _rel_err(gx[:, q_end:k_end], gc[:, q_end:k_end]) < 2e-2, "dk"
    assert _rel_err(gx[:, k_end:], gc[:, k_end:]) < 2e-2, "dv"


def test_linear_cross_entropy():
    from axolotl_b200.ops.functional import linear_cross_entropy
    torch.manual_seed(9)
    T, H, V = 700, 256, 3001 + 7
    V = 3008
    h = (torch.randn(T, H) * 0.5).bfloat16().to(_dev()).requires_grad_(True)
    w = (torch.randn(V, H) * 0.05).bfloat16().to(_dev())
    labels = torch.randint(0, V, (T,), device=_dev())
    labels[::7] = -100
    loss = linear_cross_entropy(h, w, labels, chunk_rows=256)
    loss.backward()
    hc = h.detach().cpu().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(hc @ w.cpu().float().t(), labels.cpu(), ignore_index=-100)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-2 * abs(ref.item())
    assert _rel_err(h.grad.cpu(), hc.grad) < 3e-2


def test_lora_linear_fused():
    from axolotl_b200.ops.lora import lora_linear
    torch.manual_seed(10)
    T, K, r = 512, 384, 16
    outs = [256, 128, 128]
    N, R = sum(outs), r * len(outs)
    x = (torch.randn(T, K) * 0.5).bfloat16().to(_dev()).requires_grad_(True)
    W = (torch.randn(N, K) * 0.05).bfloat16().to(_dev())
    A = (torch.randn(R, K) * 0.05).to(_dev()).requires_grad_(True)
    B = torch.zeros(N, R, device=_dev())
    blocks, row0 = [], 0
    for i, o in enumerate(outs):
        B[row0:row0 + o, i * r:(i + 1) * r] = torch.randn(o, r, device=_dev()) * 0.05
        blocks.append((row0, o, i * r, r))
        row0 += o
    B.requires_grad_(True)
    y = lora_linear(x, W, A, B, A.detach().bfloat16(), B.detach().bfloat16(), 2.0, tuple(blocks))
    g = torch.randn_like(y)
    (y.float() * g.float()).sum().backward()
    xc = x.detach().cpu().float().requires_grad_(True)
    Ac = A.detach().cpu().bfloat16().float().requires_grad_(True)
    Bc = B.detach().cpu().bfloat16().float().requires_grad_(True)
    yc = xc @ W.cpu().float().t() + 2.0 * (xc @ Ac.t()) @ Bc.t()
    (yc * g.cpu().float()).sum().backward()
    mask = (B.detach().cpu() != 0).float()
    assert _rel_err(y.cpu(), yc) < 1e-2
    assert _rel_err(x.grad.cpu(), xc.grad) < 2e-2
    assert _rel_err(A.grad.cpu(), Ac.grad) < 2e-2
    assert _rel_err(B.grad.cpu(), Bc.grad * mask) < 2e-2


def test_adamw_matches_torch():
    from axolotl_b200.ops.optim import adamw_step_, grad_sumsq
    torch.manual_seed(11)
    n = 10007
    p = torch.randn(n, device=_dev())
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, weight_decay=0.1, eps=1e-8)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    shadow = torch.empty(n, device=_dev(), dtype=torch.bfloat16)
    for step in range(1, 4):
        g = torch.randn(n, device=_dev())
        ref_p.grad = g.clone()
        torch.nn.utils.clip_grad_norm_([ref_p], 1.0)
        opt.step()
        ss = grad_sumsq(g)
        adamw_step_(p, g, m, v, step=step, lr=1e-2, weight_decay=0.1, bf16_copy=shadow,
                    gnorm_sq=ss, max_norm=1.0)
    assert _rel_err(p, ref_p.detach()) < 1e-5
    assert _rel_err(shadow, p) < 5e-3


def test_linear_token_logps():
    from axolotl_b200.ops.functional import linear_token_logps
    torch.manual_seed(21)
    T, H, V = 600, 256, 3008
    h = (torch.randn(T, H) * 0.5).bfloat16().to(_dev()).requires_grad_(True)
    w = (torch.randn(V, H) * 0.05).bfloat16().to(_dev())
    labels = torch.randint(0, V, (T,), device=_dev())
    labels[::5] = -100
    g = torch.randn(T, device=_dev())
    lp = linear_token_logps(h, w, labels, chunk_rows=256)
    (lp * g).sum().backward()
    _check_status()
    hc = h.detach().cpu().float().requires_grad_(True)
    lab = labels.cpu()
    ref = torch.log_softmax(hc @ w.cpu().float().t(), -1).gather(1, lab.clamp(min=0)[:, None]).squeeze(1) * (lab != -100)
    (ref * g.cpu()).sum().backward()
    assert _rel_err(lp.cpu(), ref.detach()) < 1e-2
    assert float(lp.detach()[::5].abs().max()) == 0.0
    assert _rel_err(h.grad.cpu(), hc.grad) < 3e-2


def test_nvfp4_dequant_kernel_matches_reference_decode():
    from axolotl_b200.ops import nvfp4
    torch.manual_seed(22)
    w = torch.randn(384, 512) * 0.1
    q, s, pts = nvfp4.quantize_nvfp4(w)
    ref = nvfp4.dequantize_nvfp4(q, s, pts, dtype=torch.float32)          # CPU table decode
    got = nvfp4.dequantize_nvfp4(q.to(_dev()), s.to(_dev()), pts.to(_dev()))
    _check_status()
    assert got.dtype == torch.bfloat16 and got.shape == w.shape
    assert torch.equal(got.cpu(), ref.bfloat16())
    assert _rel_err(got.cpu(), w) < 0.15


def test_moe_block_matches_cpu_reference():
    """Sparse MoE block (router + per-expert GEMMs with expert LoRA) on the GPU against the same
    block in fp32 on the CPU."""
    from axolotl_b200.models.config import preset
    from axolotl_b200.models.moe import SparseMoE
    torch.manual_seed(23)
    cfg = preset("tiny-qwen3-moe")
    ref = SparseMoE(cfg, torch.float32, torch.device("cpu"))
    for p in ref.parameters():
        torch.nn.init.normal_(p, std=0.05)
    ref.experts.add_lora(8, 16)
    with torch.no_grad():
        for k in ("gate_up_B", "down_B"):
            ref.experts.lora[k].normal_(0, 0.05)
    dev = SparseMoE(cfg, torch.bfloat16, _dev())
    dev.experts.add_lora(8, 16)
    with torch.no_grad():
        for (n, p), (_, q) in zip(dev.named_parameters(), ref.named_parameters()):
            p.copy_(q)
        # use the same (bf16-rounded) base weights on both sides
        for (n, p), (_, q) in zip(dev.named_parameters(), ref.named_parameters()):
            if p.dtype == torch.bfloat16:
                q.copy_(p.float().cpu())
    x = (torch.randn(300, cfg.hidden_size) * 0.5).bfloat16()
    xd = x.to(_dev()).requires_grad_(True)
    xr = x.float().requires_grad_(True)
    yd, _ = dev(xd)
    yr, _ = ref(xr)
    gy = torch.randn_like(yr)
    yd.backward(gy.to(_dev()).bfloat16())
    yr.backward(gy)
    _check_status()
    assert _rel_err(yd.cpu(), yr.detach()) < 3e-2
    assert _rel_err(xd.grad.cpu(), xr.grad) < 5e-2
    for k in ("gate_up_A", "gate_up_B", "down_A", "down_B"):
        gd = dev.experts.lora[k]
        gd = getattr(gd, "_axb_grad", None) if gd.grad is None else gd.grad
        assert gd is not None and _rel_err(gd.float().cpu().reshape(-1), ref.experts.lora[k].grad.reshape(-1)) < 6e-2, k


def test_dpo_step_on_gpu():
    from axolotl_b200.models.config import preset
    from axolotl_b200.models.lora import LoraSpec, inject_lora
    from axolotl_b200.models.transformer import CausalLM
    from axolotl_b200.rl.data import synthetic_preference
    from axolotl_b200.rl.objectives import build_objective
    from axolotl_b200.train.optimizer import FlatAdamW, build_param_groups, make_lr_lambda
    from axolotl_b200.train.trainer import TrainArgs, Trainer

    cfg = preset("tiny-llama", vocab_size=1024)
    model = CausalLM(cfg, dtype=torch.bfloat16, device=_dev()).init_weights(0)
    inject_lora(model, LoraSpec(r=8, lora_alpha=16, target_modules="all-linear"))
    obj = build_objective({"rl": "dpo", "rl_beta": 0.5})
    coll = obj.collator()
    recs = synthetic_preference(32, 12, 12, 1024, seed=1)
    opt = FlatAdamW(build_param_groups(model.named_parameters()), lr=5e-3, max_grad_norm=1.0)
    opt.bind_model_shadows(model)
    tr = Trainer(model, opt, make_lr_lambda("constant", 100, 0), TrainArgs(max_steps=12, learning_rate=5e-3),
                 lambda e: [], device=_dev(), compute_loss=obj)
    losses = []
    for s in range(12):
        losses.append(float(tr.training_step([coll([recs[(s * 8 + j) % 32] for j in range(8)])])))
    _check_status()
    assert abs(losses[0] - math.log(2)) < 2e-2
    assert losses[-1] < losses[0] - 0.05 and obj.last_metrics["rewards/accuracies"] >= 0.75


@pytest.mark.parametrize("counts", [[130, 0, 5, 300, 128, 1, 0, 77], [0, 0, 0, 0, 0, 0, 0, 9], [256] * 8])
def test_grouped_gemm_modes(counts):
    """Grouped forward (with K-extension), transposed-weight and Gram modes against per-expert fp32."""
    from axolotl_b200.ops.grouped import GroupLayout, grouped_gemm, grouped_gram
    torch.manual_seed(31)
    E, K, N, r = len(counts), 192, 328, 16
    M = sum(counts)
    dev = _dev()
    cnt = torch.tensor(counts, device=dev)
    lay = GroupLayout(cnt, M)
    xs = (torch.randn(M, K) * 0.5).bfloat16().to(dev)
    W = (torch.randn(E, N, K) * 0.05).bfloat16().to(dev)
    t = (torch.randn(M, r) * 0.5).bfloat16().to(dev)
    Bt = (torch.randn(E, N, r) * 0.05).bfloat16().to(dev)
    x, tp = lay.pad(xs), lay.pad(t)
    y = lay.unpad(grouped_gemm(x, W, lay, a2=tp, w2=Bt, alpha=0.5))
    dy = (torch.randn(M, N) * 0.5).bfloat16().to(dev)
    dyp = lay.pad(dy)
    dx = lay.unpad(grouped_gemm(dyp, W, lay, trans_w=True))
    gW = grouped_gram(dyp, x, lay, torch.empty(E, N, K, dtype=torch.float32, device=dev))
    gW2 = grouped_gram(dyp, x, lay, gW.clone(), alpha=2.0, accumulate=True)
    gB = grouped_gram(dyp, tp, lay, torch.empty(E, N, r, dtype=torch.float32, device=dev))
    _check_status()
    s = 0
    for e, n in enumerate(counts):
        sl = slice(s, s + n)
        s += n
        ref_w = dy[sl].float().t() @ xs[sl].float()
        assert _rel_err(gW[e], ref_w) < 1e-2 or (n == 0 and float(gW[e].abs().max()) == 0.0)
        assert torch.allclose(gW2[e], 3.0 * gW[e], rtol=1e-3, atol=1e-3)
        if n == 0:
            continue
        ref = 0.5 * (xs[sl].float() @ W[e].float().t() + t[sl].float() @ Bt[e].float().t())
        assert _rel_err(y[sl], ref) < 1e-2, e
        assert _rel_err(dx[sl], dy[sl].float() @ W[e].float()) < 1e-2, e
        assert _rel_err(gB[e], dy[sl].float().t() @ t[sl].float()) < 1e-2, e


@pytest.mark.parametrize("counts,N,K", [([130, 0, 5, 300, 128, 1, 0, 77], 328, 192), ([256] * 4, 256, 512),
                                         ([0, 0, 9], 72, 64)])
def test_grouped_w4a16_equals_dequantise_then_gemm(counts, N, K):
    """NVFP4 decode inside the grouped GEMM: same bits as the dequantised bf16 stack fed to the bf16 kernel,
    forward (with the LoRA K-extension) and input gradient."""
    from axolotl_b200.ops.grouped import GroupLayout, grouped_gemm, grouped_gemm_w4a16, w4a16_ok
    from axolotl_b200.ops.nvfp4 import dequantize_nvfp4, quantize_nvfp4
    torch.manual_seed(33)
    E, r, dev = len(counts), 16, _dev()
    M = sum(counts)
    lay = GroupLayout(torch.tensor(counts, device=dev), M)
    W = torch.randn(E, N, K) * 0.05
    W[1] *= 40.0                                        # a different per-expert scale
    qd, sc, pts = quantize_nvfp4(W)
    q = {"qdata": qd.to(dev), "scale": sc.to(dev), "pts": pts.to(dev)}
    assert w4a16_ok(q)
    Wd = dequantize_nvfp4(q["qdata"], q["scale"], q["pts"])            # bf16 [E, N, K] on the device
    x = lay.pad((torch.randn(M, K) * 0.5).bfloat16().to(dev))
    t = lay.pad((torch.randn(M, r) * 0.5).bfloat16().to(dev))
    Bt = (torch.randn(E, N, r) * 0.05).bfloat16().to(dev)
    A16 = (torch.randn(E, r, K) * 0.05).bfloat16().to(dev)
    dy = lay.pad((torch.randn(M, N) * 0.5).bfloat16().to(dev))
    y_ref = grouped_gemm(x, Wd, lay, a2=t, w2=Bt, alpha=0.5)
    y = grouped_gemm_w4a16(x, q, lay, a2=t, w2=Bt, alpha=0.5)
    y0_ref, y0 = grouped_gemm(x, Wd, lay), grouped_gemm_w4a16(x, q, lay, out_dtype=torch.float32)
    dx_ref = grouped_gemm(dy, Wd, lay, trans_w=True, a2=t, w2=A16)
    dx = grouped_gemm_w4a16(dy, q, lay, trans_w=True, a2=t, w2=A16)
    dx0_ref, dx0 = grouped_gemm(dy, Wd, lay, trans_w=True), grouped_gemm_w4a16(dy, q, lay, trans_w=True)
    _check_status()
    for got, ref in ((y, y_ref), (dx, dx_ref), (dx0, dx0_ref)):
        assert torch.equal(lay.unpad(got), lay.unpad(ref))
    assert torch.equal(lay.unpad(y0).bfloat16(), lay.unpad(y0_ref))
    # and against plain fp32 arithmetic on the decoded weights
    s0 = 0
    for e, n in enumerate(counts):
        if n:
            xs = lay.unpad(x)[s0:s0 + n].float()
            assert _rel_err(lay.unpad(y0)[s0:s0 + n], xs @ Wd[e].float().t()) < 1e-2
        s0 += n


def test_moe_block_nvfp4_experts_match_dequantised_reference():
    from axolotl_b200.models.config import preset
    from axolotl_b200.models.moe import SparseMoE
    from axolotl_b200.ops.grouped import quantize_experts_nvfp4_
    from axolotl_b200.ops.nvfp4 import dequantize_nvfp4
    torch.manual_seed(32)
    cfg = preset("tiny-qwen3-moe")
    dev = SparseMoE(cfg, torch.bfloat16, _dev())
    for p in dev.parameters():
        torch.nn.init.normal_(p, std=0.05)
    ref = SparseMoE(cfg, torch.bfloat16, _dev())
    with torch.no_grad():
        for p, q in zip(ref.parameters(), dev.parameters()):
            p.copy_(q)
    quantize_experts_nvfp4_(dev)
    with torch.no_grad():   # reference holds the dequantised weights in bf16
        for which, name in (("gate_up", "gate_up_proj"), ("down", "down_proj")):
            q = dev.experts.nvfp4[which]
            getattr(ref.experts, name).copy_(dequantize_nvfp4(q["qdata"].cpu(), q["scale"].cpu(), q["pts"].cpu()).to(_dev()))
    for m in (dev, ref):
        m.experts.add_lora(8, 16)
    with torch.no_grad():
        for k in ("gate_up_A", "gate_up_B", "down_A", "down_B"):
            dev.experts.lora[k].normal_(0, 0.05)
            ref.experts.lora[k].copy_(dev.experts.lora[k])
    x = (torch.randn(260, cfg.hidden_size) * 0.5).bfloat16().to(_dev())
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    ya, _ = dev(xa)
    yb, _ = ref(xb)
    gy = torch.randn_like(ya)
    ya.backward(gy)
    yb.backward(gy)
    _check_status()
    assert _rel_err(ya, yb) < 1e-2 and _rel_err(xa.grad, xb.grad) < 1e-2
    for k in ("gate_up_A", "down_B"):
        assert _rel_err(dev.experts.lora[k].grad, ref.experts.lora[k].grad) < 2e-2, k


def test_nf4_dequant_kernel_and_qlora_linear():
    from axolotl_b200.models.layers import FusedLinear
    from axolotl_b200.ops.nf4 import dequantize_fp8_block, dequantize_nf4, quantize_nf4
    torch.manual_seed(41)
    w = torch.randn(384, 512) * 0.05
    for dq in (False, True):
        q, st = quantize_nf4(w, double_quant=dq)
        ref = dequantize_nf4(q, st, dtype=torch.float32)
        got = dequantize_nf4(q.to(_dev()), st.to(_dev()))
        _check_status()
        assert torch.equal(got.cpu(), ref.bfloat16())
    lin = FusedLinear(512, [384], ["x"], device=_dev())
    with torch.no_grad():
        lin.weight.copy_(w)
    lin.quantize_nf4_()
    lin.add_lora(8, 16)
    with torch.no_grad():
        lin.lora_B.normal_(0, 0.05)
    lin.refresh_shadows()
    x = (torch.randn(200, 512) * 0.5).bfloat16().to(_dev()).requires_grad_(True)
    y = lin(x)
    y.float().square().sum().backward()
    _check_status()
    wd = dequantize_nf4(lin.weight.data.cpu(), lin.weight._axb_quant.to("cpu"), dtype=torch.float32)
    xr = x.detach().cpu().float().requires_grad_(True)
    A, B = lin.lora_A.detach().cpu().float(), lin.lora_B.detach().cpu().float()
    yr = xr @ wd.t() + lin.scaling * ((xr @ A.t()) @ B.t())
    yr.square().sum().backward()
    assert _rel_err(y.cpu(), yr.detach()) < 3e-2 and _rel_err(x.grad.cpu(), xr.grad) < 4e-2
    # blockwise FP8
    wf = (torch.randn(256, 384) * 0.5).to(torch.float8_e4m3fn)
    sc = torch.rand(2, 3) + 0.5
    ref8 = dequantize_fp8_block(wf, sc)
    got8 = dequantize_fp8_block(wf.to(_dev()), sc.to(_dev()))
    _check_status()
    assert torch.equal(got8.cpu(), ref8)


@pytest.mark.parametrize("M,N,K", [(384, 520, 2048), (2304, 2560, 1024)])
def test_gemm_accumulate_single_pass_is_read_add_write(M, N, K):
    """accumulate=True with one K pass: non-atomic beta = 1 epilogue (1-CTA kernel for the small shape,
    2-CTA kernel for the large one), transposed operands as in a weight-gradient GEMM."""
    from axolotl_b200.ops.gemm import gemm
    torch.manual_seed(51)
    a = (torch.randn(K, M) * 0.5).bfloat16().to(_dev())     # dy^T stored as [K, M]
    b = (torch.randn(K, N) * 0.5).bfloat16().to(_dev())
    acc = torch.randn(M, N, device=_dev())
    ref = acc.double().cpu() + a.double().cpu().t() @ b.double().cpu()
    gemm(a, b, trans_a=True, trans_b=True, out=acc, accumulate=True, splits=1)
    gemm(a, b, trans_a=True, trans_b=True, out=acc, accumulate=True, splits=1)
    ref = ref + a.double().cpu().t() @ b.double().cpu()
    _check_status()
    assert _rel_err(acc.cpu(), ref.float()) < 2e-3


@pytest.mark.gpu
def test_clamped_glu_gated_rmsnorm_and_entropy_match_fp32_reference():
    from axolotl_b200.ops import functional as Fn
    torch.manual_seed(0)
    dev = "cuda"
    # clamped SwiGLU
    gu = (torch.randn(300, 2 * 256, device=dev) * 4).to(torch.bfloat16).requires_grad_(True)
    dh = torch.randn(300, 256, device=dev).to(torch.bfloat16)
    h = Fn.glu(gu, "silu", limit=3.0)
    h.backward(dh)
    g32 = gu.detach().float().requires_grad_(True)
    g, u = g32[:, :256], g32[:, 256:]
    ref = torch.nn.functional.silu(g.clamp(max=3.0)) * u.clamp(-3.0, 3.0)
    ref.backward(dh.float())
    assert torch.allclose(h.float(), ref, atol=3e-2, rtol=2e-2)
    assert torch.allclose(gu.grad.float(), g32.grad, atol=6e-2, rtol=3e-2)
    # gated RMSNorm
    x = torch.randn(257, 1024, device=dev).to(torch.bfloat16).requires_grad_(True)
    gt = torch.randn(257, 1024, device=dev).to(torch.bfloat16).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(1024, device=dev)).to(torch.bfloat16).requires_grad_(True)
    dy = torch.randn(257, 1024, device=dev).to(torch.bfloat16)
    y = Fn.rmsnorm_gated(x, gt, w, 1e-6)
    y.backward(dy)
    xf, gf, wf = (t.detach().float().requires_grad_(True) for t in (x, gt, w))
    yr = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wf * torch.nn.functional.silu(gf)
    yr.backward(dy.float())
    assert torch.allclose(y.float(), yr, atol=3e-2, rtol=2e-2)
    assert torch.allclose(x.grad.float(), xf.grad, atol=5e-2, rtol=3e-2)
    assert torch.allclose(gt.grad.float(), gf.grad, atol=5e-2, rtol=3e-2)
    assert torch.allclose(w.grad.float(), wf.grad, atol=0.5, rtol=3e-2)
    # online entropy
    for V in (1000, 32003):
        z = (torch.randn(65, V, device=dev) * 3).to(torch.bfloat16)
        ent, lse = Fn.token_entropy(z, temperature=0.7, return_lse=True)
        lp = torch.log_softmax(z.float() / 0.7, -1)
        assert torch.allclose(ent, -(lp.exp() * lp).sum(-1), atol=2e-3, rtol=1e-3)
        assert torch.allclose(lse, torch.logsumexp(z.float() / 0.7, -1), atol=2e-3, rtol=1e-4)


@pytest.mark.gpu
def test_sinkgd_fused_step_matches_elementwise_definition():
    from axolotl_b200.train.optimizers_extra import SinkGD
    torch.manual_seed(0)
    for shape, dt in (((96, 256), torch.float32), ((130, 77), torch.float32), ((512, 64), torch.bfloat16)):
        p = torch.nn.Parameter(torch.randn(shape, device="cuda").to(dt))
        g = torch.randn(shape, device="cuda")
        if dt != torch.float32:
            p.grad_dtype = None    # fp32 gradient buffer behind a bf16 parameter, as the flat optimizer keeps it
        p.grad = g.clone()
        ref = p.detach().float() * (1 - 0.1 * 0.01) - 0.1 * SinkGD.sinkhorn_normalize(g, 5, 1e-8)
        SinkGD([p], lr=0.1, n_iters=5, weight_decay=0.01).step()
        tol = 1e-4 if dt == torch.float32 else 2e-2
        assert torch.allclose(p.detach().float(), ref, atol=tol, rtol=tol), (p.detach().float() - ref).abs().max()


@pytest.mark.gpu
def test_flash_varlen_bidirectional_documents_match_fp32_reference():
    from axolotl_b200.ops import functional as Fn
    torch.manual_seed(0)
    Hq, Hk, D = 8, 2, 128
    cu = [0, 200, 329, 1000, 1024]
    T = cu[-1]
    qkv = (torch.randn(T, (Hq + 2 * Hk) * D, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    dout = torch.randn(T, Hq * D, device="cuda").to(torch.bfloat16)
    meta = Fn.AttnMeta(cu, "cuda", causal=False)
    out = Fn.flash_varlen(qkv, meta, Hq, Hk, D)
    out.backward(dout)
    x = qkv.detach().float().requires_grad_(True)
    q = x[:, :Hq * D].reshape(T, Hq, D)
    k = x[:, Hq * D:(Hq + Hk) * D].reshape(T, Hk, D)
    v = x[:, (Hq + Hk) * D:].reshape(T, Hk, D)
    ref = Fn._attn_ref(q, k, v, cu, 1.0 / D ** 0.5, causal=False).reshape(T, Hq * D)
    ref.backward(dout.float())
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2), (out.float() - ref).abs().max()
    err = (qkv.grad.float() - x.grad).abs().max() / x.grad.abs().max()
    assert err < 3e-2, err
    # and it differs from the causal result (the flag is honoured)
    causal = Fn.flash_varlen(qkv.detach(), Fn.AttnMeta(cu, "cuda"), Hq, Hk, D)
    assert (causal.float() - out.float()).abs().max() > 0.05


@pytest.mark.gpu
def test_decode_attention_and_cached_generation_match_full_recompute():
    from axolotl_b200.models.config import preset
    from axolotl_b200.models.transformer import CausalLM
    from axolotl_b200.ops import functional as Fn
    torch.manual_seed(0)
    # kernel against the fp32 definition (GQA 4:1 and 8:1, ragged lengths crossing chunk boundaries)
    for Hq, Hk, D in ((8, 2, 128), (16, 2, 64)):
        B, max_len = 5, 700
        lens = torch.tensor([1, 127, 128, 129, 700], dtype=torch.int32, device="cuda")
        qkv = torch.randn(B, (Hq + 2 * Hk) * D, device="cuda").to(torch.bfloat16)
        kc = torch.randn(B, max_len, Hk * D, device="cuda").to(torch.bfloat16)
        vc = torch.randn(B, max_len, Hk * D, device="cuda").to(torch.bfloat16)
        out = Fn.decode_attention(qkv, kc, vc, lens, Hq, Hk, D)
        ref = Fn.decode_attention(qkv.cpu(), kc.cpu(), vc.cpu(), lens.cpu(), Hq, Hk, D)
        assert torch.allclose(out.float().cpu(), ref.float(), atol=2e-2, rtol=2e-2), (out.float().cpu() - ref.float()).abs().max()
    # end to end: cached decoding reproduces full-recompute greedy decoding (dense and MoE)
    for name in ("tiny-llama", "tiny-qwen3-moe"):
        cfg = preset(name, vocab_size=512)
        m = CausalLM(cfg, dtype=torch.bfloat16, device="cuda").init_weights(0)
        p = torch.tensor([1, 5, 9, 12, 40, 41, 42], device="cuda")
        a, b = m.generate(p, 12), m.generate(p, 12, use_cache=False)
        agree = (a == b).float().mean().item()
        assert agree > 0.8, (name, a.tolist(), b.tolist())   # bf16 ties may flip a late token
        from axolotl_b200.models.kv_cache import generate_cached
        outs = generate_cached(m, [[1, 5, 9], [7, 8, 9, 10, 11], [3]], 6)
        assert [len(o) for o in outs] == [6, 6, 6]
        assert outs[1][:3] == m.generate(torch.tensor([7, 8, 9, 10, 11], device="cuda"), 3, use_cache=False)[0, 5:].tolist()


@pytest.mark.gpu
def test_kernels_leave_poisoned_guard_bands_untouched():
    """Out-of-bounds writes would land in the guard rows around each output; they are filled with a bit
    pattern beforehand and must be bit-identical afterwards (odd shapes that do not fill the last tile)."""
    from axolotl_b200.ops import _lib
    from axolotl_b200.ops import functional as Fn
    from axolotl_b200.ops.gemm import gemm
    torch.manual_seed(0)
    dev = "cuda"
    G = 64   # guard rows on both sides

    def guarded(rows, cols, dtype):
        big = torch.empty(rows + 2 * G, cols, dtype=dtype, device=dev)
        big.view(torch.uint8).fill_(0xCD)
        return big, big[G:G + rows]

    def intact(big, rows):
        v = big.view(torch.uint8)
        return bool((v[:G] == 0xCD).all()) and bool((v[G + rows:] == 0xCD).all())

    # GEMM: 1-CTA kernel (odd M, N not a tile multiple) and the CTA-pair kernel (large M, N), bf16 and fp32 out
    for M, N, K, dt in ((200, 328, 192, torch.bfloat16), (1000, 72, 256, torch.float32), (2504, 4104, 512, torch.bfloat16)):
        a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        b = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
        big, out = guarded(M, N, dt)
        gemm(a, b, out=out, out_dtype=dt)
        _lib.check_status()
        assert intact(big, M), ("gemm", M, N, K)
        ref = a.float() @ b.float().t()
        assert (out.float() - ref).abs().max() / ref.abs().max() < 2e-2
    # split-K accumulation into a guarded fp32 buffer
    a = torch.randn(4096, 40, device=dev, dtype=torch.bfloat16)
    b = torch.randn(4096, 264, device=dev, dtype=torch.bfloat16)
    big, out = guarded(40, 264, torch.float32)
    out.zero_()
    gemm(a, b, trans_a=True, trans_b=True, out=out, accumulate=True, splits=8)
    assert intact(big, 40)
    assert (out - a.float().t() @ b.float()).abs().max() < 0.5
    # in-place kernels on a row window of a larger buffer: RoPE and cross-entropy
    Hq, Hk, D, T = 4, 2, 64, 333
    big, qkv = guarded(T, (Hq + 2 * Hk) * D, torch.bfloat16)
    qkv.copy_(torch.randn_like(qkv.float()))
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device=dev, dtype=torch.float32) / D))
    pos = torch.arange(T, device=dev, dtype=torch.int32)
    Fn.rope_qk_(qkv, pos, inv, Hq, Hk, D)
    assert intact(big, T)
    V = 1003
    big, logits = guarded(77, 1008, torch.bfloat16)
    logits.copy_(torch.randn(77, 1008, device=dev))
    labels = torch.randint(0, V, (77,), device=dev)
    loss = torch.empty(77, dtype=torch.float32, device=dev)
    _lib.check_rc(_lib.cuda_lib().axb_ce_fwd_bwd(logits.data_ptr(), labels.data_ptr(), loss.data_ptr(), None, 77, V,
                                                 logits.stride(0), 1.0, -100, 1, _lib.stream_ptr()), "ce")
    torch.cuda.synchronize()
    assert intact(big, 77) and torch.isfinite(loss).all()


@pytest.mark.gpu
def test_flash_varlen_sliding_window_matches_fp32_reference():
    from axolotl_b200.ops import functional as Fn
    torch.manual_seed(0)
    Hq, Hk, D = 8, 2, 128
    cu = [0, 700, 829, 1500, 1536]
    T = cu[-1]
    for window in (300, 128, 50):
        qkv = (torch.randn(T, (Hq + 2 * Hk) * D, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
        dout = torch.randn(T, Hq * D, device="cuda").to(torch.bfloat16)
        meta = Fn.AttnMeta(cu, "cuda", window=window)
        out = Fn.flash_varlen(qkv, meta, Hq, Hk, D)
        out.backward(dout)
        x = qkv.detach().float().requires_grad_(True)
        q = x[:, :Hq * D].reshape(T, Hq, D)
        k = x[:, Hq * D:(Hq + Hk) * D].reshape(T, Hk, D)
        v = x[:, (Hq + Hk) * D:].reshape(T, Hk, D)
        ref = Fn._attn_ref(q, k, v, cu, 1.0 / D ** 0.5, True, window).reshape(T, Hq * D)
        ref.backward(dout.float())
        assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2), (window, (out.float() - ref).abs().max())
        err = (qkv.grad.float() - x.grad).abs().max() / x.grad.abs().max()
        assert err < 3e-2, (window, err)
    # decode attention with a window
    B, max_len = 3, 500
    lens = torch.tensor([40, 300, 500], dtype=torch.int32, device="cuda")
    qd = torch.randn(B, (Hq + 2 * Hk) * D, device="cuda").to(torch.bfloat16)
    kc = torch.randn(B, max_len, Hk * D, device="cuda").to(torch.bfloat16)
    vc = torch.randn(B, max_len, Hk * D, device="cuda").to(torch.bfloat16)
    o = Fn.decode_attention(qd, kc, vc, lens, Hq, Hk, D, window=200)
    r = Fn.decode_attention(qd.cpu(), kc.cpu(), vc.cpu(), lens.cpu(), Hq, Hk, D, window=200)
    assert torch.allclose(o.float().cpu(), r.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
def test_selective_nvfp4_dequant_skips_idle_experts_and_moe_output_is_unchanged():
    from axolotl_b200.models.config import preset
    from axolotl_b200.models.transformer import CausalLM
    from axolotl_b200.ops import _lib
    from axolotl_b200.ops.grouped import _expert_weights, quantize_experts_nvfp4_
    torch.manual_seed(0)
    cfg = preset("tiny-qwen3-moe", vocab_size=512)
    m = CausalLM(cfg, dtype=torch.bfloat16, device="cuda").init_weights(0)
    quantize_experts_nvfp4_(m)
    ex = m.layers[0].mlp.experts
    full = _expert_weights(ex, "gate_up")
    active = torch.zeros(ex.E, dtype=torch.int32, device="cuda")
    active[1] = 128
    part = _expert_weights(ex, "gate_up", active=active)
    torch.cuda.synchronize()
    assert torch.equal(part[1], full[1])
    # a short sequence routes to few experts: the layer output equals the all-experts path
    ids = torch.tensor([[5, 9, 12]], device="cuda")
    m.eval()
    with torch.no_grad():
        y = m(ids, return_logits=True).logits
    assert torch.isfinite(y.float()).all()
    _lib.check_status()


@pytest.mark.parametrize("kind,limit", [(0, 0.0), (1, 0.0), (0, 1.5)])
@pytest.mark.parametrize("M,I,K,R", [(5120, 1024, 512, 32), (4700, 1184, 320, 0)])
def test_gemm_glu_epilogues(kind, limit, M, I, K, R, monkeypatch):
    """GLU folded into the CTA-pair GEMM: forward (gate|up tile halves) and backward (dh -> d_gate|d_up)."""
    import torch.nn.functional as F
    from axolotl_b200.ops import gemm as gemm_mod
    from axolotl_b200.ops.gemm import gemm, glu_fusable
    monkeypatch.setattr(gemm_mod, "USE_GLU_EPILOGUE", True)
    torch.manual_seed(11)
    dev = _dev()
    assert glu_fusable(M, I, dev)
    x = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
    W = (torch.randn(2 * I, K, device=dev) * 0.05).bfloat16()
    a2 = (torch.randn(M, R, device=dev) * 0.5).bfloat16() if R else None
    b2 = (torch.randn(2 * I, R, device=dev) * 0.05).bfloat16() if R else None
    gu = torch.empty(M, 2 * I, device=dev, dtype=torch.bfloat16)
    h = torch.empty(M, I, device=dev, dtype=torch.bfloat16)
    gemm(x, W, a2=a2, b2=b2, out=gu, glu=("fwd", kind, limit, h))
    _check_status()
    ref_gu = x.float() @ W.float().t() + (a2.float() @ b2.float().t() if R else 0.0)
    assert _rel_err(gu, ref_gu) < 5e-3
    act = (lambda t: F.silu(t)) if kind == 0 else (lambda t: F.gelu(t, approximate="tanh"))
    g, u = gu[:, :I].float(), gu[:, I:].float()      # the kernel rounds gate / up to bf16 first, as the saved tensor is
    gc, uc = (g.clamp(max=limit), u.clamp(-limit, limit)) if limit > 0 else (g, u)
    assert _rel_err(h, act(gc) * uc) < 5e-3
    # backward: dh = dy @ Wd (+ extension), Wd stored [H, I]
    Hd = 384
    dy = (torch.randn(M, Hd, device=dev) * 0.5).bfloat16()
    Wd = (torch.randn(Hd, I, device=dev) * 0.05).bfloat16()
    t2 = (torch.randn(M, 16, device=dev) * 0.5).bfloat16() if R else None
    A2 = (torch.randn(16, I, device=dev) * 0.05).bfloat16() if R else None
    dgu = torch.empty_like(gu)
    gemm(dy, Wd, trans_b=True, a2=t2, b2=A2, out=dgu, glu=("bwd", kind, limit, gu))
    _check_status()
    dh = dy.float() @ Wd.float() + (t2.float() @ A2.float() if R else 0.0)
    gl = gc.clone().requires_grad_(True)
    (da,) = torch.autograd.grad(act(gl).sum(), gl)
    dg, du = dh * uc * da, dh * act(gc)
    if limit > 0:
        dg, du = dg * (g <= limit), du * ((u >= -limit) & (u <= limit))
    assert _rel_err(dgu[:, :I], dg) < 8e-3
    assert _rel_err(dgu[:, I:], du) < 8e-3
    # in place over the saved gate|up
    gu2 = gu.clone()
    gemm(dy, Wd, trans_b=True, a2=t2, b2=A2, out=gu2, glu=("bwd", kind, limit, gu2))
    _check_status()
    assert torch.equal(gu2, dgu)


@pytest.mark.parametrize("lora", [True, False])
def test_fused_glu_mlp_matches_unfused(lora):
    """The one-node MLP (GLU in the GEMM epilogues) against the projection-by-projection path."""
    from axolotl_b200.models.transformer import MLP
    from axolotl_b200.ops import gemm as gemm_mod
    torch.manual_seed(12)
    dev = _dev()
    T, H, I = 4608, 512, 1152
    mlp = MLP(H, I, "silu", False, torch.bfloat16, dev)
    with torch.no_grad():
        mlp.gate_up_proj.weight.normal_(0, 0.04)
        mlp.down_proj.weight.normal_(0, 0.04)
    if lora:
        for m in (mlp.gate_up_proj, mlp.down_proj):
            m.weight.requires_grad_(False)
            m.add_lora(16, 32, init_b_zero=False)
    x = (torch.randn(T, H, device=dev) * 0.5).bfloat16().requires_grad_(True)
    dy = (torch.randn(T, H, device=dev) * 0.1).bfloat16()
    params = [p for p in mlp.parameters() if p.requires_grad]

    def run():
        y = mlp(x)
        grads = torch.autograd.grad(y, [x] + params, dy)
        return y, grads

    prev = gemm_mod.USE_GLU_EPILOGUE
    try:
        gemm_mod.USE_GLU_EPILOGUE = True
        assert gemm_mod.glu_fusable(T, I, dev)
        y1, g1 = run()
        gemm_mod.USE_GLU_EPILOGUE = False
        y0, g0 = run()
    finally:
        gemm_mod.USE_GLU_EPILOGUE = prev
    _check_status()
    assert _rel_err(y1, y0) < 1e-2
    for a, b in zip(g1, g0):
        assert _rel_err(a, b) < 2e-2


@pytest.mark.parametrize("T,N,R,blocks", [
    (4096, 1536, 48, [(0, 1024, 0, 16), (1024, 256, 16, 16), (1280, 256, 32, 16)]),   # q|k|v
    (1000, 520, 16, [(0, 520, 0, 16)]),                                                # ragged T and N
    (2048, 3072, 32, [(0, 1536, 0, 16), (1536, 1536, 16, 16)]),                        # gate|up
])
def test_lora_fused_dy_pass(T, N, R, blocks):
    """t = s dy B and dB += dy^T xa from one pass over dy, against fp32 references; entries of dB outside
    the diagonal blocks must stay untouched."""
    from axolotl_b200.ops.lora import fused_dy_ok, lora_bwd_dy
    torch.manual_seed(31)
    dev = _dev()
    dy = (torch.randn(T, N, device=dev) * 0.3).bfloat16()
    B = torch.zeros(N, R, device=dev)
    for (r0, rows, c0, r) in blocks:
        B[r0:r0 + rows, c0:c0 + r] = torch.randn(rows, r, device=dev) * 0.1
    B16 = B.bfloat16()
    xa = (torch.randn(T, R, device=dev) * 0.3).bfloat16()
    assert fused_dy_ok(dy, B16, xa)
    acc = torch.full((N, R), 0.5, device=dev, dtype=torch.float32)
    t = lora_bwd_dy(dy, B16, xa, blocks, 2.0, acc)
    _check_status()
    assert _rel_err(t, 2.0 * (dy.float() @ B16.float())) < 5e-3
    full = dy.float().t() @ xa.float()
    ref = torch.full((N, R), 0.5, device=dev)
    for (r0, rows, c0, r) in blocks:
        ref[r0:r0 + rows, c0:c0 + r] += full[r0:r0 + rows, c0:c0 + r]
    assert _rel_err(acc, ref) < 5e-3
    mask = torch.ones(N, R, dtype=torch.bool, device=dev)
    for (r0, rows, c0, r) in blocks:
        mask[r0:r0 + rows, c0:c0 + r] = False
    assert bool((acc[mask] == 0.5).all())


def test_lora_linear_backward_fused_dy_matches_two_pass():
    from axolotl_b200.models.layers import FusedLinear
    from axolotl_b200.ops import lora as lora_mod
    torch.manual_seed(32)
    dev = _dev()
    lin = FusedLinear(512, [768, 256, 256], ["q_proj", "k_proj", "v_proj"], dtype=torch.bfloat16, device=dev)
    with torch.no_grad():
        lin.weight.normal_(0, 0.04)
    lin.weight.requires_grad_(False)
    lin.add_lora(16, 32, init_b_zero=False)
    x = (torch.randn(2048, 512, device=dev) * 0.5).bfloat16().requires_grad_(True)
    dy = (torch.randn(2048, 1280, device=dev) * 0.1).bfloat16()

    def run():
        return torch.autograd.grad(lin(x), [x, lin.lora_A, lin.lora_B], dy)

    prev = lora_mod.USE_FUSED_DY
    try:
        lora_mod.USE_FUSED_DY = True
        g1 = run()
        lora_mod.USE_FUSED_DY = False
        g0 = run()
    finally:
        lora_mod.USE_FUSED_DY = prev
    _check_status()
    for a, b in zip(g1, g0):
        assert _rel_err(a, b) < 1e-2


def test_dora_weight_norm_kernel():
    """||W + s B A|| per row without forming B A: skinny GEMMs + the row-wise kernel, against fp32 torch."""
    from axolotl_b200.models.layers import FusedLinear
    torch.manual_seed(41)
    dev = _dev()
    lin = FusedLinear(512, [384, 128], ["gate_proj", "up_proj"], dtype=torch.bfloat16, device=dev)
    with torch.no_grad():
        lin.weight.normal_(0, 0.05)
    lin.weight.requires_grad_(False)
    lin.add_lora(16, 32, init_b_zero=False, use_dora=True)
    got = lin.dora_weight_norm()
    _check_status()
    W, A, B = lin.weight.float(), lin.lora_A16.float(), lin.lora_B.float()
    ref = (W + lin.scaling * (B @ A)).norm(dim=1)
    assert _rel_err(got, ref) < 5e-3
    assert got.dtype == torch.float32 and got.shape == (512,)


def test_bounds_check_build_reports_through_the_device_record():
    """The -DAXB_BOUNDS_CHECK library: a clean tiny training step records nothing; an out-of-range token id and
    label are recorded with site, index and limit while the access itself is skipped (no fault)."""
    import os
    import subprocess
    import sys
    code = r'''
import torch
from axolotl_b200.ops import _lib, functional as Fn
from axolotl_b200.models.config import preset
from axolotl_b200.models.transformer import CausalLM
assert _lib.cuda_lib().axb_bounds_check_enabled() == 1
dev = torch.device("cuda:0")
cfg = preset("tiny-llama", num_hidden_layers=2)
m = CausalLM(cfg, torch.bfloat16, dev).init_weights(0)
ids = torch.randint(0, cfg.vocab_size, (1, 256))
out = m(ids, labels=ids.clone())
out.loss.backward()
torch.cuda.synchronize()
assert _lib.bounds_violation() is None, _lib.bounds_violation()
_lib.check_status()
table = torch.randn(64, 128, device=dev).bfloat16()
bad = torch.tensor([1, 2, 99, 3], device=dev)
y = Fn.embedding(table, bad)
torch.cuda.synchronize()
v = _lib.bounds_violation()
assert v is not None and v[0] == "embedding token id" and v[1] == 99 and v[2] == 64, v
assert torch.equal(y[2], table[0])            # the access went to a valid row instead
try:
    _lib.check_bounds()
    raise SystemExit("check_bounds did not raise")
except _lib.KernelBoundsError as e:
    assert "index 99" in str(e)
assert _lib.bounds_violation() is None        # reset by check_bounds
h = torch.randn(8, 128, device=dev).bfloat16()
W = torch.randn(64, 128, device=dev).bfloat16()
lab = torch.tensor([1, 2, 3, 64, -100, 5, 6, 7], device=dev)
loss = Fn.linear_cross_entropy(h, W, lab, num_items=7)
torch.cuda.synchronize()
v = _lib.bounds_violation()
assert v is not None and v[0] == "cross-entropy label" and v[1] == 64 and v[2] == 64, v
assert torch.isfinite(loss)
print("BOUNDS_OK")
'''
    env = dict(os.environ, AXB_BOUNDS_CHECK="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "BOUNDS_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-3000:]


@pytest.mark.parametrize("name", ["tiny-gemma2", "tiny-gemma3"])
def test_gemma_models_on_gpu_match_cpu_fp32(name):
    """Gemma 2 / 3 end to end on the device (head width 256 attention, soft caps, sandwich norms, sliding and
    global layers, local rope base) against the same weights in fp32 on the CPU: loss and LoRA-free gradients."""
    from axolotl_b200.models.config import preset
    from axolotl_b200.models.layers import RMSNorm
    from axolotl_b200.models.transformer import CausalLM
    torch.manual_seed(50)
    cfg = preset(name)
    ref = CausalLM(cfg, dtype=torch.float32).init_weights(4)
    with torch.no_grad():
        for m in ref.modules():
            if isinstance(m, RMSNorm):
                m.weight.uniform_(-0.2, 0.2)
        for p in ref.parameters():                      # values the bf16 copy represents exactly
            p.copy_(p.bfloat16().float())
    dev = CausalLM(cfg, dtype=torch.bfloat16, device=_dev())
    dev.load_state_dict(ref.state_dict())
    lens = [150, 61, 300]
    ids = torch.cat([torch.randint(3, cfg.vocab_size, (l,)) for l in lens])[None]
    pos = torch.cat([torch.arange(l) for l in lens])[None].to(torch.int32)
    labels = ids.clone()
    labels[:, :20] = -100
    out_d = dev(ids, pos, labels)
    out_d.loss.backward()
    _check_status()
    out_c = ref(ids, pos, labels)
    out_c.loss.backward()
    assert abs(out_d.loss.item() - out_c.loss.item()) < 3e-2 * abs(out_c.loss.item())
    for pick in ("layers.0.self_attn.qkv_proj.weight", "layers.1.mlp.down_proj.weight", "embed_tokens"):
        gd = dict(dev.named_parameters())[pick].grad.float().cpu()
        gc = dict(ref.named_parameters())[pick].grad
        assert _rel_err(gd, gc) < 6e-2, pick


def test_deepseek_v3_latent_attention_model_on_gpu_matches_cpu_fp32():
    """Latent attention (192-wide q/k, 128-wide v through the wide kernels), grouped sigmoid routing and shared
    experts on the device against the same weights in fp32 on the CPU."""
    from axolotl_b200.models.config import ModelConfig
    from axolotl_b200.models.transformer import CausalLM
    torch.manual_seed(51)
    cfg = ModelConfig.from_hf_dict(dict(
        model_type="deepseek_v3", vocab_size=2048, hidden_size=256, intermediate_size=512, moe_intermediate_size=128,
        num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=2, n_routed_experts=8, n_shared_experts=1,
        num_experts_per_tok=2, n_group=2, topk_group=1, first_k_dense_replace=1, q_lora_rank=64, kv_lora_rank=64,
        qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, routed_scaling_factor=2.0, norm_topk_prob=True,
        rms_norm_eps=1e-6, rope_theta=10000.0, hidden_act="silu", tie_word_embeddings=False, max_position_embeddings=2048))
    ref = CausalLM(cfg, dtype=torch.float32).init_weights(5)
    with torch.no_grad():
        for p in ref.parameters():
            p.copy_(p.bfloat16().float())
    dev = CausalLM(cfg, dtype=torch.bfloat16, device=_dev())
    dev.load_state_dict(ref.state_dict())
    lens = [140, 260]
    ids = torch.cat([torch.randint(3, cfg.vocab_size, (l,)) for l in lens])[None]
    pos = torch.cat([torch.arange(l) for l in lens])[None].to(torch.int32)
    labels = ids.clone()
    out_d = dev(ids, pos, labels)
    out_d.loss.backward()
    _check_status()
    out_c = ref(ids, pos, labels)
    out_c.loss.backward()
    assert abs(out_d.loss.item() - out_c.loss.item()) < 3e-2 * abs(out_c.loss.item())
    for pick in ("layers.0.self_attn.kv_b_proj.weight", "layers.1.self_attn.q_b_proj.weight", "embed_tokens"):
        gd = dict(dev.named_parameters())[pick].grad.float().cpu()
        gc = dict(ref.named_parameters())[pick].grad
        assert _rel_err(gd, gc) < 8e-2, pick


@pytest.mark.parametrize("whitening", [False, True])
def test_ebft_feature_rewards_kernel_matches_torch(whitening):
    """Alignment (2 cos to the ground truth) and diversity (2 x mean dot to the other samples of the group) from one
    launch against the matrix formulation on the CPU."""
    from axolotl_b200.rl.ebft import feature_rewards
    torch.manual_seed(60)
    P, n, D = 5, 4, 777
    gen, gt = torch.randn(P * n, D), torch.randn(P, D)
    r_dev, m_dev = feature_rewards(gen.to(_dev()), gt.to(_dev()), n, 1.0, 0.7, use_whitening=whitening)
    r_cpu, m_cpu = feature_rewards(gen, gt, n, 1.0, 0.7, use_whitening=whitening)
    assert torch.allclose(r_dev.cpu(), r_cpu, atol=2e-3, rtol=2e-3), (r_dev.cpu() - r_cpu).abs().max()
    assert abs(m_dev["ebft/diversity"] - m_cpu["ebft/diversity"]) < 2e-3
    one, _ = feature_rewards(gen[:P].to(_dev()), gt.to(_dev()), 1)
    ref, _ = feature_rewards(gen[:P], gt, 1)
    assert torch.allclose(one.cpu(), ref, atol=1e-4)


def test_partial_rotary_kernel_matches_reference():
    from axolotl_b200.ops.functional import rope_qk_
    torch.manual_seed(61)
    T, Hq, Hk, D, rot = 300, 4, 2, 64, 32
    base = (torch.randn(T, (Hq + 2 * Hk) * D) * 0.5).bfloat16()
    pos = torch.cat([torch.arange(180), torch.arange(120)]).to(torch.int32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    x = base.to(_dev()).requires_grad_(True)
    y = rope_qk_(x * 1.0, pos.to(_dev()), inv.to(_dev()), Hq, Hk, D, 1.0, rot_dim=rot)
    g = torch.randn(T, (Hq + 2 * Hk) * D).bfloat16()
    (y.float() * g.to(_dev()).float()).sum().backward()
    xc = base.float().requires_grad_(True)
    yc = rope_qk_(xc, pos, inv, Hq, Hk, D, 1.0, rot_dim=rot)
    (yc * g.float()).sum().backward()
    assert _rel_err(y.cpu(), yc) < 1e-2 and _rel_err(x.grad.cpu(), xc.grad) < 1e-2
    assert torch.equal(y[:, rot:D].cpu(), base[:, rot:D])                 # the tail of a head passes through
    assert torch.equal(y[:, (Hq + Hk) * D:].cpu(), base[:, (Hq + Hk) * D:])   # v untouched


@pytest.mark.parametrize("fp4", [False, True])
def test_moe_decode_gemv_matches_grouped_path(fp4, monkeypatch):
    """A generation step's expert pass (matrix-vector kernel, bf16 or NVFP4 weights, expert LoRA) against the grouped
    tensor-core path on the same few tokens."""
    from axolotl_b200.models.config import preset
    from axolotl_b200.models.moe import SparseMoE
    from axolotl_b200.ops import grouped
    torch.manual_seed(62)
    cfg = preset("tiny-qwen3-moe")
    moe = SparseMoE(cfg, torch.bfloat16, _dev())
    for p in moe.parameters():
        torch.nn.init.normal_(p, std=0.05)
    if fp4:
        grouped.quantize_experts_nvfp4_(moe)
    moe.experts.add_lora(8, 16)
    with torch.no_grad():
        for k in ("gate_up_A", "gate_up_B", "down_A", "down_B"):
            moe.experts.lora[k].normal_(0, 0.05)
    x = (torch.randn(5, cfg.hidden_size) * 0.5).bfloat16().to(_dev())
    with torch.no_grad():
        y_gemv, _ = moe(x)
        monkeypatch.setattr(grouped, "GEMV_MAX_SLOTS", 0)
        y_grouped, _ = moe(x)
    _check_status()
    assert _rel_err(y_gemv, y_grouped) < 1.5e-2


@pytest.mark.parametrize("H,L,off", [(32, 300, 0), (32, 1000, 0), (64, 515, 0), (128, 260, 0), (32, 200, 333)])
def test_indexer_scores_kernel_matches_reference(H, L, off):
    """Lightning-indexer scores (relu(q.k) mixed over heads inside the GEMM epilogue) against the fp32 einsum form; `off`
    is the case of a block of queries that starts `off` positions into its document."""
    from axolotl_b200.models import dsa

    torch.manual_seed(H + L)
    q = torch.randn(L, H, 128, device="cuda").bfloat16()
    k = torch.randn(L + off, 128, device="cuda").bfloat16()
    w = torch.randn(L, H, device="cuda") * 0.1
    got = dsa.indexer_scores(q, k, w, causal_off=off)
    ref = dsa.indexer_scores_ref(q, k, w, causal_off=off)
    torch.cuda.synchronize()
    assert torch.equal(torch.isinf(got), torch.isinf(ref))
    fin = ~torch.isinf(ref)
    err = (got[fin] - ref[fin]).abs().max().item()
    assert err < 2e-2 * ref[fin].abs().max().item(), err
    # the selection that the scores feed: the two top-k sets agree but for near-ties
    kk = min(64, L)
    a, b = got.topk(kk, -1).indices, ref.topk(kk, -1).indices
    rows = torch.arange(L, device="cuda")[:, None]
    ma = torch.zeros(L, L + off, dtype=torch.bool, device="cuda")
    ma[rows, a] = True
    mb = torch.zeros_like(ma)
    mb[rows, b] = True
    vis = fin
    assert ((ma ^ mb) & vis).float().sum().item() <= 0.01 * vis.float().sum().item()


def test_glm_dsa_sparse_attention_model_on_gpu_matches_cpu_fp32():
    """GLM-5 graph on the device: 256-wide latent-attention heads through the wide kernels for the document within the
    top-k budget, indexer kernel + selected-key attention for the longer one, against fp32 on the CPU. Most of a
    query's keys are selected (256 of at most 420), so a selection that differs on a near-tie moves the loss little."""
    from axolotl_b200.models.config import ModelConfig
    from axolotl_b200.models.transformer import CausalLM
    torch.manual_seed(52)
    cfg = ModelConfig.from_hf_dict(dict(
        model_type="glm_moe_dsa", vocab_size=2048, hidden_size=256, intermediate_size=512, moe_intermediate_size=128,
        num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=2, n_routed_experts=8, n_shared_experts=1,
        num_experts_per_tok=2, n_group=1, topk_group=1, mlp_layer_types=["dense", "sparse"], q_lora_rank=64, kv_lora_rank=64,
        qk_nope_head_dim=192, qk_rope_head_dim=64, v_head_dim=256, routed_scaling_factor=2.0, norm_topk_prob=True,
        rms_norm_eps=1e-5, hidden_act="silu", tie_word_embeddings=False, max_position_embeddings=2048,
        index_topk=256, index_head_dim=128, index_n_heads=32, rope_parameters={"rope_type": "default", "rope_theta": 10000.0}))
    ref = CausalLM(cfg, dtype=torch.float32).init_weights(6)
    with torch.no_grad():
        for p in ref.parameters():
            p.copy_(p.bfloat16().float())
    dev = CausalLM(cfg, dtype=torch.bfloat16, device=_dev())
    dev.load_state_dict(ref.state_dict())
    lens = [150, 420]
    ids = torch.cat([torch.randint(3, cfg.vocab_size, (l,)) for l in lens])[None]
    pos = torch.cat([torch.arange(l) for l in lens])[None].to(torch.int32)
    labels = ids.clone()
    out_d = dev(ids, pos, labels)
    out_d.loss.backward()
    _check_status()
    out_c = ref(ids, pos, labels)
    out_c.loss.backward()
    assert abs(out_d.loss.item() - out_c.loss.item()) < 3e-2 * abs(out_c.loss.item())
    for pick in ("layers.0.self_attn.kv_b_proj.weight", "layers.1.self_attn.q_b_proj.weight", "embed_tokens"):
        gd = dict(dev.named_parameters())[pick].grad.float().cpu()
        gc = dict(ref.named_parameters())[pick].grad
        assert _rel_err(gd, gc) < 1e-1, pick


def test_head_width_512_runs_the_blocked_path_and_matches_fp32_reference():
    """A head width without a kernel of its own (512) goes through the blocked library path: same result as the
    fp32 reference, forward and backward, on packed documents with a sliding window."""
    from axolotl_b200.ops import functional as Fn
    torch.manual_seed(70)
    Hq, Hk, D = 4, 2, 512
    lens = [300, 212]
    T = sum(lens)
    cu = [0, 300, 512]
    qkv = (torch.randn(T, (Hq + 2 * Hk) * D, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    meta = Fn.AttnMeta(cu, "cuda", window=128)
    out = Fn.flash_varlen(qkv, meta, Hq, Hk, D)
    g = torch.randn_like(out)
    out.backward(g)
    x = qkv.detach().float().cpu().requires_grad_(True)
    q, k, v = x[:, : Hq * D].reshape(T, Hq, D), x[:, Hq * D:(Hq + Hk) * D].reshape(T, Hk, D), x[:, (Hq + Hk) * D:].reshape(T, Hk, D)
    ref = Fn._attn_ref(q, k, v, cu, D ** -0.5, True, 128).reshape(T, Hq * D)
    ref.backward(g.float().cpu())
    assert _rel_err(out.float().cpu(), ref) < 2e-2
    assert _rel_err(qkv.grad.float().cpu(), x.grad) < 3e-2


def test_xielu_kernel_matches_definition_forward_and_backward():
    from axolotl_b200.ops import functional as Fn
    torch.manual_seed(80)
    x = (torch.randn(777, 1031, device="cuda") * 2).bfloat16().requires_grad_(True)
    ap = torch.tensor([0.9], device="cuda", requires_grad=True)
    an = torch.tensor([1.3], device="cuda", requires_grad=True)
    g = torch.randn(777, 1031, device="cuda").bfloat16()
    y = Fn.xielu(x, ap, an, 0.5, -1e-6)
    y.backward(g)
    xr = x.detach().float().cpu().requires_grad_(True)
    apr, anr = ap.detach().cpu().requires_grad_(True), an.detach().cpu().requires_grad_(True)
    yr = Fn.xielu(xr, apr, anr, 0.5, -1e-6)
    yr.backward(g.float().cpu())
    assert _rel_err(y.float().cpu(), yr) < 1e-2
    assert _rel_err(x.grad.float().cpu(), xr.grad) < 1e-2
    assert abs(ap.grad.item() - apr.grad.item()) < 2e-2 * abs(apr.grad.item()) + 1.0
    assert abs(an.grad.item() - anr.grad.item()) < 2e-2 * abs(anr.grad.item()) + 1.0


def test_gated_softmax_pool_kernel_matches_torch():
    from axolotl_b200.ops import functional as Fn
    torch.manual_seed(81)
    kv = torch.randn(3, 41, 8, 96, device="cuda", requires_grad=True)
    gate = (torch.randn(3, 41, 8, 96, device="cuda") * 3).requires_grad_(True)
    out = Fn.gated_softmax_pool(kv, gate)
    g = torch.randn_like(out)
    out.backward(g)
    kr, gr = kv.detach().cpu().requires_grad_(True), gate.detach().cpu().requires_grad_(True)
    ref = Fn.gated_softmax_pool(kr, gr)
    ref.backward(g.cpu())
    assert torch.allclose(out.cpu(), ref, atol=1e-5, rtol=1e-4)
    assert torch.allclose(kv.grad.cpu(), kr.grad, atol=1e-5, rtol=1e-4)
    assert torch.allclose(gate.grad.cpu(), gr.grad, atol=1e-5, rtol=1e-4)


_GPU_FAMILIES = {
    "falcon_h1": dict(model_type="falcon_h1", mamba_d_ssm=512, mamba_n_heads=8, mamba_d_head=64, mamba_n_groups=2, mamba_d_state=16,
                      mamba_d_conv=4, mamba_chunk_size=64, mamba_rms_norm=True, mamba_norm_before_gate=False,
                      ssm_multipliers=[0.9, 1.1, 1.2, 0.8, 1.3], mlp_multipliers=[0.8, 1.4], key_multiplier=0.8,
                      ssm_out_multiplier=0.7, attention_out_multiplier=0.9),
    "nemotron_h": dict(model_type="nemotron_h", layers_block_type=["mamba", "attention", "mlp", "mamba"], mlp_hidden_act="relu2",
                       ssm_state_size=16, mamba_num_heads=8, mamba_head_dim=64, n_groups=2, conv_kernel=4, chunk_size=64),
    "bamba": dict(model_type="bamba", attn_layer_indices=[1], mamba_n_heads=8, mamba_d_head="auto", mamba_n_groups=1, mamba_d_state=16,
                  mamba_d_conv=4, mamba_expand=2, mamba_chunk_size=64),
    "qwen3_5_moe_text": dict(model_type="qwen3_5_moe_text", num_hidden_layers=4, linear_num_value_heads=4, linear_num_key_heads=2,
                             linear_key_head_dim=64, linear_value_head_dim=64, linear_conv_kernel_dim=4, num_experts=8,
                             num_experts_per_tok=2, moe_intermediate_size=128, shared_expert_intermediate_size=128),
    "lfm2": dict(model_type="lfm2", num_hidden_layers=3, layer_types=["conv", "full_attention", "conv"], conv_L_cache=3,
                 block_auto_adjust_ff_dim=False, tie_word_embeddings=True),
    "cohere2": dict(model_type="cohere2", num_hidden_layers=4, logit_scale=0.25, tie_word_embeddings=True, sliding_window=128,
                    layer_types=["sliding_attention", "sliding_attention", "sliding_attention", "full_attention"]),
    "starcoder2": dict(model_type="starcoder2", use_bias=True, sliding_window=256, tie_word_embeddings=True),
    "nemotron": dict(model_type="nemotron"),
    "apertus": dict(model_type="apertus", rope_parameters={"rope_type": "default", "rope_theta": 10000.0}),
    "glm4": dict(model_type="glm4", partial_rotary_factor=0.5, attention_bias=True),
    "olmo3": dict(model_type="olmo3", num_hidden_layers=4, sliding_window=128,
                  layer_types=["sliding_attention", "sliding_attention", "sliding_attention", "full_attention"]),
    "seed_oss": dict(model_type="seed_oss", attention_bias=True, attention_out_bias=True),
    "ministral3": dict(model_type="ministral3"),
    "hunyuan_v1_moe": dict(model_type="hunyuan_v1_moe", intermediate_size=128, num_experts=8, moe_topk=2),
    "ernie4_5_moe": dict(model_type="ernie4_5_moe", moe_intermediate_size=128, moe_num_experts=8, moe_k=2, moe_num_shared_experts=1,
                         moe_layer_start_index=1, moe_layer_interval=1, moe_layer_end_index=-1),
    "glm4_moe": dict(model_type="glm4_moe", moe_intermediate_size=128, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2,
                     first_k_dense_replace=1, use_qk_norm=True, attention_bias=True),
    "minimax_m2": dict(model_type="minimax_m2", intermediate_size=128, num_local_experts=8, num_experts_per_tok=2),
    "phi": dict(model_type="phi"),
    "gemma4_text": dict(model_type="gemma4_text", num_hidden_layers=3, head_dim=256, global_head_dim=512, sliding_window=128,
                        layer_types=["sliding_attention", "sliding_attention", "full_attention"], hidden_size_per_layer_input=0,
                        attention_k_eq_v=True, num_global_key_value_heads=1, tie_word_embeddings=True),
    "gemma4_text_full": dict(model_type="gemma4_text", num_hidden_layers=4, head_dim=256, global_head_dim=512, sliding_window=128,
                             layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
                             hidden_size_per_layer_input=128, num_kv_shared_layers=2, enable_moe_block=True, num_experts=8,
                             top_k_experts=2, moe_intermediate_size=128, tie_word_embeddings=True),
    "afmoe": dict(model_type="afmoe", num_hidden_layers=4, moe_intermediate_size=128, num_experts=8, num_experts_per_tok=2,
                  num_shared_experts=1, num_dense_layers=1, sliding_window=128),
    "olmo": dict(model_type="olmo", clip_qkv=8.0),
    "falcon": dict(model_type="falcon", new_decoder_architecture=True, num_kv_heads=2, ffn_hidden_size=1024),
    "lfm2_moe": dict(model_type="lfm2_moe", num_hidden_layers=3, layer_types=["conv", "full_attention", "conv"], conv_L_cache=3,
                     moe_intermediate_size=128, num_experts=8, num_experts_per_tok=2, num_dense_layers=1, tie_word_embeddings=True),
    "mistral4": dict(model_type="mistral4", moe_intermediate_size=128, num_key_value_heads=4, n_routed_experts=8, n_shared_experts=1,
                     num_experts_per_tok=2, n_group=2, topk_group=1, first_k_dense_replace=1, q_lora_rank=64, kv_lora_rank=64,
                     qk_nope_head_dim=64, qk_rope_head_dim=64, v_head_dim=128),
    "granitemoeshared": dict(model_type="granitemoeshared", intermediate_size=128, shared_intermediate_size=256, num_local_experts=8,
                             num_experts_per_tok=2, tie_word_embeddings=True, embedding_multiplier=3.0, attention_multiplier=0.125,
                             residual_multiplier=0.5, logits_scaling=2.0),
}


@pytest.mark.parametrize("family", sorted(_GPU_FAMILIES))
def test_newer_families_on_the_device_match_cpu_fp32(family):
    """One forward / backward of each newer family in bf16 through the device kernels against the same weights in fp32
    on the CPU (packed documents; loss and two gradients)."""
    from axolotl_b200.models.config import ModelConfig
    from axolotl_b200.models.transformer import CausalLM
    torch.manual_seed(90)
    d = dict(vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, head_dim=64, tie_word_embeddings=False, max_position_embeddings=2048)
    d.update(_GPU_FAMILIES[family])
    cfg = ModelConfig.from_hf_dict(d)
    ref = CausalLM(cfg, dtype=torch.float32).init_weights(7)
    with torch.no_grad():
        if cfg.model_type == "gemma4_text":
            # Gemma 4 does not scale its scores: the learned q / k norm weights set their size. With the weights at one,
            # scores reach the head width (256, 512) and a bf16 rounding step of q or k moves a probability by a factor
            # of e; a trained checkpoint's scale (scores of order one) is what the comparison is about
            for l in ref.layers:
                l.self_attn.q_norm.weight.fill_(l.self_attn.D ** -0.25)
                l.self_attn.k_norm.weight.fill_(l.self_attn.D ** -0.25)
        for p in ref.parameters():
            p.copy_(p.bfloat16().float())
    dev = CausalLM(cfg, dtype=torch.bfloat16, device=_dev())
    dev.load_state_dict(ref.state_dict())
    lens = [150, 234]
    ids = torch.cat([torch.randint(3, cfg.vocab_size, (l,)) for l in lens])[None]
    pos = torch.cat([torch.arange(l) for l in lens])[None].to(torch.int32)
    out_d = dev(ids, pos, ids.clone())
    out_d.loss.backward()
    _check_status()
    out_c = ref(ids, pos, ids.clone())
    out_c.loss.backward()
    assert abs(out_d.loss.item() - out_c.loss.item()) < 3e-2 * abs(out_c.loss.item()), (out_d.loss.item(), out_c.loss.item())
    gd = dev.embed_tokens.grad.float().cpu()
    assert _rel_err(gd, ref.embed_tokens.grad) < 0.15, _rel_err(gd, ref.embed_tokens.grad)
    name = next(n for n, p in ref.named_parameters() if n.startswith("layers.0.") and p.dim() == 2 and p.grad is not None)
    gl = dict(dev.named_parameters())[name].grad.float().cpu()
    assert _rel_err(gl, dict(ref.named_parameters())[name].grad) < 0.15, name


@pytest.mark.parametrize("has_res,has_w,has_b,offset", [(True, True, True, 0.0), (False, True, False, 0.0), (True, False, False, 0.0),
                                                         (True, True, True, 1.0)])
def test_add_layernorm_kernel_matches_fp32_reference(has_res, has_w, has_b, offset):
    from axolotl_b200.ops import functional as Fn
    torch.manual_seed(95)
    T, D = 777, 2560
    x = (torch.randn(T, D, device="cuda") * 2 + 0.5).bfloat16().requires_grad_(True)
    r = torch.randn(T, D, device="cuda").bfloat16().requires_grad_(True) if has_res else None
    w = (torch.rand(D, device="cuda") + 0.5 - offset).bfloat16().requires_grad_(True) if has_w else None
    b = (torch.randn(D, device="cuda") * 0.2).bfloat16().requires_grad_(True) if has_b else None
    y, s = Fn.add_layernorm(x, r, w, b, 1e-5, offset)
    gy, gs = torch.randn_like(y), torch.randn_like(y)
    (y.float() * gy.float()).sum().add((s.float() * gs.float()).sum() if has_res else 0).backward()
    xc = x.detach().float().cpu().requires_grad_(True)
    rc = r.detach().float().cpu().requires_grad_(True) if has_res else None
    wc = w.detach().float().cpu().requires_grad_(True) if has_w else None
    bc = b.detach().float().cpu().requires_grad_(True) if has_b else None
    sc = xc + rc if has_res else xc
    sc_q = sc + (sc.detach().bfloat16().float() - sc.detach())        # the stream as stored (bf16), gradient straight through
    yc = torch.nn.functional.layer_norm(sc_q, (D,), (wc + offset) if has_w else None, bc, 1e-5)
    (yc * gy.float().cpu()).sum().add((sc * gs.float().cpu()).sum() if has_res else 0).backward()
    assert _rel_err(y.float().cpu(), yc) < 1e-2
    assert _rel_err(x.grad.float().cpu(), xc.grad) < 2e-2
    if has_res:
        assert _rel_err(r.grad.float().cpu(), rc.grad) < 2e-2
    if has_w:
        assert _rel_err(w.grad.float().cpu(), wc.grad) < 2e-2
    if has_b:
        assert _rel_err(b.grad.float().cpu(), bc.grad) < 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["llava", "gemma3"])
def test_image_front_ends_on_the_device_match_cpu_fp32(kind):
    """Vision tower + projector feeding image placeholder tokens of the language model: bf16 on the device (tower through
    library attention, language model through the tcgen05 GEMMs and, for LLaVA, the varlen attention kernels; Gemma 3's
    image batches take the blocked attention path for the both-ways mask inside an image) against fp32 on the CPU."""
    from axolotl_b200.models.config import ModelConfig
    from axolotl_b200.models.transformer import CausalLM
    torch.manual_seed(91)
    if kind == "llava":
        vc = dict(model_type="clip_vision_model", hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
                  image_size=56, patch_size=14, num_channels=3, hidden_act="quick_gelu", projection_dim=64)
        tc = dict(model_type="llama", vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=64, tie_word_embeddings=False, max_position_embeddings=2048)
        cfg = ModelConfig.from_hf_dict(dict(model_type="llava", text_config=tc, vision_config=vc, image_token_id=2047))
    else:
        vc = dict(model_type="siglip_vision_model", hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
                  image_size=56, patch_size=7, num_channels=3, hidden_act="gelu_pytorch_tanh")
        tc = dict(model_type="gemma3_text", vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=256, sliding_window=64, layer_types=["sliding_attention", "full_attention"],
                  query_pre_attn_scalar=256, max_position_embeddings=2048)
        cfg = ModelConfig.from_hf_dict(dict(model_type="gemma3", text_config=tc, vision_config=vc, mm_tokens_per_image=16, image_token_index=2047))
    ref = CausalLM(cfg, dtype=torch.float32).init_weights(7)
    with torch.no_grad():
        for p in ref.parameters():
            p.copy_(p.bfloat16().float())
    dev = CausalLM(cfg, dtype=torch.bfloat16, device=_dev())
    dev.load_state_dict(ref.state_dict())
    for m in (ref, dev):
        for p in m.vision.multi_modal_projector.parameters():
            p.requires_grad_(True)
    pixels = torch.randn(2, 3, 56, 56).bfloat16().float()
    rows = [torch.cat([torch.randint(3, 2000, (40,)), torch.full((16,), 2047), torch.randint(3, 2000, (90,))]) for _ in range(2)]
    ids = torch.cat(rows)[None]
    pos = torch.cat([torch.arange(len(r)) for r in rows])[None].to(torch.int32)
    labels = ids.clone()
    labels[ids == 2047] = -100
    out_d = dev(ids, pos, labels, pixel_values=pixels)
    out_d.loss.backward()
    _check_status()
    out_c = ref(ids, pos, labels, pixel_values=pixels)
    out_c.loss.backward()
    assert abs(out_d.loss.item() - out_c.loss.item()) < 3e-2 * abs(out_c.loss.item()), (out_d.loss.item(), out_c.loss.item())
    proj = (lambda m: m.vision.multi_modal_projector.linear_2.weight) if kind == "llava" else \
        (lambda m: m.vision.multi_modal_projector.mm_input_projection_weight)
    gd, gc = proj(dev).grad.float().cpu(), proj(ref).grad
    assert _rel_err(gd, gc) < 0.15, _rel_err(gd, gc)


@pytest.mark.gpu
@pytest.mark.parametrize("iters", [1, 20])
def test_hyperconnection_mixer_kernel_matches_reference(iters):
    """Sinkhorn mixer kernel pair (a token's 4 x 4 matrix in registers through the whole chain; the backward walks the
    chain back from the stored sums) against autograd through the plain fp32 form."""
    from axolotl_b200.ops import functional as Fn
    torch.manual_seed(92)
    M = 1000
    mixes = (torch.randn(M, 24) * 2).to(_dev())
    scale = torch.tensor([0.7, 1.3, 0.9], device=_dev())
    base = (torch.randn(24) * 0.3).to(_dev())
    wp, wq, wc = (torch.randn(M, 4, device=_dev()), torch.randn(M, 4, device=_dev()), torch.randn(M, 4, 4, device=_dev()))
    outs = []
    for fn in (Fn.sinkhorn_mix, Fn.sinkhorn_mix_ref):
        a, s, b = (t.clone().requires_grad_(True) for t in (mixes, scale, base))
        pre, post, comb = fn(a, s, b, 4, iters, 1e-6, 2.0)
        ((pre * wp).sum() + (post * wq).sum() + (comb * wc).sum()).backward()
        outs.append((pre, post, comb, a.grad, s.grad, b.grad))
    _check_status()
    for got, want in zip(*outs):
        assert _rel_err(got.float().cpu(), want.float().cpu()) < 2e-4, _rel_err(got.float().cpu(), want.float().cpu())
