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


@pytest.mark.parametrize("D,Hq,Hk", [(128, 4, 2), (64, 4, 2), (128, 8, 8)])
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
