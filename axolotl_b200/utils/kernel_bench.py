"""Kernel micro-benchmarks with roofline fractions.

``python -m axolotl_b200.utils.kernel_bench [gemm|lora|attn|decode|elementwise|all]`` times each hand-written
kernel with CUDA events (after warm-up, L2 flushed between iterations) and prints achieved
TFLOP/s or GB/s next to the library kernel for the same shape (cuBLAS via torch.matmul,
flash-attn 2 where installed) and the measured peaks in ``MEASURED_PEAKS.json`` if present.
"""
from __future__ import annotations

import json
import os
import sys

import torch


def _peaks():
    for p in ("MEASURED_PEAKS.json", os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")):
        if os.path.exists(p):
            with open(p) as fh:
                d = json.load(fh)
            return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    return 1590.0, 6650.0, "fallback"


_flush = None


def time_cuda(fn, iters=10, warmup=3, flush_l2=True):
    """Median milliseconds of ``fn`` on the current stream."""
    global _flush
    if flush_l2 and _flush is None:
        _flush = torch.empty(256 * 1024 * 1024, dtype=torch.int8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush_l2:
            _flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def bench_gemm(rows):
    from axolotl_b200.ops.gemm import gemm

    peak, _, how = _peaks()
    shapes = [
        ("qkv  8B", 8192, 6144, 4096, False), ("o    8B", 8192, 4096, 4096, False),
        ("gate_up", 8192, 28672, 4096, False), ("down   ", 8192, 4096, 14336, False),
        ("dX gu  ", 8192, 4096, 28672, True), ("dX down", 8192, 14336, 4096, True),
        ("lm_head", 2048, 128256, 4096, False), ("square ", 8192, 8192, 8192, False),
    ]
    for name, M, N, K, tb in shapes:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn((K, N) if tb else (N, K), device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ours = time_cuda(lambda: gemm(a, b, trans_b=tb, out=out))
        lib = time_cuda(lambda: torch.matmul(a, b if tb else b.t(), out=out))
        fl = 2.0 * M * N * K / 1e9
        rows.append(f"gemm {name} M={M} N={N} K={K} transB={int(tb)}: ours {ours:.3f} ms "
                    f"{fl / ours:.0f} TFLOP/s ({fl / ours / peak:.2f} of {how} peak) | cuBLAS {lib:.3f} ms "
                    f"{fl / lib:.0f} TFLOP/s | ratio {lib / ours:.2f}")


def bench_gemm_sustained(rows, seconds=2.0):
    """Every large GEMM shape of a Llama-3-8B LoRA step run back to back for a couple of seconds: the
    rate under the board power limit, which is what a training step sees, next to cuBLAS driven the
    same way, for several rasterisation band heights of the CTA-pair kernel. SM clock and power are
    sampled meanwhile."""
    import subprocess
    import threading
    import time

    from axolotl_b200.ops import _lib
    from axolotl_b200.ops.gemm import gemm

    lib = _lib.cuda_lib()

    def sample(stop, out):
        while not stop.is_set():
            try:
                r = subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm,power.draw", "--format=csv,noheader,nounits",
                                    "-i", str(torch.cuda.current_device())], capture_output=True, text=True, timeout=5)
                a, b = r.stdout.strip().split(",")
                out.append((float(a), float(b)))
            except Exception:
                pass
            time.sleep(0.2)

    def run(fn, fl):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        stop, samples = threading.Event(), []
        th = threading.Thread(target=sample, args=(stop, samples), daemon=True)
        th.start()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n, t0 = 0, time.perf_counter()
        s.record()
        while time.perf_counter() - t0 < seconds:
            for _ in range(20):
                fn()
            n += 20
            torch.cuda.synchronize()
        e.record()
        torch.cuda.synchronize()
        stop.set()
        th.join()
        ms = s.elapsed_time(e) / n
        samples = samples[len(samples) // 3:] or [(0.0, 0.0)]
        clk = sorted(c for c, _ in samples)[len(samples) // 2]
        return fl / ms / 1e9, clk

    shapes = [("qkv", 8192, 6144, 4096, False), ("gate_up", 8192, 28672, 4096, False), ("down", 8192, 4096, 14336, False),
              ("dX gate_up", 8192, 4096, 28672, True), ("dX down", 8192, 14336, 4096, True),
              ("lm_head", 2048, 128256, 4096, False)]
    bands = (2, 4, 8, 12, 16, 24)
    for name, M, N, K, tb in shapes:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn((K, N) if tb else (N, K), device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        fl = 2.0 * M * N * K
        ref, rclk = run(lambda: torch.matmul(a, b if tb else b.t(), out=out), fl)
        cells = []
        for g in bands:
            lib.axb_gemm_set_pair_tuning(g, 1, 0)
            t, clk = run(lambda: gemm(a, b, trans_b=tb, out=out), fl)
            cells.append(f"{g}: {t:.0f} @{clk:.0f}")
        lib.axb_gemm_set_pair_tuning(0, 1, 0)
        t, clk = run(lambda: gemm(a, b, trans_b=tb, out=out), fl)
        rows.append(f"sustained {name} M={M} N={N} K={K}: cuBLAS {ref:.0f} TFLOP/s @{rclk:.0f} MHz | ours by band height "
                    f"[{' | '.join(cells)}] | default {t:.0f} @{clk:.0f} ({t / ref:.2f} of cuBLAS)")
        del a, b, out


def bench_glu_mlp(rows):
    """One Llama-3-8B MLP with LoRA, forward + backward: GLU in the GEMM epilogues against the
    projection-by-projection path with stand-alone GLU kernels."""
    from axolotl_b200.models.transformer import MLP
    from axolotl_b200.ops import gemm as gemm_mod

    T, H, I = 8192, 4096, 14336
    mlp = MLP(H, I, "silu", False, torch.bfloat16, "cuda")
    with torch.no_grad():
        mlp.gate_up_proj.weight.normal_(0, 0.02)
        mlp.down_proj.weight.normal_(0, 0.02)
    for m in (mlp.gate_up_proj, mlp.down_proj):
        m.weight.requires_grad_(False)
        m.add_lora(16, 32, init_b_zero=False)
    x = (torch.randn(T, H, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    dy = (torch.randn(T, H, device="cuda") * 0.1).bfloat16()
    params = [p for p in mlp.parameters() if p.requires_grad]

    def step():
        torch.autograd.grad(mlp(x), [x] + params, dy)

    prev = gemm_mod.USE_GLU_EPILOGUE
    for flag in (True, False):
        gemm_mod.USE_GLU_EPILOGUE = flag
        ms = time_cuda(step)
        rows.append(f"mlp fwd+bwd LoRA r16 T={T} (GLU {'in GEMM epilogues' if flag else 'as kernels'}): {ms:.3f} ms")
    gemm_mod.USE_GLU_EPILOGUE = prev
    # the two GEMMs that carry the GLU, alone
    from axolotl_b200.ops.gemm import gemm

    Wgu, Wd = mlp.gate_up_proj.weight, mlp.down_proj.weight
    xd = x.detach()
    gu = torch.empty(T, 2 * I, device="cuda", dtype=torch.bfloat16)
    h = torch.empty(T, I, device="cuda", dtype=torch.bfloat16)
    dgu = torch.empty_like(gu)
    dh = torch.empty_like(h)
    gemm(xd, Wgu, out=gu)
    t0 = time_cuda(lambda: gemm(xd, Wgu, out=gu))
    gemm_mod.USE_GLU_EPILOGUE = True
    t1 = time_cuda(lambda: gemm(xd, Wgu, out=gu, glu=("fwd", 0, 0.0, h)))
    t2 = time_cuda(lambda: gemm(dy, Wd, trans_b=True, out=dh))
    t3 = time_cuda(lambda: gemm(dy, Wd, trans_b=True, out=dgu, glu=("bwd", 0, 0.0, gu)))
    gemm_mod.USE_GLU_EPILOGUE = prev
    from axolotl_b200.ops import functional as Fn

    t4 = time_cuda(lambda: Fn.glu(gu))
    rows.append(f"gate|up GEMM {t0:.3f} ms, with GLU epilogue {t1:.3f} ms | dX(down) GEMM {t2:.3f} ms, with GLU-backward "
                f"epilogue {t3:.3f} ms | stand-alone GLU forward kernel {t4:.3f} ms")


def bench_lora_skinny(rows):
    """The adapter-side GEMMs of one LoRA projection: memory-bound passes over x or dy."""
    from axolotl_b200.ops.gemm import gemm, pick_splits

    _, hbm, how = _peaks()
    T = 8192
    cases = [("qkv", 4096, 6144, 48), ("o", 4096, 4096, 16), ("gate_up", 4096, 28672, 32), ("down", 14336, 4096, 16)]
    for name, K, N, R in cases:
        x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
        dy = torch.randn(T, N, device="cuda", dtype=torch.bfloat16)
        A = torch.randn(R, K, device="cuda", dtype=torch.bfloat16)
        B = torch.randn(N, R, device="cuda", dtype=torch.bfloat16)
        xa = torch.randn(T, R, device="cuda", dtype=torch.bfloat16)
        dA = torch.zeros(R, K, device="cuda", dtype=torch.float32)
        dB = torch.zeros(N, R, device="cuda", dtype=torch.float32)
        from axolotl_b200.ops import lora as _lora

        t_xa = time_cuda(lambda: gemm(x, A))
        t_t = time_cuda(lambda: gemm(dy, B, trans_b=True))
        split_note = ""
        for sp in (2, 4):
            _lora.SKINNY_SPLITS = sp
            a_ = time_cuda(lambda: _lora.skinny_gemm(x, A))
            b_ = time_cuda(lambda: _lora.skinny_gemm(dy, B, trans_b=True))
            split_note += f" | split-K {sp}: x@A^T {a_ * 1e3:.0f} us, dy@B {b_ * 1e3:.0f} us"
        _lora.SKINNY_SPLITS = 0
        sp_a = pick_splits((K + 255) // 256, (T + 63) // 64)
        t_dA = time_cuda(lambda: gemm(xa, x, trans_a=True, trans_b=True, out=dA, accumulate=True, splits=sp_a))
        sp_b = pick_splits((N + 127) // 128, (T + 63) // 64)
        t_dB = time_cuda(lambda: gemm(dy, xa, trans_a=True, trans_b=True, out=dB, accumulate=True, splits=sp_b, bn=64))
        nb = 3 if name == "qkv" else (2 if name == "gate_up" else 1)
        blocks = [(i * (N // nb), N // nb, i * (R // nb), R // nb) for i in range(nb)]
        t_fused = time_cuda(lambda: _lora.lora_bwd_dy(dy, B, xa, blocks, 2.0, dB))
        gb = lambda elems, ms: elems * 2 / 1e6 / ms   # GB/s
        rows.append(f"lora {name} r={R}: x@A^T {t_xa * 1e3:.0f} us ({gb(T * K, t_xa) / hbm:.2f}) | dy@B {t_t * 1e3:.0f} us "
                    f"({gb(T * N, t_t) / hbm:.2f}) | dA=t^T x {t_dA * 1e3:.0f} us ({gb(T * K, t_dA) / hbm:.2f}, splits {sp_a}) | "
                    f"dB=dy^T xa {t_dB * 1e3:.0f} us ({gb(T * N, t_dB) / hbm:.2f}, splits {sp_b}) | ONE pass over dy for "
                    f"both (incl. memset + cast): {t_fused * 1e3:.0f} us ({gb(T * N, t_fused) / hbm:.2f}){split_note}  "
                    f"[fractions of {how} HBM copy rate]")


def bench_w4a16(rows):
    """NVFP4 expert projections at Qwen3-30B-A3B shapes (128 experts, hidden 2048, expert width 768, 8192 tokens
    x top-8 = 512 rows per expert): decode inside the grouped GEMM against dequantise-then-GEMM."""
    from axolotl_b200.ops.grouped import GroupLayout, _lib as L, grouped_gemm, grouped_gemm_w4a16
    tf, bw, src = _peaks()
    E, H, I, per = 128, 2048, 768, 512
    dev = "cuda"
    lay = GroupLayout(torch.full((E,), per, device=dev), E * per)
    for name, N, K in (("gate_up", 2 * I, H), ("down", H, I)):
        q = {"qdata": torch.randint(0, 256, (E, N, K // 2), dtype=torch.uint8, device=dev),
             "scale": torch.randint(40, 120, (E, N, K // 16), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn),
             "pts": torch.full((E,), 1e-3, device=dev)}
        Wd = torch.empty(E, N, K, dtype=torch.bfloat16, device=dev)
        pts = q["pts"].float()

        def deq():
            L.check_rc(L.cuda_lib().axb_nvfp4_dequant_batched(q["qdata"].data_ptr(), q["scale"].data_ptr(), pts.data_ptr(),
                                                              Wd.data_ptr(), E, N, K, None, L.stream_ptr()), "dequant")
        x = torch.randn(lay.max_rows, K, device=dev).bfloat16()
        dy = torch.randn(lay.max_rows, N, device=dev).bfloat16()
        deq()
        fl = 2.0 * E * per * N * K
        t_deq = time_cuda(deq)
        t_f16 = time_cuda(lambda: grouped_gemm(x, Wd, lay))
        t_f4 = time_cuda(lambda: grouped_gemm_w4a16(x, q, lay))
        t_b16 = time_cuda(lambda: grouped_gemm(dy, Wd, lay, trans_w=True))
        t_b4 = time_cuda(lambda: grouped_gemm_w4a16(dy, q, lay, trans_w=True))
        rows.append(f"w4a16 {name} [E={E}, N={N}, K={K}] x {per} rows/expert: dequant {t_deq*1e3:.0f} us | fwd bf16-stack "
                    f"{t_f16*1e3:.0f} us, in-kernel decode {t_f4*1e3:.0f} us ({fl/t_f4/1e9/tf:.2f} of {src} bf16 peak) | "
                    f"dX bf16-stack {t_b16*1e3:.0f} us, in-kernel decode {t_b4*1e3:.0f} us ({fl/t_b4/1e9/tf:.2f}) | "
                    f"fwd+dX: {2*t_deq*1e3 + t_f16*1e3 + t_b16*1e3:.0f} us (dequantise twice + GEMMs) -> {t_f4*1e3 + t_b4*1e3:.0f} us")


def bench_decode(rows):
    """Single-query attention over a KV cache (memory-bound: one pass over the live cache) and
    end-to-end KV-cache generation on a randomly initialised Llama-3-8B."""
    import time

    from axolotl_b200.ops.functional import decode_attention

    _, hbm, how = _peaks()
    Hq, Hk, D = 32, 8, 128
    for B, n in ((8, 4096), (64, 4096), (64, 16384)):
        lens = torch.full((B,), n, dtype=torch.int32, device="cuda")
        qkv = torch.randn(B, (Hq + 2 * Hk) * D, device="cuda", dtype=torch.bfloat16)
        kc = torch.randn(B, n, Hk * D, device="cuda", dtype=torch.bfloat16)
        vc = torch.randn(B, n, Hk * D, device="cuda", dtype=torch.bfloat16)
        ms = time_cuda(lambda: decode_attention(qkv, kc, vc, lens, Hq, Hk, D))
        gbs = 2 * B * n * Hk * D * 2 / 1e6 / ms
        rows.append(f"decode attn B={B} len={n}: {ms * 1e3:.0f} us, {gbs:.0f} GB/s of cache ({gbs / hbm:.2f} of {how} HBM copy rate)")
        del kc, vc
    from axolotl_b200.models.config import preset
    from axolotl_b200.models.kv_cache import generate_cached
    from axolotl_b200.models.transformer import CausalLM

    model = CausalLM(preset("llama-3-8b"), dtype=torch.bfloat16, device="cuda").init_weights(0)
    for B, plen, new in ((8, 512, 64), (64, 512, 64)):
        prompts = [[1] + [100 + (i * 7 + j) % 1000 for j in range(plen - 1)] for i in range(B)]
        generate_cached(model, prompts[:8], 4)     # warm-up
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        generate_cached(model, prompts, new)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        rows.append(f"generate llama-3-8b B={B} prompt={plen} new={new}: {dt:.2f} s, {B * new / dt:.0f} new tokens/s "
                    f"(prefill included)")


def bench_attn_wide(rows):
    """Wide-head attention (csrc/flash_wide.cu): head width 256 (Gemma, with and without the soft cap) and 192/128
    (latent attention), causal packed documents; against flash-attn 2 where it takes the shape."""
    from axolotl_b200.ops.functional import AttnMeta, flash_varlen

    try:
        from flash_attn import flash_attn_varlen_func
    except Exception:  # pragma: no cover
        flash_attn_varlen_func = None
    tf, _, src = _peaks()
    for name, Hq, Hk, D, Dv, cap, lens in (("gemma 256/256", 16, 8, 256, 256, 0.0, [2048] * 4),
                                           ("gemma-2 256/256 softcap 50", 16, 8, 256, 256, 50.0, [2048] * 4),
                                           ("gemma 256/256 one 8192 doc", 16, 8, 256, 256, 0.0, [8192]),
                                           ("latent 192/128", 32, 32, 192, 128, 0.0, [2048] * 4)):
        cu = [0]
        for l in lens:
            cu.append(cu[-1] + l)
        T = cu[-1]
        meta = AttnMeta(cu, "cuda")
        qkv = (torch.randn(T, Hq * D + Hk * D + Hk * Dv, device="cuda") * 0.5).bfloat16().requires_grad_(True)
        g = torch.randn(T, Hq * Dv, device="cuda", dtype=torch.bfloat16)
        fl = sum(2.0 * Hq * l * l * (D + Dv) / 2 for l in lens)          # causal: half of the full square
        t_f = time_cuda(lambda: flash_varlen(qkv, meta, Hq, Hk, D, Dv=Dv, softcap=cap))
        out = flash_varlen(qkv, meta, Hq, Hk, D, Dv=Dv, softcap=cap)
        t_b = time_cuda(lambda: torch.autograd.grad(out, qkv, g, retain_graph=True))
        line = (f"attn wide {name}, {len(lens)} x {lens[0]} tokens, Hq={Hq} Hk={Hk}: fwd {t_f*1e3:.0f} us "
                f"({fl / t_f / 1e9:.0f} TFLOP/s, {fl / t_f / 1e9 / tf:.2f} of {src} bf16 peak) | bwd {t_b*1e3:.0f} us "
                f"({2.5 * fl / t_b / 1e9:.0f} TFLOP/s)")
        if flash_attn_varlen_func is not None and D == Dv and not cap:
            q = qkv.detach()[:, : Hq * D].reshape(T, Hq, D).contiguous().requires_grad_(True)
            k = qkv.detach()[:, Hq * D:(Hq + Hk) * D].reshape(T, Hk, D).contiguous().requires_grad_(True)
            v = qkv.detach()[:, (Hq + Hk) * D:].reshape(T, Hk, Dv).contiguous().requires_grad_(True)
            cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
            try:
                f2 = lambda: flash_attn_varlen_func(q, k, v, cu_t, cu_t, max(lens), max(lens), causal=True)
                t2 = time_cuda(f2)
                o2 = f2()
                t2b = time_cuda(lambda: torch.autograd.grad(o2, (q, k, v), g.view(T, Hq, Dv), retain_graph=True))
                line += f" | flash-attn 2: fwd {t2*1e3:.0f} us, bwd {t2b*1e3:.0f} us"
            except Exception as e:  # noqa: BLE001
                line += f" | flash-attn 2: {type(e).__name__}"
        rows.append(line)


def bench_indexer(rows):
    """Lightning-indexer scores (csrc/indexer.cu) of one document against the einsum form that holds the per-head
    scores (queries in blocks of 512 so that [512, H, L] fp32 fits)."""
    from axolotl_b200.models import dsa

    tf, hbm, src = _peaks()
    for L, H in ((8192, 32), (16384, 32), (8192, 64)):
        q = torch.randn(L, H, 128, device="cuda").bfloat16()
        k = torch.randn(L, 128, device="cuda").bfloat16()
        w = torch.randn(L, H, device="cuda") * 0.1
        fl = 2.0 * L * H * 128 * L / 2                                   # causal half of the square
        t = time_cuda(lambda: dsa.indexer_scores(q, k, w))
        fill = time_cuda(lambda: torch.full((L, L), float("-inf"), dtype=torch.float32, device="cuda"))

        def eager():
            for b0 in range(0, L, 512):
                dsa.indexer_scores_ref(q[b0:b0 + 512], k[: b0 + 512], w[b0:b0 + 512], causal_off=b0)
        t_e = time_cuda(eager, iters=3, warmup=1)
        t_k = max(t - fill, 1e-6)
        rows.append(f"indexer scores L={L} H={H}: {t*1e3:.0f} us with the -inf fill of the output ({fill*1e3:.0f} us), kernel "
                    f"{fl / t_k / 1e9:.0f} TFLOP/s ({fl / t_k / 1e9 / tf:.2f} of {src} bf16 peak), output "
                    f"{L * L * 2 / t_k / 1e6:.0f} GB/s | einsum form {t_e*1e3:.0f} us ({t_e / t:.1f}x)")


def bench_hyperconnection(rows):
    """The DeepSeek-V4 hyper-connection mixer (sigmoid / softmax / 20-step Sinkhorn over one 4 x 4 matrix per token) at
    8192 and 65536 tokens: the register-resident kernel pair against the eager chain of ~40 small launches."""
    from axolotl_b200.ops import functional as Fn

    scale = torch.tensor([0.7, 1.3, 0.9], device="cuda")
    base = torch.randn(24, device="cuda") * 0.3
    for M in (8192, 65536):
        mixes = (torch.randn(M, 24, device="cuda") * 2).requires_grad_(True)
        w = torch.randn(M, 4, 4, device="cuda")
        for name, fn in (("kernel", Fn.sinkhorn_mix), ("eager", Fn.sinkhorn_mix_ref)):
            f = lambda: fn(mixes, scale, base, 4, 20, 1e-6, 2.0)
            t_f = time_cuda(f, iters=20, warmup=5)
            t_fb = time_cuda(lambda: torch.autograd.grad((f()[2] * w).sum() + f()[0].sum(), mixes), iters=20, warmup=5)
            rows.append(f"hyper-connection mixer, {M} tokens, 20 Sinkhorn steps, {name}: fwd {t_f * 1e3:.1f} us, fwd+bwd {t_fb * 1e3:.1f} us")


def bench_mixers(rows):
    """The recurrent token mixers of the hybrid families at one 8192-token row (four 2048-token documents): the
    Mamba-2 chunked scan and the gated delta rule, both written as dense tensor contractions (library batched GEMMs),
    forward and forward + backward; flash-linear-attention's Triton kernel for the delta rule beside it for context."""
    from axolotl_b200.models.deltanet import gated_delta_rule, gated_delta_rule_packed
    from axolotl_b200.models.mamba import ssd_chunked, ssd_packed

    L, docs = 2048, 4
    # Granite-4.0-H-small-like mixer: 128 heads x 64, state 128
    h, P, N = 128, 64, 128
    xd = (torch.randn(docs * L, h, P, device="cuda") * 0.5).requires_grad_(True)
    a = -torch.rand(docs * L, h, device="cuda") * 0.1
    B = torch.randn(docs * L, h, N, device="cuda") * 0.3
    C = torch.randn(docs * L, h, N, device="cuda") * 0.3

    def scan():
        return torch.cat([ssd_chunked(xd[i * L:(i + 1) * L], a[i * L:(i + 1) * L], B[i * L:(i + 1) * L], C[i * L:(i + 1) * L], 256)
                          for i in range(docs)], 0)
    t_f = time_cuda(scan, iters=5, warmup=2)
    t_fb = time_cuda(lambda: torch.autograd.grad(scan().sum(), xd), iters=5, warmup=2)
    fl = 2.0 * docs * L * h * (256 * (N + P) + 2 * N * P)          # intra-chunk scores + outputs, state update + read-out
    rows.append(f"mamba-2 scan h={h} P={P} N={N}, {docs} x {L} tokens, per document, chunk 256, fp32 contractions: fwd {t_f:.2f} ms "
                f"({fl / t_f / 1e9:.0f} TFLOP/s), fwd+bwd {t_fb:.2f} ms")
    cu = [i * L for i in range(docs + 1)]
    Bg, Cg = B[:, ::16].contiguous(), C[:, ::16].contiguous()               # 8 groups of 16 heads, as the checkpoints have
    for lowp, tag in ((None, "fp32"), (torch.bfloat16, "bf16 operands")):
        f = lambda: ssd_packed(xd, a, Bg, Cg, cu, 128, lowp)
        t_f = time_cuda(f, iters=5, warmup=2)
        t_fb = time_cuda(lambda: torch.autograd.grad(f().sum(), xd), iters=5, warmup=2)
        rows.append(f"mamba-2 scan, whole row in one batched pass, chunk 128, {tag}: fwd {t_f:.2f} ms, fwd+bwd {t_fb:.2f} ms")
    # Qwen3-Next-like DeltaNet: 32 value heads, 128-wide keys and values
    hv, dk, dv = 32, 128, 128
    q = torch.nn.functional.normalize(torch.randn(docs * L, hv, dk, device="cuda"), dim=-1).requires_grad_(True)
    k = torch.nn.functional.normalize(torch.randn(docs * L, hv, dk, device="cuda"), dim=-1)
    v = torch.randn(docs * L, hv, dv, device="cuda")
    g = -torch.rand(docs * L, hv, device="cuda") * 0.1
    beta = torch.rand(docs * L, hv, device="cuda")

    def delta():
        return torch.cat([gated_delta_rule(q[i * L:(i + 1) * L], k[i * L:(i + 1) * L], v[i * L:(i + 1) * L], g[i * L:(i + 1) * L],
                                           beta[i * L:(i + 1) * L]) for i in range(docs)], 0)
    t_f = time_cuda(delta, iters=5, warmup=2)
    t_fb = time_cuda(lambda: torch.autograd.grad(delta().sum(), q), iters=5, warmup=2)
    line = f"gated delta rule hv={hv} dk={dk} dv={dv}, {docs} x {L} tokens, per document, fp32: fwd {t_f:.2f} ms, fwd+bwd {t_fb:.2f} ms"
    for lowp, tag in ((None, "fp32"), (torch.bfloat16, "bf16 operands")):
        f = lambda: gated_delta_rule_packed(q, k, v, g, beta, cu, 64, lowp)
        t_f = time_cuda(f, iters=5, warmup=2)
        t_fb = time_cuda(lambda: torch.autograd.grad(f().sum(), q), iters=5, warmup=2)
        line += f" | all documents together, {tag}: fwd {t_f:.2f} ms, fwd+bwd {t_fb:.2f} ms"
    try:
        from fla.ops.gated_delta_rule import chunk_gated_delta_rule

        cu = torch.arange(0, (docs + 1) * L, L, device="cuda", dtype=torch.int32)
        qb, kb, vb = (t.detach().bfloat16()[None] for t in (q, k, v))
        f2 = lambda: chunk_gated_delta_rule(qb, kb, vb, g[None], beta[None], scale=dk ** -0.5, cu_seqlens=cu.long())
        t2 = time_cuda(f2, iters=5, warmup=2)
        line += f" | flash-linear-attention (Triton, bf16): fwd {t2:.2f} ms"
    except Exception as e:  # noqa: BLE001
        line += f" | flash-linear-attention: {type(e).__name__}"
    rows.append(line)


def bench_attn(rows):
    from axolotl_b200.ops.functional import AttnMeta, flash_varlen

    try:
        from flash_attn import flash_attn_varlen_func
    except Exception:  # pragma: no cover
        flash_attn_varlen_func = None
    D = 128
    for Hq, Hk, lens in [(32, 8, [8192]), (32, 8, [2048] * 4), (32, 8, [4096, 1024, 3072]), (32, 8, [512] * 16),
                         (32, 4, [2048] * 4), (32, 4, [4096, 1024, 3072])]:
        cu = [0]
        for l in lens:
            cu.append(cu[-1] + l)
        T = cu[-1]
        meta = AttnMeta(cu, "cuda")
        qkv = (torch.randn(T, (Hq + 2 * Hk) * D, device="cuda") * 0.5).bfloat16().requires_grad_(True)
        g = torch.randn(T, Hq * D, device="cuda", dtype=torch.bfloat16)
        fl_f = sum(4.0 * l * l * D * Hq / 2 for l in lens) / 1e9
        fwd = time_cuda(lambda: flash_varlen(qkv.detach(), meta, Hq, Hk, D))
        out = flash_varlen(qkv, meta, Hq, Hk, D)
        bwd = time_cuda(lambda: torch.autograd.grad(out, qkv, g, retain_graph=True))
        line = (f"attn Hq={Hq} Hk={Hk} lens={lens if len(lens) < 5 else str(lens[0]) + 'x' + str(len(lens))}: fwd {fwd:.3f} ms "
                f"{fl_f / fwd:.0f} TFLOP/s, bwd {bwd:.3f} ms {2.5 * fl_f / bwd:.0f} TFLOP/s")
        if flash_attn_varlen_func is not None:
            q = qkv.detach()[:, :Hq * D].reshape(T, Hq, D).contiguous().requires_grad_(True)
            k = qkv.detach()[:, Hq * D:(Hq + Hk) * D].reshape(T, Hk, D).contiguous().requires_grad_(True)
            v = qkv.detach()[:, (Hq + Hk) * D:].reshape(T, Hk, D).contiguous().requires_grad_(True)
            cu_t = meta.cu_seqlens
            mx = max(lens)
            f2 = time_cuda(lambda: flash_attn_varlen_func(q, k, v, cu_t, cu_t, mx, mx, causal=True))
            o2 = flash_attn_varlen_func(q, k, v, cu_t, cu_t, mx, mx, causal=True)
            g2 = g.view(T, Hq, D)
            b2 = time_cuda(lambda: torch.autograd.grad(o2, (q, k, v), g2, retain_graph=True))
            line += f" | FA2 fwd {f2:.3f} ms bwd {b2:.3f} ms | ratio fwd {f2 / fwd:.2f} bwd {b2 / bwd:.2f}"
        rows.append(line)


def bench_elementwise(rows):
    from axolotl_b200.ops import functional as Fn

    _, hbm, how = _peaks()
    T, H, I = 8192, 4096, 14336
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    r = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    ms = time_cuda(lambda: Fn.add_rmsnorm(x, r, w, 1e-5))
    gb = 4 * T * H * 2 / 1e6
    rows.append(f"add_rmsnorm fwd [{T},{H}]: {ms:.3f} ms {gb / ms:.0f} GB/s ({gb / ms / hbm:.2f} of {how} HBM)")
    gu = torch.randn(T, 2 * I, device="cuda", dtype=torch.bfloat16)
    ms = time_cuda(lambda: Fn.glu(gu))
    gb = 3 * T * I * 2 / 1e6
    rows.append(f"swiglu fwd [{T},{2 * I}]: {ms:.3f} ms {gb / ms:.0f} GB/s ({gb / ms / hbm:.2f} of {how} HBM)")
    logits = torch.randn(2048, 128256, device="cuda", dtype=torch.bfloat16)
    labels = torch.randint(0, 128256, (2048,), device="cuda")
    loss = torch.empty(2048, device="cuda")
    from axolotl_b200.ops import _lib
    lib = _lib.cuda_lib()
    ms = time_cuda(lambda: lib.axb_ce_fwd_bwd(logits.data_ptr(), labels.data_ptr(), loss.data_ptr(), None,
                                               2048, 128256, 128256, 1.0, -100, 1, _lib.stream_ptr()))
    gb = 2 * 2048 * 128256 * 2 / 1e6
    rows.append(f"ce fwd+bwd [2048,128256]: {ms:.3f} ms {gb / ms:.0f} GB/s algorithmic ({gb / ms / hbm:.2f} of {how} HBM)")


def profile_case(what):
    """Small fixed workloads for `ncu` captures: a handful of launches, a few hundred MB."""
    from axolotl_b200.ops.functional import AttnMeta, flash_varlen
    from axolotl_b200.ops.gemm import gemm

    if what == "one_gemm":
        a = torch.randn(8192, 4096, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(6144, 4096, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(8192, 6144, device="cuda", dtype=torch.bfloat16)
        for _ in range(4):
            gemm(a, b, out=out)
    elif what == "one_mlp":
        # the two GEMMs of a Llama-3-8B MLP that carry the GLU in their epilogues (forward gate|up with
        # h = silu(gate) * up, backward dX(down) with d_gate | d_up), 4096 token rows
        from axolotl_b200.ops import gemm as gemm_mod

        gemm_mod.USE_GLU_EPILOGUE = True
        T, H, I = 4096, 4096, 14336
        x = (torch.randn(T, H, device="cuda") * 0.5).bfloat16()
        Wgu = (torch.randn(2 * I, H, device="cuda") * 0.02).bfloat16()
        Wd = (torch.randn(H, I, device="cuda") * 0.02).bfloat16()
        dy = (torch.randn(T, H, device="cuda") * 0.1).bfloat16()
        gu = torch.empty(T, 2 * I, device="cuda", dtype=torch.bfloat16)
        h = torch.empty(T, I, device="cuda", dtype=torch.bfloat16)
        dgu = torch.empty_like(gu)
        for _ in range(3):
            gemm(x, Wgu, out=gu, glu=("fwd", 0, 0.0, h))
            gemm(dy, Wd, trans_b=True, out=dgu, glu=("bwd", 0, 0.0, gu))
    elif what == "one_hyperconnection":
        # the hyper-connection mixer kernel pair at 1 M tokens (24 + 24 fp32 numbers per token and direction)
        from axolotl_b200.ops import functional as Fn

        M = 1 << 20
        mixes = (torch.randn(M, 24, device="cuda") * 2).requires_grad_(True)
        scale = torch.tensor([0.7, 1.3, 0.9], device="cuda")
        base = torch.randn(24, device="cuda") * 0.3
        for _ in range(3):
            pre, post, comb = Fn.sinkhorn_mix(mixes, scale, base, 4, 20, 1e-6, 2.0)
            torch.autograd.grad([pre, post, comb], mixes, [torch.ones_like(pre), torch.ones_like(post), torch.ones_like(comb)])
    elif what == "one_w4a16":
        # NVFP4 expert projection with the decode inside the grouped GEMM: 32 experts of Qwen3-MoE-30B-A3B's
        # gate|up shape, 512 rows each (forward and input gradient)
        from axolotl_b200.ops.grouped import GroupLayout, grouped_gemm_w4a16

        E, N, K, per = 32, 1536, 2048, 512
        lay = GroupLayout(torch.full((E,), per, device="cuda"), E * per)
        q = {"qdata": torch.randint(0, 256, (E, N, K // 2), dtype=torch.uint8, device="cuda"),
             "scale": torch.randint(40, 120, (E, N, K // 16), dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn),
             "pts": torch.full((E,), 1e-3, device="cuda")}
        x = torch.randn(lay.max_rows, K, device="cuda").bfloat16()
        dy = torch.randn(lay.max_rows, N, device="cuda").bfloat16()
        for _ in range(3):
            grouped_gemm_w4a16(x, q, lay)
            grouped_gemm_w4a16(dy, q, lay, trans_w=True)
    elif what == "one_indexer":
        from axolotl_b200.models import dsa

        L, H = 8192, 32
        q = torch.randn(L, H, 128, device="cuda").bfloat16()
        k = torch.randn(L, 128, device="cuda").bfloat16()
        w = torch.randn(L, H, device="cuda") * 0.1
        for _ in range(3):
            dsa.indexer_scores(q, k, w)
    elif what == "one_grouped":
        # one MoE projection of Qwen3-MoE-30B-A3B: 128 experts, 8192 tokens x top-8 = 65536 routed rows
        from axolotl_b200.ops.grouped import GroupLayout, grouped_gemm, grouped_gram

        E, H, I, r = 128, 2048, 768, 16
        g = torch.Generator(device="cuda").manual_seed(0)
        e_of_row = torch.randint(0, E, (65536,), device="cuda", generator=g)
        lay = GroupLayout(torch.bincount(e_of_row, minlength=E), 65536)
        x = (torch.randn(lay.max_rows, H, device="cuda") * 0.5).bfloat16()
        W = (torch.randn(E, 2 * I, H, device="cuda") * 0.02).bfloat16()
        t = (torch.randn(lay.max_rows, r, device="cuda") * 0.5).bfloat16()
        Bt = (torch.randn(E, 2 * I, r, device="cuda") * 0.02).bfloat16()
        gA = torch.zeros(E, r, H, device="cuda")
        for _ in range(3):
            y = grouped_gemm(x, W, lay, a2=t, w2=Bt)
            dx = grouped_gemm(y, W, lay, trans_w=True)
            grouped_gram(t, x, lay, gA)
    else:
        Hq, Hk, D = 32, 8, 128
        meta = AttnMeta([0, 2048, 4096, 6144, 8192], "cuda")
        qkv = (torch.randn(8192, (Hq + 2 * Hk) * D, device="cuda") * 0.5).bfloat16().requires_grad_(True)
        g = torch.randn(8192, Hq * D, device="cuda", dtype=torch.bfloat16)
        for _ in range(3):
            out = flash_varlen(qkv, meta, Hq, Hk, D)
            torch.autograd.grad(out, qkv, g)
    torch.cuda.synchronize()
    print("done", what)


def main(argv):
    what = argv[1] if len(argv) > 1 else "all"
    if what in ("one_gemm", "one_attn", "one_grouped", "one_mlp", "one_w4a16", "one_indexer", "one_hyperconnection"):
        return profile_case(what)
    rows = []
    if what in ("gemm", "all"):
        bench_gemm(rows)
    if what in ("sustained",):
        bench_gemm_sustained(rows)
    if what in ("mlp", "all"):
        bench_glu_mlp(rows)
    if what in ("lora", "all"):
        bench_lora_skinny(rows)
    if what in ("attn", "all"):
        bench_attn(rows)
    if what in ("decode",):
        bench_decode(rows)
    if what in ("w4a16",):
        bench_w4a16(rows)
    if what in ("attn_wide",):
        bench_attn_wide(rows)
    if what in ("indexer",):
        bench_indexer(rows)
    if what in ("mixers",):
        bench_mixers(rows)
    if what in ("hyperconnection",):
        bench_hyperconnection(rows)
    if what in ("elementwise", "all"):
        bench_elementwise(rows)
    from axolotl_b200.ops import _lib
    _lib.check_status()
    print("\n".join(rows))


if __name__ == "__main__":
    main(sys.argv)
