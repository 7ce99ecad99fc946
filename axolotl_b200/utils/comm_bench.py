"""Device-timed micro-benchmarks of the fused compute + collective paths, one process per GPU:

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m axolotl_b200.utils.comm_bench

Every number is CUDA-event time, max over ranks, after warm-up. For each path the line reports the
achieved rate and its fraction of the roofline = the slower of (FLOPs / measured GEMM peak) and
(bytes that must cross NVLink per GPU / per-direction link bandwidth). Peaks are read from
MEASURED_PEAKS.json at the repository root when present (fallback: 1.59 PFLOP/s); the NVLink
reference is the measured peer-copy figure of 770 GB/s per direction per GPU.
"""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _peak_tflops():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(p) as fh:
            return float(json.load(fh)["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


def timed(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    from axolotl_b200.models.layers import FusedLinear
    from axolotl_b200.ops import _lib
    from axolotl_b200.ops.gemm import gemm
    from axolotl_b200.parallel.fsdp import FSDPContext
    from axolotl_b200.parallel.mesh import DeviceMesh, MeshSpec
    from axolotl_b200.parallel.runtime import ParallelRuntime
    from axolotl_b200.parallel.tp import TPContext
    from axolotl_b200.train.optimizer import FlatAdamW

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    peak, how = _peak_tflops()
    out = []
    M = 8192

    # ---- 1. FSDP: GEMMs of one Llama-3-8B layer against row-sharded weights; spare CTAs of every
    # launch all-gather the next weight. Compare with the same GEMMs on local full weights.
    shapes = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)]
    mods = []
    for N, K in shapes:
        m = FusedLinear(K, [N], ["w"], device=dev)
        torch.nn.init.normal_(m.weight, std=0.02)
        m.weight.requires_grad_(False)
        mods.append(m)
    full = [m.weight.detach().clone() for m in mods]

    class Holder:
        def fused_linears(self):
            return [(str(i), m) for i, m in enumerate(mods)]

    ctx = FSDPContext(dev, dist.group.WORLD, world, rank)
    ctx.shard_model(Holder())
    xs = [torch.randn(M, K, device=dev, dtype=torch.bfloat16) for _, K in shapes]
    t_plain = timed(lambda: [gemm(x, w) for x, w in zip(xs, full)])
    t_shard = timed(lambda: [gemm(x, m.weight) for x, m in zip(xs, mods)])
    flops = sum(2.0 * M * N * K for N, K in shapes)
    gathered = sum(N * K * 2 for N, K in shapes) * (world - 1) / world
    roof = max(flops / (peak * 1e12), gathered / (NVLINK_GBS * 1e9)) * 1e3
    out.append(f"fsdp all-gather fused into GEMM (one 8B layer fwd, M={M}): local weights {t_plain:.3f} ms, sharded + prefetch "
               f"{t_shard:.3f} ms ({flops / t_shard / 1e9:.0f} TFLOP/s; {gathered / 1e6:.0f} MB over NVLink per GPU hidden behind the MMAs); "
               f"roofline {roof:.3f} ms -> {roof / t_shard:.2f} of {how} roofline; overhead vs local weights {100 * (t_shard / t_plain - 1):.1f} %")

    # ---- 2. reduce-scatter + AdamW + all-gather of a flat fp32 gradient buffer (LoRA-sized and large)
    for n in (42_000_000, 512_000_000):
        n = n // (8 * world) * (8 * world)
        p = torch.nn.Parameter(torch.zeros(n, device=dev))
        rt = ParallelRuntime(DeviceMesh(MeshSpec.from_cfg(world), rank), dev, "fused")
        opt = FlatAdamW([{"name": "g", "params": [("p", p)], "lr_scale": 1.0, "weight_decay": 0.0}], lr=1e-3,
                        max_grad_norm=1.0, alloc=rt.optimizer_alloc(), pad_multiple=8 * world, moment_shard=rt.moment_shard())
        rt.attach_optimizer(opt)
        p._axb_grad.normal_()
        t = timed(lambda: rt.optimizer_step(opt, 1e-3), iters=5)
        # per GPU over NVLink: reads (world-1)/world of the fp32 gradient slice owners need, writes its
        # updated slice (fp32 master + bf16 shadow) to the world-1 peers
        link = n * 4 * (world - 1) / world + (n / world) * 6 * (world - 1)
        local = n * 4 * 2 + (n / world) * (4 * 6)          # clear + read grad, moments and master traffic
        roof = max(link / (NVLINK_GBS * 1e9), 0.0) * 1e3
        out.append(f"reduce-scatter + AdamW + all-gather, {n / 1e6:.0f} M fp32 elements: {t:.3f} ms "
                   f"({link / t / 1e6:.0f} GB/s per GPU over NVLink, {roof / t:.2f} of the {NVLINK_GBS:.0f} GB/s link roofline; "
                   f"local HBM traffic {local / 1e6:.0f} MB)")
        del opt, rt, p
        torch.cuda.empty_cache()

    # ---- 3. tensor parallel: row-parallel GEMM with the all-reduce in its epilogue (o_proj / down_proj of a 70B layer)
    if world >= 2:
        tp = TPContext(dev, dist.group.WORLD, world, rank, M * 8192)
        for K_full, N in ((8192, 8192), (28672, 8192)):
            Kl = K_full // world
            a = torch.randn(M, Kl, device=dev, dtype=torch.bfloat16) * 0.1
            w = torch.randn(N, Kl, device=dev, dtype=torch.bfloat16) * 0.02
            t = timed(lambda: tp.reduced_gemm(a, w))
            fl = 2.0 * M * N * Kl
            # Per GPU and direction: the reducer CTAs of a rank own 1/world of the row blocks. With in-switch
            # reduction (multimem.ld_reduce / multimem.st) a rank sends (world-1)/world of its partial tile to the
            # other owners and its reduced 1/world once into the switch, i.e. one output tile in total; with plain
            # peer loads and stores it pulls world-1 partial blocks and writes its sum to world-1 peers.
            mc = any(getattr(b, "multicast_ptr", 0) for b in getattr(tp, "bufs", []) or []) or bool(getattr(getattr(tp, "buf", None), "multicast_ptr", 0))
            link = M * N * 2 * (1.0 if mc else 2.0 * (world - 1) / world)
            roof = max(fl / (peak * 1e12), link / (NVLINK_GBS * 1e9)) * 1e3
            out.append(f"tp GEMM + all-reduce epilogue [M={M}, N={N}, K/tp={Kl}]: {t:.3f} ms ({fl / t / 1e9:.0f} TFLOP/s, "
                       f"{link / t / 1e6:.0f} GB/s per GPU and direction, {'in-switch reduction' if mc else 'peer loads'}); roofline {roof:.3f} ms -> {roof / t:.2f} of {how} roofline")
    _lib.check_status()
    if rank == 0:
        print("\n".join(out))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
