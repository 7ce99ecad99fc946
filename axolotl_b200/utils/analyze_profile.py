"""Offline analysis of the traces the profiler callback writes (``profiler_trace.json``):

    python -m axolotl_b200.utils.analyze_profile TRACE [--compare OTHER] [--top N]

Kernel time is bucketed into categories by kernel name (GEMM, grouped GEMM, attention forward /
backward, elementwise, loss, optimizer, communication, dequantisation, library/other), the number
of optimizer steps is estimated from the optimizer kernel count, and two traces can be diffed
category by category. Reference counterpart: scripts/analyze_profile.py (KERNEL_CATEGORIES,
compare_traces).
"""
from __future__ import annotations

import argparse
import collections
import json
import re

CATEGORIES = [
    ("grouped gemm (MoE)", r"grouped_gemm_kernel"),
    ("gemm (tcgen05)", r"gemm_bf16_(tcgen05|pair)_kernel|gather_only_kernel"),
    ("attention fwd", r"flash_fwd_kernel"),
    ("attention bwd", r"flash_bwd_kernel|attn_delta_kernel|dq_convert_kernel"),
    ("loss", r"ce_fwd_bwd_kernel"),
    ("norm / rope / glu / embedding", r"rmsnorm_|rope_qk|glu_(fwd|bwd)|embedding_"),
    ("optimizer", r"adamw_kernel|rs_adamw_ag_kernel|sumsq_kernel"),
    ("communication", r"peer_barrier|allgather|ep_gather_rows|ep_scatter_add|nccl|peer_put|peer_allreduce"),
    ("dequantisation", r"nvfp4_dequant|nf4_dequant|fp8_block_dequant"),
    ("moe dispatch / combine", r"moe_(dispatch|combine)"),
    ("memcpy / memset", r"^Memcpy|^Memset"),
]


def load_kernels(path):
    with open(path) as fh:
        data = json.load(fh)
    events = data["traceEvents"] if isinstance(data, dict) else data
    out = []
    for e in events:
        if e.get("ph") == "X" and e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset", "Kernel"):
            out.append((e.get("name", ""), float(e.get("dur", 0.0))))
    return out


def categorize(kernels):
    agg = collections.OrderedDict((c, [0, 0.0]) for c, _ in CATEGORIES)
    agg["library / other"] = [0, 0.0]
    for name, dur in kernels:
        for cat, pat in CATEGORIES:
            if re.search(pat, name):
                agg[cat][0] += 1
                agg[cat][1] += dur
                break
        else:
            agg["library / other"][0] += 1
            agg["library / other"][1] += dur
    return agg


def estimate_steps(kernels):
    n = sum(1 for name, _ in kernels if re.search(r"rs_adamw_ag_kernel|adamw_kernel", name))
    return max(n, 1)


def summarize(path, top=10):
    ks = load_kernels(path)
    agg = categorize(ks)
    total = sum(v[1] for v in agg.values()) or 1.0
    steps = estimate_steps(ks)
    lines = [f"{path}: {len(ks)} device events, {total / 1e3:.1f} ms device time, ~{steps} optimizer step(s)"]
    for cat, (n, t) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        if n:
            lines.append(f"  {100 * t / total:5.1f}%  {t / steps / 1e3:9.3f} ms/step  n/step={n / steps:7.1f}  {cat}")
    by_name = collections.defaultdict(float)
    for name, dur in ks:
        by_name[name[:90]] += dur
    lines.append("  top kernels:")
    for name, t in sorted(by_name.items(), key=lambda kv: -kv[1])[:top]:
        lines.append(f"    {100 * t / total:5.1f}%  {name}")
    return agg, steps, lines


def compare(path_a, path_b):
    a, sa, _ = summarize(path_a)
    b, sb, _ = summarize(path_b)
    lines = [f"per-step device time by category: {path_a} -> {path_b}"]
    for cat in a:
        ta, tb = a[cat][1] / sa / 1e3, b[cat][1] / sb / 1e3
        if ta or tb:
            lines.append(f"  {cat:32s} {ta:9.3f} ms -> {tb:9.3f} ms  ({(tb - ta):+.3f})")
    return lines


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("trace")
    ap.add_argument("--compare")
    ap.add_argument("--top", type=int, default=10)
    args = ap.parse_args(argv)
    print("\n".join(summarize(args.trace, args.top)[2]))
    if args.compare:
        print("\n".join(compare(args.trace, args.compare)))


if __name__ == "__main__":
    main()
