"""Times one DFlash2 draft step of one rank in isolation at the public size (synthetic weights drawn on the device).

    python -m sgl_muse_mega_b200.muse_spark.b200.dflash.probe [--ranks 8] [--rows 16] [--reps 5] [--per-kernel] [--plain]

Prints microseconds per step under programmatic dependent launch and, with ``--per-kernel``, every kernel's time between
CUDA events (serialised: each figure carries the launch and event overhead of a lone kernel, about 8 us).
"""

from __future__ import annotations

import argparse

import torch

from . import draft as DR
from . import synthetic as dsyn
from .weights import DraftConfig, TargetShared

ENTRY = ["feats", "fc", "ctx_norm", "ctx_kv_gemm", "ctx_kv_rows", "embed_norm"]
LAYER = ["conv_proj+conv (attn)", "qkv+rows", "attn_split", "attn_merge", "o_proj", "post_norm", "conv_proj+conv (mlp)", "gate_up+swiglu",
         "down", "next_norm"]  # fmt: skip
HEAD = ["w_p", "top16", "lattice+walk"]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=8, help="tensor-parallel world the slice belongs to (rank 0's slice is timed)")
    ap.add_argument("--rows", type=int, default=16)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--per-kernel", action="store_true")
    ap.add_argument("--plain", action="store_true", help="row-major weights instead of item images")
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    cfg = DraftConfig()
    dw = dsyn.device_shard(cfg, 0, args.ranks, dev, 0)
    n = cfg.vocab // args.ranks
    t = TargetShared(torch.randn(n, cfg.hidden, device=dev).to(torch.bfloat16), (torch.randn(n, cfg.hidden, device=dev) * 0.01).to(torch.bfloat16))
    dr = DR.DraftRank(cfg, dw, t, 0, args.ranks, dev, rows=args.rows, pool_rows=4096, rope_rows=9000, packed=not args.plain)
    dr.bind()
    dr.set_state(8192, 5, 6, torch.randn(cfg.features, args.rows, cfg.hidden))
    for p in dr.k_pool + dr.v_pool:
        p.normal_()
    s = torch.cuda.current_stream().cuda_stream
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dr.launch_all(s, True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.reps):
        dr.launch_all(s, True)
    e1.record()
    torch.cuda.synchronize()
    print(f"{e0.elapsed_time(e1) / args.reps * 1e3:.1f} us per draft step ({dr.kernels()} kernels)", flush=True)
    if args.per_kernel:
        tot: dict = {}
        for li, l in enumerate(dr.launches):
            names = ENTRY if li == 0 else LAYER if li <= cfg.layers else ["lm_head"] if li == cfg.layers + 1 else HEAD
            for k in range(l.info().kernels):
                e0.record()
                l.step(s, k, 1)
                e1.record()
                torch.cuda.synchronize()
                tot.setdefault(names[k], []).append(e0.elapsed_time(e1) * 1e3)
        for k, v in tot.items():
            print(f"  {k:28s} x{len(v)}  {sum(v) / len(v):7.1f} us")
    assert dr.statuses() == [], dr.statuses()


if __name__ == "__main__":
    main()
