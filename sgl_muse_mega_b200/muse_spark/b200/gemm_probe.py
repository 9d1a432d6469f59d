"""Times one skinny GEMM of the item engine in isolation: ``out[16, N] = x[16, K] W[N, K]^T`` through ``mk_lm_head_bind``
(f32 outputs), weights as item images or row-major, L2 flushed between launches (or left warm).

    python -m sgl_muse_mega_b200.muse_spark.b200.gemm_probe --n 25256 --k 8192 [--plain] [--reps 5]

Prints microseconds per launch and the weight-streaming rate. The default shape is the lm_head shard of the TP8 slice.
"""

from __future__ import annotations

import argparse

import torch

from ...common import host
from . import headtail as HT
from . import weights as W


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=25256)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--rows", type=int, default=16)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--plain", action="store_true", help="row-major weights (one bulk copy per weight row)")
    ap.add_argument("--warm", action="store_true", help="no L2 flush between launches: weights that fit L2 are read from it")
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    lib = host.library()
    mod = lib.load()
    w = (torch.randn(args.n, args.k, device=dev) * 0.01).to(torch.bfloat16)
    if not args.plain:
        w = W.pack_items(w)
    x = torch.randn(args.rows, args.k, device=dev).to(torch.bfloat16)
    out = torch.zeros(args.rows, args.n, dtype=torch.float32, device=dev)
    lm = HT.LmHead(lib, mod, w=w, x=x, gathered=[out], rank=0, v_total=args.n, w_packed=not args.plain, n_out=args.n, hidden=args.k)
    s = torch.cuda.current_stream().cuda_stream
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(args.reps):
        if not args.warm:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        lm.launch(s, False)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3
        print(f"{us:.1f} us  {args.n * args.k * 2 / us / 1e6:.2f} TB/s", flush=True)
    assert lm.launch.status(s).code == 0


if __name__ == "__main__":
    main()
