"""Times the sampled accept (``MkAcceptBind.samp``) on seeded rows of the full vocabulary, next to the greedy accept.

    python -m sgl_muse_mega_b200.muse_spark.b200.sample_probe [--trace]

Four settings (temperature alone, top-k, top-p, both), CUDA events around the bound launch. ``--trace`` loads a variant
of the library built here with ``-DSAMPLE_TRACE`` (``lib/libmk_sample_trace.so``), whose kernel stamps the global timer at
its stage boundaries into ``sample_out[2:]``, and prints the stage durations: the row phase of cluster (0, 0) (y and max,
top-k search, exp and mass, top-p search), the wait for the last cluster, verification, the bonus search, words and feeds.
"""

from __future__ import annotations

import argparse

import torch

from ...common import build, host
from . import headtail as HT
from .dflash.draft import sampling_words

STAGES = ("y_max", "top_k", "exp_mass", "top_p", "last_cluster", "verify", "bonus", "words_feeds")
SETTINGS = ((0.8, 1 << 30, 1.0, True), (1.0, 50, 1.0, True), (1.0, 1 << 30, 0.9, True), (1.0, 50, 0.9, False))


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--vocab", type=int, default=202048)
    ap.add_argument("--rows", type=int, default=16)
    ap.add_argument("--reps", type=int, default=6)
    ap.add_argument("--trace", action="store_true")
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    lib = host.Library(build.build_variant("sample_trace", ["SAMPLE_TRACE"])) if args.trace else host.library()
    module = lib.load()
    g = torch.Generator().manual_seed(3)
    rows, vocab = args.rows, args.vocab
    logits = torch.randn(rows, vocab, generator=g) * 12.0
    cand = torch.stack([torch.randperm(vocab, generator=g)[:16] for _ in range(rows - 1)])
    q = torch.softmax(torch.randn(rows - 1, 16, generator=g) / 0.7, -1)
    drafts = cand.gather(1, torch.randint(0, 16, (rows - 1, 1), generator=g))[:, 0]
    tokens = torch.cat([torch.randint(0, vocab, (1,), generator=g), drafts])
    logits[torch.arange(rows - 1), drafts] += 45.0
    logits, tokens, cand, q = logits.to(dev), tokens.to(dev), cand.to(dev), q.to(dev)
    s = torch.cuda.current_stream().cuda_stream

    def time(acc):
        out = []
        for _ in range(args.reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            acc.launch(s)
            b.record()
            torch.cuda.synchronize()
            out.append(round(a.elapsed_time(b) * 1e3, 1))
        assert acc.launch.status(s).code == 0
        return out

    for temp, top_k, top_p, block in SETTINGS:
        samp = sampling_words(0xFEDCBA9876543210, 5, temp, top_k, top_p).to(dev)
        acc = HT.Accept(lib, module, logits=logits, tokens=tokens, b_live=rows, scale=32**-0.5, cap=20.0, ring=40, samp=samp,
                        cand=cand, walk_q=q, block_verify=block)  # fmt: skip
        print(f"T {temp} top_k {top_k if top_k < vocab else 'all'} top_p {top_p} {'block' if block else 'token-wise'}: us {time(acc)}")
        if args.trace:
            st = acc.sample_out.cpu()[2:11]
            print("   ", {n: round(float(st[i + 1] - st[i]) / 1e3, 1) for i, n in enumerate(STAGES)})
    greedy = HT.Accept(lib, module, logits=logits, tokens=tokens, b_live=rows, scale=32**-0.5, cap=20.0, ring=40)
    print(f"greedy accept: us {time(greedy)}")


if __name__ == "__main__":
    main()
