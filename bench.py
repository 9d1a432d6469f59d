"""Benchmark of the decode hot path: one full-shape Muse-Spark-Open decoder layer, one rank's TP8 slice per GPU, the
16-row verify window (DFlash2 block 16) over an 8192-token bf16 paged KV cache.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one layer launch through the C ABI (mk_launch of a bound layer). Consecutive steps walk a ring of distinct
layers (3 sliding-window : 1 global, as the model interleaves them) so that no weight byte is read from L2: the ring is
several times larger than the 126 MB L2. Prints ONE JSON line (rank 0).

The CPU leg (``cpu_baseline`` and ``--impl reference``) times the CPU oracle port of the reference's torch layer
(oracle/muse_layer.py, which restates test/reference/muse_spark.py) on the host cores. It is the only place this file
touches ``oracle/``.
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "decoder-layer latency, batch-1 verify window M=16 (per-layer us vs HBM roofline)"
WORKLOAD = "configs[1]: one full-shape Muse-Spark-Open decoder layer, TP8/EP8 slice on 1 B200, M=16, ctx 8192, NVFP4 experts"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--config", type=int, default=1, choices=(1, 2, 3, 4),
                    help="BASELINE.json configuration: 1 (default) one full-shape layer, M=16, ctx 8192, plus the whole-step leg; "
                         "2 the isolated NVFP4 expert block, M in {1,4,8,16} x EP in {1,2,4,8}; 3 the whole model at a 200-token "
                         "context generating 256 tokens; 4 the same at a 131072-token context generating 64 tokens")
    ap.add_argument("--ring", type=int, default=8, help="distinct layers in the ring")
    ap.add_argument("--ctx", type=int, default=None, help="context length (default: the configuration's)")
    ap.add_argument("--rows", type=int, default=16)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--cpu-sample-experts", type=int, default=24)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--timeline", action="store_true",
                    help="one layer's timeline from the trace build (per kernel: first CTA in, programmatic wait returned, last CTA "
                         "out) instead of the bench line")
    ap.add_argument("--form", type=int, default=0, choices=(0, 1, 2, 3, 4),
                    help="dense stages: 0 tcgen05 stream-K GEMM kernels over tile images (default), 1 two persistent segment "
                         "kernels (mma.sync item engine), 2 cluster split-K GEMMs, 3 item-engine GEMM kernels, 4 two fused "
                         "tcgen05 kernels (GEMM stages and the row work between them)")
    ap.add_argument("--decode-layers", type=int, default=62, help="layers of the whole-step leg (0: skip it)")
    ap.add_argument("--decode-steps", type=int, default=24)
    ap.add_argument("--no-draft", action="store_true", help="whole-step leg without the DFlash2 draft (ids from the host)")
    ap.add_argument("--temperature", type=float, default=0.0,
                    help="> 0: the whole-step leg runs the sampled step (sampled draft walk, sampled accept with --top-k / --top-p; "
                         "the accept length stays forced)")
    ap.add_argument("--top-k", type=int, default=1 << 30)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--tp", type=int, default=8, choices=(4, 8),
                    help="tensor-parallel width of the model whose slice each GPU holds (8: the reference's two-node world; "
                         "4 with --gpus 4: the whole model as the single-node TP4 world, configs[3] / [4] only)")
    ap.add_argument("--exchange", default="auto", choices=("auto", "packets", "flags"),
                    help="how a layer's bf16 rows reach their consumers, between GPUs and inside one: rows that carry their own "
                         "validity (packets: the default, except with --form 4), or counter words in the flag block between "
                         "GPUs and kernel completion inside one (flags)")
    ap.add_argument("--tree", action="store_true",
                    help="whole-step leg with the DFlash2 token tree (tree walk, ancestor-masked attention, tree accept, "
                         "compaction); --accept then names the forced leaf ROW, the accept length is its depth")
    ap.add_argument("--accept", type=int, default=5, help="forced accept length of the whole-step leg (5 drafts + the bonus = 6 tokens a step)")
    args = ap.parse_args()
    if args.ctx is None:
        args.ctx = {1: 8192, 2: 16, 3: 200, 4: 131072}[args.config]
    if args.config in (3, 4):  # generated tokens / committed tokens per step, rounded up
        commit = args.accept + 1
        args.decode_steps = -(-(256 if args.config == 3 else 64) // commit)
    return args


# DRAM traffic of the g1 expert kernel from its ncu capture (profiles/experts_umma_kernel_config1_full.md): 238.46 MB read +
# 3.87 MB written for 238.3 MB of algorithmic bytes; it grows with the routed experts like the algorithmic bytes, so the
# bench scales it by them.
G1_TRAFFIC_RATIO = (238.46 + 3.87) / 238.3
G1_TRAFFIC_NOTE = "dram read + write per launch: ncu capture at ring 2 scaled by the algorithmic bytes of this run"


def peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---- algorithmic bytes (per layer, per GPU) ---------------------------------------------------------------------------


def layer_bytes(cfg, d: int, ctx: int, rows: int, global_attn: bool) -> dict:
    """Weight + KV bytes one layer launch must read: qkv, o_proj, the node block of pooler and unpooler, the router
    (f32), d distinct experts' W1 + W2 codes and scales, and the visible KV rows (K and V)."""
    tp, g, H, P = cfg.tp, cfg.node_ranks, cfg.hidden, cfg.moe_hidden
    qkv = cfg.qkv_row * H * 2
    o = H * cfg.oproj_k * 2
    pool = P * H * 2 // g
    unpool = H * P * 2 // g
    router = cfg.experts * H * 4
    per_expert_g1 = 2 * cfg.inter_rank * (P // 2 + P // 16)
    per_expert_g2 = cfg.moe_hidden_rank * (cfg.moe_inter // 2 + cfg.moe_inter // 16)
    keys = ctx + rows if global_attn else min(ctx + rows, cfg.swa_window + rows)
    kv = 2 * keys * cfg.kv_row_bytes
    dense = qkv + o + pool + unpool + router
    return dict(dense=dense, g1=d * per_expert_g1, g2=d * per_expert_g2, kv=kv,
                total=dense + d * (per_expert_g1 + per_expert_g2) + kv)  # fmt: skip


# ---- clocks -----------------------------------------------------------------------------------------------------------


class ClockSampler:
    FIELDS = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )  # fmt: skip
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6 or not parts[0].isdigit():
                continue
            sm.append(int(parts[0]))
            mx.append(int(parts[1]))
            for n, v in zip(names, parts[2:6]):
                if v.lower() == "active":
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [s for s in sm if s >= 0.5 * max(mx)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ---- CPU leg ----------------------------------------------------------------------------------------------------------


def cpu_layer_sample(args, threads: int, repeats: int = 1) -> dict:
    """The CPU oracle on one full-shape layer of the whole TP8 world (all 8 ranks' slices), routing confined to a hot
    subset of experts so that the weights fit in host memory; returns the wall time per rank slice."""
    import torch

    from oracle import muse_layer as O
    from oracle.cases import rank_layers
    from sgl_muse_mega_b200.muse_spark.b200 import synthetic
    from sgl_muse_mega_b200.muse_spark.config import Config

    torch.set_num_threads(threads)
    cfg = Config()
    synthetic.set_device("cpu")
    hot = torch.randperm(cfg.experts, generator=torch.Generator().manual_seed(args.seed))[: args.cpu_sample_experts]
    case = synthetic.layer_case(cfg, rows=args.rows, ctx=args.ctx, band="baseline", seed=args.seed, experts_subset=hot)
    layers = rank_layers(case)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        out = O.run_layer(layers, cfg.node_ranks)
        times.append(time.perf_counter() - t0)
    wall = statistics.median(times)
    return {
        "wall_s": wall,
        "distinct_experts": int(torch.unique(out[0]["ids"]).numel()),
        "us_per_rank_layer": wall / cfg.tp * 1e6,
        "sample": f"1 full-shape layer, all {cfg.tp} rank slices of the TP8 world, M={args.rows}, ctx={args.ctx}, routing "
        f"confined to {args.cpu_sample_experts} experts; value = wall / {cfg.tp} ranks; median of {repeats}",
    }


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    t0 = time.perf_counter()
    r = cpu_layer_sample(args, threads, repeats=max(1, min(args.steps, 3)))
    v = r["us_per_rank_layer"]
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "us", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": v / 1e3, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "nvfp4 weights x nvfp4/bf16 activations, f64 accumulate (CPU oracle)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows": args.rows, "ctx": args.ctx, "distinct_experts_per_layer": [r["distinct_experts"]],
                   "note": "the CPU arm confines routing to a hot subset of experts (its weights must fit host memory and the run a "
                           "few seconds): it does LESS expert work than the GPU arm's ~100 distinct experts, so the GPU / CPU "
                           "ratio is a lower bound; the port is bit-exact against the reference's test/reference/muse_spark.py "
                           "on the committed golden cases"},
        "cpu_baseline": {"value": v, "unit": "us", "cores": threads, "kind": "port", "sample": r["sample"]},
        "e2e": {"value": v, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }  # fmt: skip
    print(json.dumps(line), flush=True)


# ---- the whole verify step: every layer of the model plus head and tail, one CUDA graph ------------------------------


def decode_leg(args, cfg, lib, module, device, rank: int, world: int, stream) -> dict:
    """Builds this rank's slice of a ``--decode-layers`` model (layer variants as the model interleaves them), binds it
    against the present ranks (``world`` processes, one per GPU; alone: no peers) and times the step: CUDA graph replays
    with the forced accept length, the layers alone, and end to end with the ids coming from and the step words going
    to pinned host memory."""
    import torch
    import torch.distributed as dist

    from sgl_muse_mega_b200.common import symm
    from sgl_muse_mega_b200.muse_spark.b200 import stack as S
    from sgl_muse_mega_b200.muse_spark.b200 import synthetic

    tp_rank = rank % cfg.tp
    n_layers, K, W = args.decode_layers, args.decode_steps, 3
    commit = args.accept + 1
    total_steps = 3 * (K + W) + 8
    rows = args.rows
    kv_rows = (args.ctx + commit * total_steps + rows + 127) // 128 * 128
    model = cfg
    if n_layers != cfg.layers:  # a shorter model for quick runs: bf16 experts in its first and last layer, as the full one
        model = dataclasses.replace(cfg, layers=n_layers, bf16_moe_layers=(0, n_layers - 1) if n_layers > 2 else ())
    case = synthetic.stack_case(model, n_layers=n_layers, rows=rows, ctx=args.ctx, seed=args.seed, only_ranks=[tp_rank],
                                max_pos=kv_rows + rows, lazy=True)  # fmt: skip
    forced = torch.tensor([args.accept], dtype=torch.int32, device=device)
    arena = symm.Arena(lib, S.exchange_layout(model, rows), device) if world > 1 else None
    sampling = None
    if args.temperature > 0:
        from sgl_muse_mega_b200.muse_spark.b200.dflash.draft import sampling_words

        assert not args.no_draft, "the sampled accept reads the draft head's candidates"
        sampling = sampling_words(args.seed, 0, args.temperature, args.top_k, args.top_p)
    st = S.Stack(case, tp_rank, device, lib, module, arena=arena, kv_rows=kv_rows, keep_plain_experts=False,
                 accept_override=forced, wait_budget=1 << 25, sampling=sampling, fused=args.form == 4, tree=args.tree,
                 packets=args.form != 4 if args.exchange == "auto" else args.exchange == "packets")  # fmt: skip
    peers = S.connect_world(st) if world > 1 else st.bind()
    s = stream.cuda_stream
    # the DFlash2 draft at its public size (this rank's TP slice, synthetic weights drawn on the device): with it the step
    # is the whole fused iteration - draft, verify, accept - and needs no ids from the host
    it = None
    if not args.no_draft:
        from sgl_muse_mega_b200.muse_spark.b200.dflash import synthetic as dsyn
        from sgl_muse_mega_b200.muse_spark.b200.dflash.iteration import Iteration
        from sgl_muse_mega_b200.muse_spark.b200.dflash.weights import DraftConfig

        dcfg = DraftConfig()
        capture = list(dcfg.capture) if n_layers == cfg.layers else [min(n_layers - 1, i * n_layers // 5) for i in range(5)]
        dw = dsyn.device_shard(dcfg, tp_rank, cfg.tp, device, args.seed)
        kw = dict(capture=capture, pool_rows=4096, rope_rows=kv_rows + rows, wait_budget=1 << 25)
        it = Iteration.connect(st, peers, dcfg, dw, **kw) if world > 1 else Iteration(st, dcfg, dw, **kw)
    step = it.step if it is not None else st.step

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    gen = torch.Generator().manual_seed(args.seed)
    h_tokens = torch.randint(0, model.vocab, (rows,), generator=gen).pin_memory()
    h_words = torch.zeros(8, dtype=torch.int64).pin_memory()
    h_forced = torch.tensor([args.accept], dtype=torch.int32).pin_memory()
    with torch.cuda.stream(stream):
        st.tokens.copy_(h_tokens)
        st.feeds.launch(s)
    barrier()
    with torch.cuda.stream(stream):
        if it is not None:
            it.capture_graph(pdl=True, warmup=True)
        else:
            st.capture(pdl=True, warmup=True)
    barrier()
    # ---- graph replays, inputs resident ----
    with torch.cuda.stream(stream):
        for _ in range(W):
            step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pos0 = int(st.accept.words[0].item())
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(K):
            step()
        e1.record(stream)
    barrier()
    step_ms = max_over_ranks(e0.elapsed_time(e1) / K)
    # tokens a step as the position word counts them (a tree's forced leaf row has the depth its lattice gives it)
    committed = (int(st.accept.words[0].item()) - pos0) / K
    # ---- the layers alone (eager launches with programmatic dependent launch), same exchange partners ----
    with torch.cuda.stream(stream):
        for lr in st.layers:
            lr.launch(s, True)
    barrier()
    reps = max(2, min(8, K // 4))
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(reps):
            for lr in st.layers:
                lr.launch(s, True)
        e1.record(stream)
    barrier()
    layer_us = max_over_ranks(e0.elapsed_time(e1) / (reps * n_layers) * 1e3)
    # ---- per attention type: every layer between its own events (one pass), and a global layer's attention stages alone ----
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(n_layers + 1)]
    with torch.cuda.stream(stream):
        evs[0].record(stream)
        for j, lr in enumerate(st.layers):
            lr.launch(s, True)
            evs[j + 1].record(stream)
    barrier()
    per_layer = [evs[j].elapsed_time(evs[j + 1]) * 1e3 for j in range(n_layers)]
    kinds = {"swa_nvfp4": [t for t, lr in zip(per_layer, st.layers) if not lr.case.global_attn and not lr.case.bf16],
             "global_nvfp4": [t for t, lr in zip(per_layer, st.layers) if lr.case.global_attn and not lr.case.bf16],
             "bf16_experts": [t for t, lr in zip(per_layer, st.layers) if lr.case.bf16]}
    layer_kinds = {k: round(max_over_ranks(sum(v) / len(v)), 1) for k, v in kinds.items() if v}
    attn = None
    glob = [lr for lr in st.layers if lr.case.global_attn and not lr.case.bf16][:8]
    if glob and world == 1:  # stage stepping is for one process: the exchanges of a world need every rank in step
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in glob]
        with torch.cuda.stream(stream):
            for lr, (a, b) in zip(glob, pairs):
                a.record(stream)
                lr.launch_record.step(s, 0, 2)  # split + merge
                b.record(stream)
        barrier()
        us = sum(a.elapsed_time(b) for a, b in pairs) / len(pairs) * 1e3
        keys = int(st.feeds.kv_len.item())
        kv_bytes = 2 * keys * cfg.kv_row_bytes
        attn = {"us": round(us, 1), "keys": keys, "kv_bytes": kv_bytes, "gb_s": round(kv_bytes / (us * 1e-6) / 1e9, 1),
                "frac_of_hbm": round(kv_bytes / (us * 1e-6) / 1e9 / peaks()[0], 3),
                "note": "attention split + merge of a global layer between events (includes two event records, ~5 us)"}
    # ---- the draft alone (its launch list under programmatic dependent launch) ----
    draft = None
    if it is not None:
        with torch.cuda.stream(stream):
            it.draft.launch_all(s, True)
        barrier()
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(reps):
                it.draft.launch_all(s, True)
            e1.record(stream)
        barrier()
        draft_us = max_over_ranks(e0.elapsed_time(e1) / reps * 1e3)
        dbytes = draft_bytes(it.draft.cfg, cfg.tp, rows)
        draft = {"us_per_step": draft_us, "kernels": it.draft.kernels(), "bytes": dbytes,
                 "roofline_frac": dbytes / (draft_us * 1e-6) / 1e9 / peaks()[0], "config": f"DFlash2 public config, TP{cfg.tp} slice"}
    # ---- end to end: ids from pinned host memory, step words back ----
    def e2e_step():
        with torch.cuda.stream(stream):
            if it is None:
                st.tokens.copy_(h_tokens, non_blocking=True)
            else:  # the ids come from the draft; the host's per-step input is the accept control word
                forced.copy_(h_forced, non_blocking=True)
            step()
            h_words.copy_(st.accept.words, non_blocking=True)
        stream.synchronize()

    for _ in range(W):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) / K * 1e3)
    bad = st.statuses()
    assert bad == [], f"device status after the whole-step leg: {bad}"
    if args.tree:
        assert 0 <= int(h_words[2]) <= args.accept and int(h_words[3]) == int(h_words[2]) + 1, h_words.tolist()
        commit = committed
    else:
        assert int(h_words[2]) == args.accept and int(h_words[3]) == commit and committed == commit, h_words.tolist()
    d_list = [int(torch.unique(lr.o["ids"]).numel()) for lr in st.layers]
    byts = [layer_bytes(cfg, d, int(h_words[0]), rows, lr.case.global_attn) for d, lr in zip(d_list, st.layers)]
    for b, lr in zip(byts, st.layers):
        if lr.case.bf16:  # bf16 experts: 2 bytes an element instead of 0.5625
            scale = 2.0 / 0.5625
            b["total"] += int((b["g1"] + b["g2"]) * (scale - 1))
    out = {
        "layers": n_layers, "steps": K, "accept_len": args.accept, "tokens_per_step": commit, "ms_per_step": step_ms,
        "tok_s": commit / (step_ms * 1e-3), "e2e_ms_per_step": e2e_ms, "e2e_tok_s": commit / (e2e_ms * 1e-3),
        "h2d_bytes_per_step": h_tokens.numel() * 8 if it is None else 4, "d2h_bytes_per_step": 64,
        "layer_only_us": layer_us, "layer_us_by_kind": layer_kinds, "global_attention": attn, "ctx": args.ctx,
        "kernels_per_step": it.kernels if it is not None else st.kernels,
        "bytes_per_step": int(sum(b["total"] for b in byts)), "mean_distinct_experts": sum(d_list) / len(d_list),
        "present_ranks": world if world > 1 else 1, "model_ranks": cfg.tp,
        "draft": draft if draft is not None else "not in the step (--no-draft): ids come from the host",
        "sampling": "greedy" if sampling is None else {"temperature": args.temperature, "top_k": args.top_k, "top_p": args.top_p},
        "window": "token tree (forced leaf row %d)" % args.accept if args.tree else "chain",
        "exchange": "packets (bf16 rows and router logits with in-band validity, their consumers do not wait for the producing "
                    "grid's end; h planes and vocabulary logits on counter words)" if st.packets else
                    "kernel completion (one rank)" if world == 1 else "counter words",
    }  # fmt: skip
    if it is not None:
        bad = it.statuses()
        assert bad == [], f"device status of the draft: {bad}"
    if world > 1:
        # every present rank ends the run with the same step state, bit for bit: the gathered logits, the arg-max, the step
        # words, the window's ids and the residuals the draft captured
        state = {"logits": st.gathered, "top1": st.accept.top1, "words": st.accept.words, "tokens": st.tokens}
        if it is not None:
            state["capture_residuals"] = torch.stack([st.layers[c].o["stream_out"] for c in it.capture])
        out["ranks_equal"] = ranks_equal(state, world)
    del peers
    return out, st


def ranks_equal(state: dict, world: int) -> dict:
    """All-gathers the named tensors and compares every rank's copy with rank 0's bit for bit: name -> equal."""
    import torch
    import torch.distributed as dist

    res = {}
    for name, t in state.items():
        t = t.contiguous()
        got = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(got, t)
        same = all(torch.equal(g.view(torch.uint8), got[0].view(torch.uint8)) for g in got[1:])
        # equal, or how many elements of the worst rank differ from rank 0's
        res[name] = True if same else {"differing_elements": max(int((g != got[0]).sum()) for g in got[1:]), "of": t.numel()}
    return res


def parity_world(args, lib, module, device, rank: int, world: int) -> dict:
    """The world of ``world`` processes against the same world emulated on one GPU (every rank's launches interleaved in
    one process, rank 0's GPU), on a 4-layer model of tensor-parallel width ``world``: three verify steps as CUDA graph
    replays, after each the step words, the arg-max and the gathered logits of every rank all-gathered and compared bit
    for bit with the emulated ranks' (the fused form's GEMMs sum in another fixed order: its logits are held to a relative
    distance instead, its ranks to each other bit for bit)."""
    import torch
    import torch.distributed as dist

    from sgl_muse_mega_b200.common import symm
    from sgl_muse_mega_b200.muse_spark.b200 import stack as S
    from sgl_muse_mega_b200.muse_spark.b200 import synthetic
    from sgl_muse_mega_b200.muse_spark.config import Config

    cfg = Config(hidden=1024, q_heads=64, kv_heads=8, experts=16, topk=8, moe_hidden=1024, moe_inter=1024, swa_window=7,
                 vocab=4096, layers=4, bf16_moe_layers=(0,), tp=world, node_ranks=min(4, world))  # fmt: skip
    rows, ctx, steps, accept = 16, 24, 3, 6
    fused = args.form == 4
    gen = torch.Generator().manual_seed(31)
    ids = [torch.randint(0, cfg.vocab, (rows,), generator=gen) for _ in range(steps)]
    case = synthetic.stack_case(cfg, n_layers=4, rows=rows, ctx=ctx, seed=21, only_ranks=[rank])
    forced = torch.tensor([accept], dtype=torch.int32, device=device)
    arena = symm.Arena(lib, S.exchange_layout(cfg, rows), device)
    st = S.Stack(case, rank, device, lib, module, arena=arena, accept_override=forced, wait_budget=1 << 25, fused=fused,
                 packets=None if args.exchange == "auto" else args.exchange == "packets")  # fmt: skip
    peers = S.connect_world(st)
    st.feeds.launch(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    st.capture(warmup=False)
    names = ("words", "top1", "logits")
    got = []  # per step: name -> every rank's copy
    for t in ids:
        st.tokens.copy_(t)
        st.step()
        torch.cuda.synchronize()
        mine = {"words": st.accept.words, "top1": st.accept.top1, "logits": st.gathered}
        step = {}
        for k in names:
            every = [torch.empty_like(mine[k]) for _ in range(world)]
            dist.all_gather(every, mine[k].contiguous())
            step[k] = [e.cpu() for e in every]
        got.append(step)
    status = st.statuses()
    dist.barrier()
    del peers
    res = None
    if rank == 0:
        whole = synthetic.stack_case(cfg, n_layers=4, rows=rows, ctx=ctx, seed=21)
        w = S.StackWorld(whole, device, lib, accept_override=forced)
        mismatch, worst = [], 0.0
        for i, t in enumerate(ids):
            for e in w.ranks:
                e.tokens.copy_(t)
            w.run_interleaved(feeds=i == 0)
            torch.cuda.synchronize()
            for r, e in enumerate(w.ranks):
                ref = {"words": e.accept.words.cpu(), "top1": e.accept.top1.cpu(), "logits": e.gathered.cpu()}
                for k in names:
                    a = got[i][k][r]
                    if not torch.equal(a, got[i][k][0]):
                        mismatch.append(f"step {i}: rank {r}'s {k} differ from rank 0's")
                    if fused:
                        if k == "logits":
                            worst = max(worst, float((a - ref[k]).norm() / ref[k].norm()))
                    elif not torch.equal(a, ref[k]):
                        mismatch.append(f"step {i}: rank {r}'s {k} differ from the emulated world's")
        emu_status = [x for e in w.ranks for x in e.statuses()]
        res = {"model": "4 layers (one with bf16 experts), hidden 1024, 16 experts, vocab 4096, tensor-parallel over the ranks",
               "steps": steps, "compared": list(names), "bit_equal": not mismatch and not fused, "mismatch": mismatch[:8],
               "exchange": "packets" if st.packets else "counter words",
               "status": [str(x) for x in status + emu_status]}  # fmt: skip
        if fused:
            res["ranks_bit_equal"] = not mismatch
            res["logits_rel_to_per_stage_world"] = worst
            res["note"] = "the fused form sums its GEMMs in another fixed order than the emulated world's per-stage kernels"
    return res


def decode_line(args, cfg, dec: dict, world: int, clocks) -> dict:
    """The JSON line of configs[3] / configs[4]: decode tokens per second of the whole fused iteration at the forced accept
    length, the model's TP8 slice per GPU (ranks 0 .. world - 1 of the TP8 world present)."""
    peak, peak_kind = peaks()
    n_layers = dec["layers"]
    gen = 256 if args.config == 3 else 64
    what = (f"configs[{args.config}]: full-shape 62-layer model + DFlash2 draft, TP{cfg.tp} slice per GPU on {world} B200(s)"
            f"{' (the whole world)' if world == cfg.tp else ''}, "
            f"{args.ctx}-token context (KV filled directly: no prefill path here), {gen} generated tokens, block 16, "
            f"forced accept {args.accept} (commit {args.accept + 1} a step)")
    if args.tree:
        what = what.replace(f"forced accept {args.accept} (commit {args.accept + 1} a step)",
                            f"token-tree window, forced leaf row {args.accept} (its depth + 1 = {dec['tokens_per_step']:.2f} tokens a step "
                            "on synthetic lattices: the number shows the tree step's cost, not the tree's acceptance gain)")
    layer_gbs = dec["bytes_per_step"] / (dec["layer_only_us"] * n_layers * 1e-6) / 1e9
    return {
        "metric": "batch-1 decode tok/s at fixed accept len", "value": dec["tok_s"], "unit": "tok/s", "n_gpus": world,
        "steps": dec["steps"], "warmup": 3, "ms_per_step": dec["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 experts (e2m1 x e4m3 block scales), bf16 dense, f32 accumulate", "data": "synthetic",
        "config": {"workload": what, "rows": args.rows, "ctx": args.ctx, "l2": "inputs larger than L2 (every layer of the model is distinct)",
                   "kernels_per_step": dec["kernels_per_step"]},
        "roofline": {"bound": "hbm", "kernel": "whole step's layers", "achieved": layer_gbs, "peak": peak, "unit": "GB/s",
                     "frac": layer_gbs / peak, "traffic": None, "peak_kind": peak_kind},
        "e2e": {"value": dec["e2e_tok_s"], "unit": "tok/s", "h2d_bytes_per_step": dec["h2d_bytes_per_step"],
                "d2h_bytes_per_step": dec["d2h_bytes_per_step"]},
        "gpu_launches": dec["kernels_per_step"] * (2 * dec["steps"] + 7), "decode": dec, "clocks": clocks, "cpu_baseline": None,
    }  # fmt: skip


def draft_bytes(dcfg, ranks: int, rows: int) -> int:
    """Algorithmic HBM bytes of one draft step on one rank: every weight once (bf16), the attention window's K / V."""
    h, d = dcfg.hidden, dcfg.head_dim
    qh, kvh, inter = dcfg.q_heads // ranks, dcfg.kv_heads // ranks, dcfg.inter // ranks
    per_layer = 2 * dcfg.coeffs * h + (qh + 2 * kvh) * d * h + h * qh * d + 2 * inter * h + h * inter
    kv = dcfg.layers * 2 * (dcfg.window_left + rows) * kvh * d
    head = (dcfg.vocab // ranks) * h + dcfg.selector_rank * h + (rows - 1) * dcfg.vocab * 2  # lm_head shard, W_P, the f32 logits written + read (x2 bytes/2)
    entry = (h // ranks) * dcfg.features * h + dcfg.layers * 2 * kvh * d * h
    return 2 * (dcfg.layers * per_layer + kv + head + entry)


# ---- GPU leg ----------------------------------------------------------------------------------------------------------


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from sgl_muse_mega_b200.common import host
    from sgl_muse_mega_b200.muse_spark.b200 import layer as L
    from sgl_muse_mega_b200.muse_spark.b200 import synthetic
    from sgl_muse_mega_b200.muse_spark.config import Config

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device: there is no CPU fallback"
    device = torch.device(f"cuda:{local}")
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    cfg = Config()
    if args.tp != cfg.tp:
        assert args.config in (3, 4), "--tp 4 serves the decode legs (--config 3 / 4)"
        cfg = cfg.with_tp(args.tp)
    lib = host.library()
    module = lib.load()
    synthetic.set_device(device)
    if world > 1:
        run_world(args, cfg, lib, module, device, rank, world, local)
        dist.destroy_process_group()
        return
    if args.config in (3, 4):
        stream = torch.cuda.Stream(device)
        sampler = ClockSampler(local)
        dec, _st = decode_leg(args, cfg, lib, module, device, rank, world, stream)
        print(json.dumps(decode_line(args, cfg, dec, world, sampler.stop())), flush=True)
        return
    # a ring of distinct layers: global iff i % 4 == 3 here (3 swa : 1 global). Each GPU holds the slice of TP rank
    # `rank % 8`; with N GPUs the ranks are independent replicas of the per-GPU work (no exchange partner is waited for).
    tp_rank = rank % cfg.tp
    ring = []
    for i in range(args.ring):
        glob = i % 4 == 3
        case = synthetic.layer_case(cfg, rows=args.rows, ctx=args.ctx, global_attn=glob, next_global=(i + 1) % 4 == 3,
                                    band="baseline", seed=args.seed, layer=2 + i, only_ranks=[tp_rank])  # fmt: skip
        lr = L.LayerRank(lib, module, case, tp_rank, device, tensors=case.ranks[0], keep_plain_experts=False,
                         packed={0: 2, 1: 1, 2: 0, 3: 1, 4: 2}[args.form])
        assert lr.tensor_cores, "the full shape runs its experts on the tcgen05 kernels"
        # the absent ranks' contributions: values of the right kind already in the exchange buffers
        g = torch.Generator(device=device).manual_seed(1000 + i)
        lr.ar.view(torch.bfloat16).copy_(torch.randn(lr.ar.numel() // 2, generator=g, device=device) * 0.3)
        lr.pool_ag.copy_(torch.randn(lr.pool_ag.shape, generator=g, device=device))
        lr.unpool_ag.copy_(torch.randn(lr.unpool_ag.shape, generator=g, device=device))
        lr.z.copy_(torch.randint(0, 256, lr.z.shape, generator=g, device=device, dtype=torch.uint8))
        lr.z_sf.copy_(torch.randint(0x30, 0x40, lr.z_sf.shape, generator=g, device=device, dtype=torch.uint8))
        lr.z_ex.copy_(torch.randint(0, 3, lr.z_ex.shape, generator=g, device=device, dtype=torch.uint8))
        lr.zb.view(torch.bfloat16).copy_(torch.randn(lr.zb.numel() // 2, generator=g, device=device))
        lr.bind(None, fused={0: 0, 1: 1, 2: 2, 3: 0, 4: 1}[args.form], packets=args.form == 0 and args.exchange != "flags")
        case.ranks = []  # the device copies live in lr.w
        ring.append(lr)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream(device)
    s = stream.cuda_stream
    info = ring[0].launch_record.info()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    # ---- kernel-resident timing: inputs already in HBM --------------------------------------------------------------
    for i in range(args.warmup):
        ring[i % args.ring].launch(s, True)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for i in range(args.steps):
        ring[i % args.ring].launch(s, True)
    ev1.record(stream)
    barrier()
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    us_layer = ms * 1e3 / args.steps
    for lr in ring:
        st = lr.launch_record.status(s)
        assert st.code == 0, f"device status {st.code} at stage {st.stage}"
    # distinct experts actually routed, per ring layer (drives the algorithmic bytes)
    d_list = [int(torch.unique(lr.o["ids"]).numel()) for lr in ring]
    byt = [layer_bytes(cfg, d, args.ctx, args.rows, lr.case.global_attn) for d, lr in zip(d_list, ring)]
    steps_per_layer = [len(range(i, args.steps, args.ring)) for i in range(args.ring)]
    total_bytes = sum(b["total"] * n for b, n in zip(byt, steps_per_layer))
    peak, peak_kind = peaks()
    layer_gbs = total_bytes / (ms * 1e-3) / 1e9

    # ---- dominant kernel (g1, the gate/up expert GEMM): CUDA events around that stage alone -------------------------
    G1 = L.STAGE_NAMES.index("g1")
    k_steps = max(8, min(args.steps, 64))
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(k_steps)]
    barrier()
    for i, (a, b) in enumerate(pairs):
        lr = ring[i % args.ring]
        lr.launch_record.step(s, 0, G1)
        a.record(stream)
        lr.launch_record.step(s, G1, 1)
        b.record(stream)
        lr.launch_record.step(s, G1 + 1, len(L.STAGE_NAMES) - G1 - 1)
    barrier()
    g1_ms = [a.elapsed_time(b) for a, b in pairs]
    g1_bytes = sum(byt[i % args.ring]["g1"] for i in range(k_steps))
    g1_gbs = g1_bytes / (sum(g1_ms) * 1e-3) / 1e9

    # ---- per-stage breakdown (diagnostic): every stage launched alone between two events; serialised, so the sum
    # exceeds the layer time measured above (no PDL overlap here)
    n_st = len(L.STAGE_NAMES)
    stage_ms = [0.0] * n_st
    reps = max(4, min(args.steps, 24))
    for i in range(reps):
        lr = ring[i % args.ring]
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(n_st + 1)]
        evs[0].record(stream)
        for st in range(n_st):
            lr.launch_record.step(s, st, 1)
            evs[st + 1].record(stream)
        stream.synchronize()
        for st in range(n_st):
            stage_ms[st] += evs[st].elapsed_time(evs[st + 1])
    stage_us = {name: round(t / reps * 1e3, 2) for name, t in zip(L.STAGE_NAMES, stage_ms) if t > 0}

    # ---- end to end: host buffers in, host buffers out, through the same C-ABI launch -------------------------------
    M, H = args.rows, cfg.hidden
    h_qkv = torch.randn(M, cfg.qkv_row).bfloat16().pin_memory()
    h_stream = torch.randn(M, H).pin_memory()
    h_out_stream = torch.empty(M, H).pin_memory()
    h_out_qkv = torch.empty(M, cfg.qkv_row, dtype=torch.bfloat16).pin_memory()
    h2d = h_qkv.numel() * 2 + h_stream.numel() * 4
    d2h = h_out_stream.numel() * 4 + h_out_qkv.numel() * 2

    def e2e_step(i):
        lr = ring[i % args.ring]
        with torch.cuda.stream(stream):
            lr.w["qkv_in"].copy_(h_qkv, non_blocking=True)
            lr.w["stream_in"].copy_(h_stream, non_blocking=True)
            lr.launch(s, True)
            h_out_stream.copy_(lr.o["stream_out"], non_blocking=True)
            h_out_qkv.copy_(lr.o["qkv_next"], non_blocking=True)
        stream.synchronize()

    for i in range(min(args.warmup, 8)):
        e2e_step(i)
    barrier()
    e_steps = max(8, min(args.steps, 200))
    t0 = time.perf_counter()
    for i in range(e_steps):
        e2e_step(i)
    torch.cuda.synchronize()
    e2e_us = (time.perf_counter() - t0) / e_steps * 1e6
    if world > 1:
        t = torch.tensor([e2e_us], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_us = float(t.item())
    clocks = sampler.stop() if sampler else None

    seg_trace = None
    if args.form == 1:
        # stage timestamps CTA 0 of the two segment kernels left in the status block (ns of the global timer)
        names_a = ["pdl_wait", "o_proj", "barrier", "ar_finish_signal", "post_norm_row", "barrier", "pooler_router", "barrier",
                   "pool_finish_signal", "routing_nq"]  # fmt: skip
        names_b = ["pdl_wait", "combine_row", "barrier", "unpooler", "barrier", "finish_cross_norm", "barrier", "qkv",
                   "barrier", "qkv_rowops"]  # fmt: skip
        t = ring[0].status.view(torch.int32)[64:192].view(torch.int64).cpu().tolist()
        a, b = t[0:11], t[16:27]
        seg_trace = {"segment_a": [[n, round((a[i + 1] - a[i]) / 1e3, 2)] for i, n in enumerate(names_a)],
                     "segment_b": [[n, round((b[i + 1] - b[i]) / 1e3, 2)] for i, n in enumerate(names_b)]}  # fmt: skip
    dec = None
    if args.decode_layers > 0:
        del ring, lr
        torch.cuda.empty_cache()
        dec, _st = decode_leg(args, cfg, lib, module, device, rank, world, stream)
        del _st
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        r = cpu_layer_sample(args, threads, repeats=3)
        cpu = {"value": r["us_per_rank_layer"], "unit": "us", "cores": threads, "kind": "port", "sample": r["sample"]}
    if rank == 0:
        # The line's value is the same quantity at every N: the mean layer of the whole-step leg's 62-layer model (60 NVFP4
        # layers, 3 sliding-window : 1 global, and the two bf16-expert layers), eager launches with programmatic dependent
        # launch. The ring of eight NVFP4 layers above stays in the line as ``ring_layer_us`` (and is the value when the
        # whole-step leg is skipped).
        value, timed = us_layer, f"a ring of {args.ring} distinct NVFP4 layers, eager with programmatic dependent launch"
        value_gbs, value_bytes = layer_gbs, int(total_bytes / args.steps)
        e2e = {"value": e2e_us, "unit": "us", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
        if dec is not None:
            n_dec = dec["layers"]
            value, timed = dec["layer_only_us"], "the layer launches of the whole-step leg, eager with programmatic dependent launch"
            value_bytes = dec["bytes_per_step"] // n_dec
            value_gbs = value_bytes / (value * 1e-6) / 1e9
            e2e = {"value": dec["e2e_ms_per_step"] * 1e3 / n_dec, "unit": "us", "h2d_bytes_per_step": dec["h2d_bytes_per_step"],
                   "d2h_bytes_per_step": dec["d2h_bytes_per_step"],
                   "note": "whole fused iteration through the CUDA graph with the host's control word in and the step words out, divided by its layers",
                   "layer_call": {"value": e2e_us, "unit": "us", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                                  "note": "one layer launch through the C-ABI with its host rows in and out"}}  # fmt: skip
        line = {
            "metric": METRIC, "value": value, "unit": "us", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": value / 1e3, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
            "dtype": "nvfp4 experts (e2m1 x e4m3 block scales), bf16 dense, f32 accumulate", "data": "synthetic",
            "config": {
                "workload": WORKLOAD, "rows": args.rows, "ctx": args.ctx, "ring_layers": args.ring,
                "ring_bytes": int(sum(b["total"] for b in byt)), "l2": "inputs larger than L2 (every layer of the model is distinct)",
                "distinct_experts_per_layer": d_list, "multi_gpu": "independent replicas of the per-GPU slice" if world > 1 else "1 GPU",
                "kernels_per_step": int(info.kernels), "timed": timed,
            },
            "ring_layer_us": us_layer,
            "ring_roofline": {"achieved": layer_gbs, "frac": layer_gbs / peak, "bytes_per_layer": int(total_bytes / args.steps)},
            "layer_roofline": {"bound": "hbm", "achieved": value_gbs, "peak": peak, "unit": "GB/s", "frac": value_gbs / peak,
                               "bytes_per_layer": value_bytes, "peak_kind": peak_kind},
            "roofline": {"bound": "hbm", "kernel": "experts_umma_kernel<g1>", "achieved": g1_gbs, "peak": peak, "unit": "GB/s",
                         "frac": g1_gbs / peak, "traffic": G1_TRAFFIC_RATIO * g1_bytes / len(pairs), "traffic_note": G1_TRAFFIC_NOTE,
                         "peak_kind": peak_kind,
                         "us_per_launch": sum(g1_ms) / k_steps * 1e3},
            "e2e": e2e,
            "gpu_launches": int(info.kernels) * args.steps + (dec["kernels_per_step"] * (2 * args.decode_steps + 7) if dec else 0),
            "stage_us_serialised": stage_us,
            "decode": dec,
            "segment_trace_us": seg_trace,
            "clocks": clocks,
            "cpu_baseline": cpu,
        }  # fmt: skip
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_world(args, cfg, lib, module, device, rank: int, world: int, local: int) -> None:
    """N > 1: one process per GPU, ranks 0 .. N - 1 of the model's TP8 world present (N = 8: the whole world), exchanging
    through each other's memory inside the kernels. Per-GPU work is the same TP8 slice at every N (weak scaling)."""
    import torch
    import torch.distributed as dist

    from sgl_muse_mega_b200.muse_spark.b200 import layer as L

    stream = torch.cuda.Stream(device)
    s = stream.cuda_stream
    sampler = ClockSampler(local) if rank == 0 else None
    assert args.decode_layers > 0, "the multi-GPU run times the layers of the whole-step leg"
    dec, st = decode_leg(args, cfg, lib, module, device, rank, world, stream)
    if args.config in (3, 4):
        clocks = sampler.stop() if sampler else None
        del st
        torch.cuda.empty_cache()
        emu = parity_world(args, lib, module, device, rank, world)
        if rank == 0:
            line = decode_line(args, cfg, dec, world, clocks)
            line["parity_n"] = parity_n(world, dec, emu)
            print(json.dumps(line), flush=True)
        return
    n_layers = dec["layers"]
    peak, peak_kind = peaks()
    # the dominant kernel (g1) between events, every rank stepping the same stages in the same order
    G1 = L.STAGE_NAMES.index("g1")
    fp4 = [lr for lr in st.layers if not lr.case.bf16][:32]
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in fp4]
    with torch.cuda.stream(stream):
        for lr, (a, b) in zip(fp4, pairs):
            lr.launch_record.step(s, 0, G1)
            a.record(stream)
            lr.launch_record.step(s, G1, 1)
            b.record(stream)
            lr.launch_record.step(s, G1 + 1, len(L.STAGE_NAMES) - G1 - 1)
    torch.cuda.synchronize()
    dist.barrier()
    g1_ms = sum(a.elapsed_time(b) for a, b in pairs)
    g1_bytes = sum(layer_bytes(cfg, int(torch.unique(lr.o["ids"]).numel()), args.ctx, args.rows, False)["g1"] for lr in fp4)
    t = torch.tensor([g1_ms], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    g1_gbs = g1_bytes / (float(t.item()) * 1e-3) / 1e9
    assert st.statuses() == []
    clocks = sampler.stop() if sampler else None
    del st, fp4, lr
    torch.cuda.empty_cache()
    emu = parity_world(args, lib, module, device, rank, world)
    if rank == 0:
        us_layer = dec["layer_only_us"]
        layer_gbs = dec["bytes_per_step"] / (us_layer * n_layers * 1e-6) / 1e9
        line = {
            "metric": METRIC, "value": us_layer, "unit": "us", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": us_layer / 1e3, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
            "dtype": "nvfp4 experts (e2m1 x e4m3 block scales), bf16 dense, f32 accumulate", "data": "synthetic",
            "config": {
                "workload": WORKLOAD.replace("on 1 B200", f"per GPU, ranks 0..{world - 1} of the TP8 world on {world} B200s"),
                "rows": args.rows, "ctx": args.ctx, "layers": n_layers,
                "l2": "inputs larger than L2 (every layer of the model is distinct)",
                "multi_gpu": f"{world} of 8 ranks present, in-kernel exchange through peer memory (flag-polled P2P stores)",
                "kernels_per_step": dec["kernels_per_step"],
                "timed": "the layer launches of the whole-step leg, eager with programmatic dependent launch",
            },
            "layer_roofline": {"bound": "hbm", "achieved": layer_gbs, "peak": peak, "unit": "GB/s", "frac": layer_gbs / peak,
                               "bytes_per_layer": dec["bytes_per_step"] // n_layers, "peak_kind": peak_kind},
            "roofline": {"bound": "hbm", "kernel": "experts_umma_kernel<g1>", "achieved": g1_gbs, "peak": peak, "unit": "GB/s",
                         "frac": g1_gbs / peak, "traffic": G1_TRAFFIC_RATIO * g1_bytes / len(pairs), "traffic_note": G1_TRAFFIC_NOTE,
                         "peak_kind": peak_kind,
                         "us_per_launch": float(t.item()) / len(pairs) * 1e3},
            "e2e": {"value": dec["e2e_ms_per_step"] * 1e3 / n_layers, "unit": "us",
                    "h2d_bytes_per_step": dec["h2d_bytes_per_step"], "d2h_bytes_per_step": dec["d2h_bytes_per_step"],
                    "note": "whole verify step through the CUDA graph with host ids in and step words out, divided by its layers"},
            "gpu_launches": dec["kernels_per_step"] * (2 * args.decode_steps + 7),
            "parity_n": parity_n(world, dec, emu),
            "decode": dec,
            "clocks": clocks,
            "cpu_baseline": None,
        }  # fmt: skip
        print(json.dumps(line), flush=True)


def parity_n(world: int, dec: dict, emu: dict) -> dict:
    """The multi-GPU run's parity record: the timed model's end state equal on every rank, and the small model's world
    equal to the same world emulated on one GPU."""
    same = dec.get("ranks_equal") or {}
    ok = bool(same) and all(v is True for v in same.values()) and bool(emu) and (emu["bit_equal"] or emu.get("ranks_bit_equal", False)) and not emu["status"]
    return {"ranks": world, "bit_equal": ok, "timed_model_ranks_equal": same, "emulated_world": emu}


def run_timeline(args) -> None:
    """One full-shape NVFP4 layer of the ring under programmatic dependent launch on the trace build of the library
    (``common/build.py`` ``trace=True``): every kernel's CTAs stamp %globaltimer at entry, when their programmatic wait
    returns and when they leave. Prints per kernel, in launch order: first entry, wait returned (first CTA), end (last
    CTA), body = end - wait returned, and the boundary = wait returned - the predecessor's end. The stamps cost a few
    hundred nanoseconds a kernel: read the proportions, not the sum."""
    import ctypes

    import torch

    from sgl_muse_mega_b200.common import build, host
    from sgl_muse_mega_b200.muse_spark.b200 import layer as L
    from sgl_muse_mega_b200.muse_spark.b200 import synthetic
    from sgl_muse_mega_b200.muse_spark.config import Config

    assert torch.cuda.is_available(), "bench.py needs a CUDA device: there is no CPU fallback"
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    lib = host.Library(build.build(trace=True))
    module = lib.load()
    synthetic.set_device(device)
    cfg = Config()
    ring = []
    for i in range(3):
        case = synthetic.layer_case(cfg, rows=args.rows, ctx=args.ctx, global_attn=False, next_global=False, band="baseline",
                                    seed=args.seed, layer=2 + i, only_ranks=[0])  # fmt: skip
        lr = L.LayerRank(lib, module, case, 0, device, tensors=case.ranks[0], keep_plain_experts=False)
        g = torch.Generator(device=device).manual_seed(1000 + i)
        lr.ar.view(torch.bfloat16).copy_(torch.randn(lr.ar.numel() // 2, generator=g, device=device) * 0.3)
        lr.pool_ag.copy_(torch.randn(lr.pool_ag.shape, generator=g, device=device))
        lr.unpool_ag.copy_(torch.randn(lr.unpool_ag.shape, generator=g, device=device))
        lr.zb.view(torch.bfloat16).copy_(torch.randn(lr.zb.numel() // 2, generator=g, device=device))
        lr.bind(None, fused=0, packets=args.exchange != "flags")
        case.ranks = []
        ring.append(lr)
    stream = torch.cuda.Stream(device)
    s = stream.cuda_stream
    for rep in range(12):
        ring[rep % 3].launch(s, True)
    stream.synchronize()
    st = ring[2].launch_record.status(s)
    assert st.code == 0, f"device status {st.code} at stage {st.stage}"

    def read(fn: str, shape) -> "torch.Tensor":
        n = 1
        for d in shape:
            n *= d
        buf = (ctypes.c_ulonglong * n)()
        assert getattr(lib.dll, fn)(buf) == 0, fn
        return torch.tensor(list(buf), dtype=torch.int64).view(*shape)

    dense = read("mk_dense_trace_read", (8, 160, 16))  # [o_proj, pooler + router, unpooler, qkv][CTA]: 0 entry, 3 wait, 9 out
    umma = read("mk_umma_trace_read", (2, 160, 16))  # [g1, g2][CTA]: 0 entry, 2 tables copied, 9 out
    rows = read("mk_rows_trace_read", (8, 160, 4))  # [post norm, cross norm, routing, -, combine][CTA]: entry, wait, out, tables
    attn = read("mk_attn_trace_read", (8, 160, 4))  # [5 split, 6 combine][CTA]
    kernels = [
        ("attn_split", attn[5, :, 0], attn[5, :, 1], attn[5, :, 2]), ("attn_combine", attn[6, :, 0], attn[6, :, 1], attn[6, :, 2]),
        ("o_proj", dense[0, :, 0], dense[0, :, 3], dense[0, :, 9]), ("post_norm", rows[0, :, 0], rows[0, :, 1], rows[0, :, 2]),
        ("pooler+router", dense[1, :, 0], dense[1, :, 3], dense[1, :, 9]),
        ("routing+quantisation", rows[2, :, 0], rows[2, :, 1], torch.maximum(rows[2, :, 2], rows[2, :, 3])),
        ("g1", umma[0, :, 0], umma[0, :, 2], umma[0, :, 9]), ("g2", umma[1, :, 0], umma[1, :, 2], umma[1, :, 9]),
        ("combine", rows[4, :, 0], rows[4, :, 1], rows[4, :, 2]), ("unpooler", dense[2, :, 0], dense[2, :, 3], dense[2, :, 9]),
        ("cross_norm", rows[1, :, 0], rows[1, :, 1], rows[1, :, 2]), ("qkv", dense[3, :, 0], dense[3, :, 3], dense[3, :, 9]),
    ]  # fmt: skip
    ev = []
    for name, entry, wait, end in kernels:
        entry, wait, end = entry[entry > 0], wait[wait > 0], end[end > 0]
        if entry.numel() and wait.numel() and end.numel():
            ev.append((name, int(entry.min()), int(wait.min()), int(end.max())))
    ev.sort(key=lambda e: e[1])  # each kernel's stamps are its last launch's; the ring's launches follow one another
    t0, prev = ev[0][1], None
    out = []
    for name, entry, wait, end in ev:
        rec = {"kernel": name, "entry_us": round((entry - t0) / 1e3, 2), "wait_returned_us": round((wait - t0) / 1e3, 2),
               "end_us": round((end - t0) / 1e3, 2), "body_us": round((end - wait) / 1e3, 2),
               "boundary_us": None if prev is None else round((wait - prev) / 1e3, 2)}  # fmt: skip
        # g2 copies its route tables before g1 has finished: its "wait" stamp is not a wait on g1
        if name == "g2":
            rec["boundary_us"], rec["body_us"] = None, round((end - prev) / 1e3, 2)
            rec["note"] = "body counted from g1's end (the roles that read g1's output wait inside the kernel)"
        out.append(rec)
        prev = end
    print(json.dumps({"timeline": out, "workload": WORKLOAD, "note": "trace build, one layer under programmatic dependent launch"}))


def run_expert_block(args) -> None:
    """configs[2]: the isolated NVFP4 expert block at the full expert shape (256 experts x 28.31 MB), M in {1, 4, 8, 16}
    rows, experts partitioned over EP in {1, 2, 4, 8} ranks. One GPU: the ranks' launches run one after the other on it (a
    rank's time is what its GPU would take; the block's time is the slowest rank's). Reports the achieved HBM GB/s of the
    routed experts' weight bytes, L2 flushed before every sample."""
    import torch

    from sgl_muse_mega_b200.common import host
    from sgl_muse_mega_b200.muse_spark.b200 import expert_block as X

    assert torch.cuda.is_available(), "bench.py needs a CUDA device: there is no CPU fallback"
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        return run_expert_block_world(args)
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    lib = host.library()
    module = lib.load()
    sampler = ClockSampler(0)
    cfg = X.block_config()
    full = X.draw_case(cfg, 16, device, seed=args.seed)
    peak, peak_kind = peaks()
    sweep, launches = [], 0
    iters = max(3, min(args.steps, 10))
    for rows in (1, 4, 8, 16):
        case = X.with_rows(full, rows)
        for ep in (1, 2, 4, 8):
            blk = X.ExpertBlock(case, device, ep=ep, lib=lib, module=module)
            blk.run()
            torch.cuda.synchronize()
            assert not any(blk.statuses()), blk.statuses()
            d = blk.local_experts()
            us = blk.time_experts(iters)
            launches += 2 * ep * (iters + 2)
            slow = max(range(ep), key=lambda r: us[r])
            sweep.append({"rows": rows, "ep": ep, "distinct_experts": d, "us": [round(t, 1) for t in us],
                          "gb_s": [round(n * X.EXPERT_BYTES / (t * 1e-6) / 1e9, 1) if n else None for n, t in zip(d, us)],
                          "block_us": round(us[slow], 1),
                          "block_gb_s": round(sum(d) * X.EXPERT_BYTES / (us[slow] * 1e-6) / 1e9, 1)})  # fmt: skip
            del blk
            torch.cuda.empty_cache()
    head = next(x for x in sweep if x["rows"] == 16 and x["ep"] == 1)
    gbs = head["block_gb_s"]
    line = {
        "metric": "isolated NVFP4 expert block: achieved HBM GB/s of the routed experts' weight bytes", "value": gbs, "unit": "GB/s",
        "n_gpus": 1, "steps": iters, "warmup": 2, "ms_per_step": head["block_us"] / 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 experts (e2m1 x e4m3 block scales), f32 accumulate", "data": "synthetic",
        "config": {"workload": "configs[2]: isolated NVFP4 expert block, full expert shape, M in {1,4,8,16}, EP in {1,2,4,8} "
                               "(ranks run one after the other on 1 B200)", "l2": "flushed before every sample (512 MB write)",
                   "headline": "M=16, EP=1"},
        "roofline": {"bound": "hbm", "kernel": "experts_umma_kernel<g1> + <g2>", "achieved": gbs, "peak": peak, "unit": "GB/s",
                     "frac": gbs / peak, "traffic": None, "peak_kind": peak_kind},
        "sweep": sweep, "gpu_launches": launches, "clocks": sampler.stop(), "cpu_baseline": None,
        "e2e": {"value": None, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "the block has no host-facing call of its own: the layer launch of --config 1 is the end-to-end path"},
    }  # fmt: skip
    print(json.dumps(line), flush=True)


def run_expert_block_world(args) -> None:
    """configs[2] on N GPUs, one process each: an expert-parallel world of N ranks with E / N whole experts a rank; g2 stores
    its zb rows into every rank's zb, every rank's combine waits for all ranks. Per M in {1, 4, 8, 16}: g1 + g2 + combine
    between CUDA events on every rank (L2 flushed and the ranks aligned before each sample), the block's time = the slowest
    rank's median; the combined rows of every rank are compared bit for bit with rank 0's and with the same world emulated
    on rank 0's GPU."""
    import torch
    import torch.distributed as dist

    from sgl_muse_mega_b200.common import host
    from sgl_muse_mega_b200.muse_spark.b200 import expert_block as X

    world, rank, local = int(os.environ["WORLD_SIZE"]), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device(f"cuda:{local}")
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    lib = host.library()
    module = lib.load()
    sampler = ClockSampler(local) if rank == 0 else None
    cfg = X.block_config()
    full = X.draw_case(cfg, 16, device, seed=args.seed)
    peak, peak_kind = peaks()
    iters = max(3, min(args.steps, 10))
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=device)
    stream = torch.cuda.current_stream(device)
    sweep, launches, equal = [], 0, True
    for rows in (1, 4, 8, 16):
        case = X.with_rows(full, rows)
        blk = X.ExpertBlockRank(case, device, rank, world, lib=lib, module=module)
        blk.run()
        torch.cuda.synchronize()
        dist.barrier()
        assert blk.status() == 0, blk.status()
        ys = [torch.empty_like(blk.y) for _ in range(world)]
        dist.all_gather(ys, blk.y.contiguous())
        same = all(torch.equal(y.view(torch.int16), ys[0].view(torch.int16)) for y in ys[1:])
        emu_same = None
        if rank == 0:
            emu = X.ExpertBlock(case, device, ep=world, lib=lib, module=module)
            emu.run()
            torch.cuda.synchronize()
            emu_same = bool(torch.equal(emu.ranks[0].o["y"], blk.y))
            del emu
            torch.cuda.empty_cache()
        ts = []
        for _ in range(iters + 2):
            flush.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            blk.run_experts(stream.cuda_stream)
            b.record(stream)
            b.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        launches += 3 * (iters + 2)
        mine = torch.tensor([sorted(ts[2:])[len(ts[2:]) // 2], float(blk.local_experts())], device=device)
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        us, d = [float(e[0]) for e in every], [int(e[1]) for e in every]
        equal = equal and same and emu_same is not False
        sweep.append({"rows": rows, "ep": world, "distinct_experts": d, "us": [round(t, 1) for t in us], "block_us": round(max(us), 1),
                      "block_gb_s": round(sum(d) * X.EXPERT_BYTES / (max(us) * 1e-6) / 1e9, 1), "y_equal_on_every_rank": same,
                      "y_equal_to_the_emulated_world": emu_same})  # fmt: skip
        del blk
        torch.cuda.empty_cache()
        dist.barrier()
    clocks = sampler.stop() if sampler else None
    if rank == 0:
        head = sweep[-1]
        line = {
            "metric": "isolated NVFP4 expert block: achieved HBM GB/s of the routed experts' weight bytes", "value": head["block_gb_s"],
            "unit": "GB/s", "n_gpus": world, "steps": iters, "warmup": 2, "ms_per_step": head["block_us"] / 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4 experts (e2m1 x e4m3 block scales), f32 accumulate", "data": "synthetic",
            "config": {"workload": f"configs[2]: isolated NVFP4 expert block, full expert shape, M in {{1,4,8,16}}, EP = {world} ranks on "
                                   f"{world} B200s (whole experts per rank, zb rows exchanged through peer memory)",
                       "l2": "flushed before every sample (512 MB write)", "headline": f"M=16, EP={world}",
                       "timed": "g1 + g2 + combine (the combine waits for every rank's zb rows)"},
            "roofline": {"bound": "hbm", "kernel": "experts_umma_kernel<g1> + <g2>", "achieved": head["block_gb_s"] / world,
                         "peak": peak, "unit": "GB/s", "frac": head["block_gb_s"] / world / peak, "traffic": None, "peak_kind": peak_kind,
                         "note": "per GPU: the block's bytes over the slowest rank's time, divided by the ranks"},
            "parity_n": {"ranks": world, "bit_equal": equal},
            "sweep": sweep, "gpu_launches": launches, "clocks": clocks, "cpu_baseline": None,
            "e2e": {"value": None, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "note": "the block has no host-facing call of its own: the layer launch of --config 1 is the end-to-end path"},
        }  # fmt: skip
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def main() -> None:
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    elif args.timeline:
        run_timeline(args)
    elif args.config == 2:
        run_expert_block(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
