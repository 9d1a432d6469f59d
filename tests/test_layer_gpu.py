"""GPU parity of the decoder layer through the C ABI: every golden case (NVFP4 and bf16 experts, sliding-window and
global attention, tensor-parallel worlds 1/2/4/8 emulated on one device, ragged rows, the tail layer, b_live pads)."""

import pytest
import torch

from golden_cases import CASES
from parity import check_world
from sgl_muse_mega_b200.muse_spark.b200 import layer as L
from sgl_muse_mega_b200.muse_spark.b200 import synthetic

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    assert torch.cuda.is_available(), "these tests need the B200"
    return torch.device("cuda:0")


def _paths():
    """Every golden case on the default expert path (tcgen05: block-scaled NVFP4 stages, or the grouped bf16 GEMM of the
    bf16 layers, for shapes with whole tiles) and again on the general CUDA-core expert kernels."""
    out = []
    for name in CASES:
        out.append((name, True))
        out.append((name, False))
    return out


@pytest.mark.parametrize("name,tensor_cores", _paths())
def test_layer_parity(name, tensor_cores, device, golden_dir):
    cfg, kw = CASES[name]
    case = synthetic.layer_case(cfg, **kw)
    world = L.LayerWorld(case, device, tensor_cores=tensor_cores)
    taken = [r.tensor_cores_bf16 if kw.get("bf16") else r.tensor_cores for r in world.ranks]
    assert all(t == tensor_cores for t in taken), "the case did not take the expert path under test"
    world.run_interleaved()
    torch.cuda.synchronize()
    for r in world.ranks:
        st = r.launch_record.status(torch.cuda.current_stream().cuda_stream)
        assert st.code == 0, f"rank {r.rank}: device status {st.code} at {st.stage} (block {st.block}, observed {st.observed})"
    golden = torch.load(golden_dir / f"{name}.pt")
    check_world(world, sorted({0, cfg.tp - 1}), golden=golden)


def test_expert_paths_agree_to_rounding(device):
    """The tcgen05 expert kernels and the CUDA-core expert kernels, from bit-identical routed rows (ids and quantised
    expert inputs are compared exactly): both accumulate exact products in f32 but in another order, so a sum may differ
    in its last bit and move a value across a rounding boundary of the h requantisation: at least 99.9 % of the h-plane
    bytes are equal and zb agrees to 2e-3 (measured: all bytes equal on most seeds)."""
    cfg, kw = CASES["small_fp4_swa_tp2"]
    case = synthetic.layer_case(cfg, **kw)
    a = L.LayerWorld(case, device, tensor_cores=False)
    b = L.LayerWorld(case, device, tensor_cores=True)
    for w in (a, b):
        w.run_interleaved()
    torch.cuda.synchronize()
    for ra, rb in zip(a.ranks, b.ranks):
        assert torch.equal(ra.o["ids"], rb.o["ids"]) and torch.equal(ra.o["xq"], rb.o["xq"])
        for pa, pb in zip(ra.h_planes(), rb.h_planes()):
            assert (pa == pb).float().mean() > 0.999
        za, zb = ra.zb.view(torch.bfloat16).float(), rb.zb.view(torch.bfloat16).float()
        assert ((za - zb).norm() / za.norm()).item() < 2e-3


def test_bf16_expert_paths_agree_to_rounding(device):
    """A bf16 layer's experts as the grouped tensor-core GEMM and on the CUDA-core kernels, from bit-identical routed rows:
    both round the gate and up sums to bf16 before the SwiGLU, so the h rows differ only where an f32 sum in another order
    crosses a bf16 rounding boundary (one ulp, on well under 1 % of the elements), and zb agrees to 4e-3."""
    cfg, kw = CASES["small_bf16_global_tp8"]
    case = synthetic.layer_case(cfg, **kw)
    a = L.LayerWorld(case, device, tensor_cores=False)
    b = L.LayerWorld(case, device, tensor_cores=True)
    assert all(r.tensor_cores_bf16 for r in b.ranks) and not any(r.tensor_cores_bf16 for r in a.ranks)
    for w in (a, b):
        w.run_interleaved()
    torch.cuda.synchronize()
    for ra, rb in zip(a.ranks, b.ranks):
        for r in (ra, rb):
            st = r.launch_record.status(torch.cuda.current_stream().cuda_stream)
            assert st.code == 0, (st.code, st.stage)
        assert torch.equal(ra.o["ids"], rb.o["ids"]) and torch.equal(ra.o["xq"], rb.o["xq"])
        ha, hb = ra.z.view(torch.bfloat16).float(), rb.z.view(torch.bfloat16).float()
        assert (ha != hb).float().mean() < 0.01 and ((ha - hb).norm() / ha.norm()).item() < 2e-3
        za, zb = ra.zb.view(torch.bfloat16).float(), rb.zb.view(torch.bfloat16).float()
        assert ((za - zb).norm() / za.norm()).item() < 4e-3


def test_b_live_pads(device, golden_dir):
    cfg, kw = CASES["small_fp4_swa_tp2"]
    case = synthetic.layer_case(cfg, **kw)
    world = L.LayerWorld(case, device, b_live=8)
    world.run_interleaved()
    torch.cuda.synchronize()
    check_world(world, [0, 1], b_live=8)
    assert not world.ranks[0].o["y"][8:].any()


def test_replay_is_bitwise_deterministic(device):
    """Eager run == second run == CUDA-graph replay, bit for bit (the reference's determinism check,
    test/kernels/test_verify_step.py)."""
    cfg, kw = CASES["small_fp4_swa_tp1_m5"]
    case = synthetic.layer_case(cfg, **kw)
    world = L.LayerWorld(case, device)
    rank = world.ranks[0]
    stream = torch.cuda.Stream(device)

    def snapshot():
        torch.cuda.synchronize()
        return {k: v.clone() for k, v in rank.values().items()}

    with torch.cuda.stream(stream):
        rank.launch(stream.cuda_stream, pdl=True)
    first = snapshot()
    with torch.cuda.stream(stream):
        rank.launch(stream.cuda_stream, pdl=False)
    second = snapshot()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        rank.launch(torch.cuda.current_stream().cuda_stream, pdl=True)
    for v in rank.o.values():
        v.zero_()
    graph.replay()
    third = snapshot()
    graph.replay()
    fourth = snapshot()
    for k in first:
        for other in (second, third, fourth):
            assert torch.equal(first[k].view(torch.uint8), other[k].view(torch.uint8)), k
    assert rank.launch_record.status(stream.cuda_stream).code == 0


def test_non_finite_rows_are_routed_in_range_and_recorded(device):
    """A NaN residual row gives NaN router scores: the routing still names k distinct experts of the model for it (the
    lowest ids), the other rows are untouched, and the status block says which stage met it; nothing traps."""
    cfg, kw = CASES["small_fp4_swa_tp1_m5"]
    case = synthetic.layer_case(cfg, **kw)
    clean = L.LayerWorld(case, device)
    clean.run_interleaved()
    world = L.LayerWorld(case, device)
    rank = world.ranks[0]
    rank.w["stream_in"][2] = float("nan")
    world.run_interleaved()
    torch.cuda.synchronize()
    ids = rank.o["ids"].cpu()
    assert int(ids.min()) >= 0 and int(ids.max()) < cfg.experts
    assert ids[2].tolist() == list(range(cfg.topk))
    keep = [0, 1, 3, 4]
    assert torch.equal(ids[keep], clean.ranks[0].o["ids"].cpu()[keep])
    st = rank.launch_record.status(torch.cuda.current_stream().cuda_stream)
    assert (st.code, st.stage, st.block) == (6, 6, 2)


@pytest.mark.parametrize("name", ["small_fp4_swa_tp1_m5", "downscaled_m1"])
def test_fused_layer_parity(name, device):
    """The fused form (two persistent segment kernels around the expert kernels) through one mk_launch, stage by stage
    against the oracle like the per-stage kernels."""
    cfg, kw = CASES[name]
    case = synthetic.layer_case(cfg, **kw)
    world = L.LayerWorld(case, device, packed=0)
    rank = world.ranks[0]
    rank.bind(world.ranks, fused=True)
    assert rank.launch_record.info().kernels == 7 - int(rank.tensor_cores)  # the tensor-core g2 forms the h-row view itself
    rank.launch(torch.cuda.current_stream().cuda_stream, pdl=True)
    torch.cuda.synchronize()
    assert rank.launch_record.status(torch.cuda.current_stream().cuda_stream).code == 0
    check_world(world, [0])


@pytest.mark.parametrize("name", ["small_fp4_swa_tp8", "small_bf16_tail_tp4", "small_fp4_global_tp8_baseline"])
def test_fused_matches_per_stage_kernels_on_a_lone_rank(name, device):
    """One rank of a larger world alone (its peers' contributions absent in every run): the three forms of the dense
    stages (cluster split-K GEMMs, item-engine GEMMs, two fused segments) give the same routing and the same values up to
    f32 summation order."""
    cfg, kw = CASES[name]
    case = synthetic.layer_case(cfg, **kw)
    outs = []
    drop = (1 if case.bf16 else 0) + (1 if case.tail else 0)  # no h-row view, no successor qkv
    for form in (2, 0, 1):
        rank = L.LayerRank(host_lib(), _module(device), case, 1, device, packed=0)
        rank.bind(None, fused=form)
        hrow = 0 if case.bf16 or rank.tensor_cores else 1  # the h-row kernel: CUDA-core NVFP4 experts only
        assert rank.launch_record.info().kernels == {2: 13 + hrow - (1 if case.tail else 0), 0: 12 + hrow - (1 if case.tail else 0),
                                                     1: 6 + hrow}[form]
        rank.launch(torch.cuda.current_stream().cuda_stream, pdl=True)
        torch.cuda.synchronize()
        assert rank.launch_record.status(torch.cuda.current_stream().cuda_stream).code == 0
        outs.append({k: v.clone() for k, v in rank.values().items()})
    b = outs[0]
    for a in outs[1:]:
        assert torch.equal(a["ids"], b["ids"])
        for k in a:
            if a[k].dtype in (torch.int32, torch.uint8):
                continue
            x, y = a[k].float(), b[k].float()
            rel = ((x - y).norm() / y.norm().clamp_min(1e-20)).item()
            assert rel < 2e-2, (k, rel)


_MOD = {}


def host_lib():
    from sgl_muse_mega_b200.common import host

    return host.library()


def _module(device):
    if device not in _MOD:
        with torch.cuda.device(device):
            _MOD[device] = host_lib().load()
    return _MOD[device]


@pytest.mark.parametrize("name", ["small_fp4_swa_tp2", "small_bf16_tail_tp4"])
def test_item_images_give_the_same_bits(name, device):
    """The dense weights as item images (one bulk copy an item) against row-major weights (one copy a row): the same
    arithmetic in the same order, so every output of the layer is bit-identical."""
    cfg, kw = CASES[name]
    case = synthetic.layer_case(cfg, **kw)
    a, b = L.LayerWorld(case, device, packed=0), L.LayerWorld(case, device, packed=1)
    a.run_interleaved()
    b.run_interleaved()
    torch.cuda.synchronize()
    for ra, rb in zip(a.ranks, b.ranks):
        assert ra.launch_record.status(torch.cuda.current_stream().cuda_stream).code == 0
        assert rb.launch_record.status(torch.cuda.current_stream().cuda_stream).code == 0
        for k, v in ra.o.items():
            if torch.is_tensor(v):
                assert torch.equal(v, rb.o[k]), k


@pytest.mark.parametrize("rows", [1, 4, 8, 16])
@pytest.mark.parametrize("tp", [1, 2])
def test_window_rows_sweep(rows, tp, device):
    """The verify window of M = 1, 4, 8 and 16 rows (the expert-block sweep of the benchmark configurations) through the
    whole layer, every stage against the oracle fed the kernels' own inputs; tensor-core experts, dense weights as tile
    images on the tensor-core engine."""
    from golden_cases import small_cfg

    cfg = small_cfg(tp)
    case = synthetic.layer_case(cfg, rows=rows, ctx=29, band="baseline", seed=40 + rows)
    world = L.LayerWorld(case, device)
    world.run_interleaved()
    torch.cuda.synchronize()
    for r in world.ranks:
        assert r.tensor_cores and r.packed == 2
        assert r.launch_record.status(torch.cuda.current_stream().cuda_stream).code == 0
    check_world(world, list(range(tp)))


@pytest.mark.parametrize("name", ["small_fp4_swa_tp8", "small_fp4_swa_tp1_m5", "small_bf16_tail_tp4", "downscaled_m1"])
def test_dense_engines_agree(name, device, golden_dir):
    """The dense GEMMs on the tensor-core engine (tile images, tcgen05 with the whole K accumulated in tensor memory) against
    the item engine (mma.sync, partial sums per K chunk): the same routing, the same values up to f32 summation order, and
    each engine within the per-stage bounds of the oracle."""
    cfg, kw = CASES[name]
    case = synthetic.layer_case(cfg, **kw)
    outs = []
    for packed in (2, 1):
        world = L.LayerWorld(case, device, packed=packed)
        assert all(r.packed == packed for r in world.ranks)
        world.run_interleaved()
        torch.cuda.synchronize()
        for r in world.ranks:
            st = r.launch_record.status(torch.cuda.current_stream().cuda_stream)
            assert st.code == 0, (packed, r.rank, st.code, st.stage, st.block, st.observed)
        check_world(world, [0])
        outs.append({k: v.clone() for k, v in world.ranks[0].values().items()})
    a, b = outs
    assert torch.equal(a["ids"], b["ids"])
    for k in ("branch", "h3", "pooled", "logits", "ffn_out", "qkv_next"):
        if k in a:
            x, y = a[k].float(), b[k].float()
            assert ((x - y).norm() / y.norm().clamp_min(1e-20)).item() < 4e-3, k


@pytest.mark.parametrize("name", ["small_fp4_swa_tp1_m5", "downscaled_m1"])
def test_fused_tensor_core_layer_parity(name, device):
    """The fused form on the tensor-core engine (kernel A: o_proj .. routing, kernel B: combine .. qkv head, the row work
    on the epilogue warps between the GEMM stages) through one mk_launch: stage by stage against the oracle like the
    per-stage kernels, twice in a row (the dependency words only grow), then as a CUDA graph, bit for bit the same."""
    cfg, kw = CASES[name]
    case = synthetic.layer_case(cfg, **kw)
    world = L.LayerWorld(case, device)
    rank = world.ranks[0]
    assert rank.packed == 2
    rank.bind(world.ranks, fused=True)
    assert rank.launch_record.info().kernels == 6
    s = torch.cuda.current_stream().cuda_stream
    rank.launch(s, pdl=True)
    torch.cuda.synchronize()
    st = rank.launch_record.status(s)
    assert st.code == 0, (st.code, st.stage, st.block, st.observed, st.expected)
    check_world(world, [0])
    first = {k: v.clone() for k, v in rank.values().items()}
    for v in rank.o.values():
        v.zero_()
    rank.launch(s, pdl=False)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream(device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        rank.launch(torch.cuda.current_stream().cuda_stream, pdl=True)
    for rep in range(2):
        for v in rank.o.values():
            v.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for k, v in rank.values().items():
            assert torch.equal(first[k].view(torch.uint8), v.view(torch.uint8)), (rep, k)
    assert rank.launch_record.status(s).code == 0


@pytest.mark.parametrize("name", ["small_fp4_swa_tp8", "small_bf16_tail_tp4", "small_fp4_global_tp8_baseline"])
def test_fused_tensor_core_matches_per_stage_on_a_lone_rank(name, device):
    """One rank of a larger world alone (its peers' contributions absent in both runs): the fused tensor-core kernels
    against the per-stage kernels on the same tile images: the same routing and the same values up to f32 summation order
    (the fused kernel cuts its GEMM stages over one grid, the row stages sum on 128 threads)."""
    cfg, kw = CASES[name]
    case = synthetic.layer_case(cfg, **kw)
    outs = []
    for form in (0, 1):
        rank = L.LayerRank(host_lib(), _module(device), case, 1, device)
        rank.bind(None, fused=form)
        rank.launch(torch.cuda.current_stream().cuda_stream, pdl=True)
        torch.cuda.synchronize()
        st = rank.launch_record.status(torch.cuda.current_stream().cuda_stream)
        assert st.code == 0, (form, st.code, st.stage, st.block, st.observed, st.expected)
        outs.append({k: v.clone() for k, v in rank.values().items()})
    b, a = outs
    assert torch.equal(a["ids"], b["ids"])
    for k in a:
        if a[k].dtype in (torch.int32, torch.uint8):
            continue
        x, y = a[k].float(), b[k].float()
        rel = ((x - y).norm() / y.norm().clamp_min(1e-20)).item()
        assert rel < 2e-2, (k, rel)


def test_a_missing_peer_runs_the_wait_out_and_is_recorded(device):
    """Failure detection without a fault: rank 0 of a two-rank world is launched alone with a poll budget of 64, so the
    all-reduce wait of its post-attention norm expects two arrivals and sees one. The launch must return (nothing hangs,
    nothing traps), the status block must name the wait (code 1, the post-norm stage, one of two arrivals seen), the later
    waits of the launch give up at once, and the next launch on the device (a lone rank bound normally: tensor memory was
    released, the context is intact) is clean and within the oracle's bounds."""
    cfg, kw = CASES["small_fp4_swa_tp2"]
    case = synthetic.layer_case(cfg, **kw)
    world = L.LayerWorld(case, device)
    r0 = world.ranks[0]
    r0.bind(world.ranks, wait_budget=64)
    s = torch.cuda.current_stream().cuda_stream
    r0.launch(s, pdl=True)  # rank 1 never launches: its contributions never arrive
    torch.cuda.synchronize()
    st = r0.launch_record.status(s)
    assert (st.code, st.stage) == (1, L.STAGE_NAMES.index("post_norm")), (st.code, st.stage)
    assert (st.observed, st.expected) == (1, 2), (st.observed, st.expected)
    # the same device right after: a normally bound launch is clean
    cfg1, kw1 = CASES["small_fp4_swa_tp1_m5"]
    clean = L.LayerWorld(synthetic.layer_case(cfg1, **kw1), device)
    clean.run_interleaved()
    torch.cuda.synchronize()
    assert clean.ranks[0].launch_record.status(s).code == 0
    check_world(clean, [0])


@pytest.mark.parametrize("global_attn,bf16", [(False, False), (True, False), (True, True)])
def test_full_shape_layer_parity(global_attn, bf16, device):
    """The benchmark's own configuration as a whole layer: the full-shape model's TP8 world (hidden 8192, 16 query / 2 kv
    heads a rank, 256 experts top-8, expert width 4096) on one device, M = 16 rows over an 8192-token context, one
    sliding-window and one global layer, NVFP4 experts on the tensor cores (and a bf16-expert layer on the grouped
    tensor-core GEMM), dense GEMMs on tile images. Every stage of
    ranks 0 and 7 against the oracle fed the kernels' own inputs, routing ids exact. The routing is confined to 24 hot
    experts (a +1 bias on them, as the reference's real-dims CPU test does) so that the CPU oracle holds the weights."""
    from sgl_muse_mega_b200.muse_spark.config import Config

    cfg = Config()
    hot = torch.randperm(cfg.experts, generator=torch.Generator().manual_seed(1))[:24]
    case = synthetic.layer_case(cfg, rows=16, ctx=8192, global_attn=global_attn, band="baseline", seed=1, experts_subset=hot,
                                bf16=bf16)  # fmt: skip
    world = L.LayerWorld(case, device)
    assert all((r.tensor_cores_bf16 if bf16 else r.tensor_cores) and r.packed == 2 for r in world.ranks)
    world.run_interleaved()
    torch.cuda.synchronize()
    for r in world.ranks:
        st = r.launch_record.status(torch.cuda.current_stream().cuda_stream)
        assert st.code == 0, f"rank {r.rank}: device status {st.code} at {st.stage} (block {st.block}, observed {st.observed})"
    report = check_world(world, [0, cfg.tp - 1])
    ids = world.ranks[0].o["ids"].cpu()
    assert set(ids.flatten().tolist()) <= set(hot.tolist())
    print({k[1]: f"{v:.1e}" for k, v in report.items() if k[0] == 0})
