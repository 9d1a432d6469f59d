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


@pytest.mark.parametrize("name", list(CASES))
def test_layer_parity(name, device, golden_dir):
    cfg, kw = CASES[name]
    case = synthetic.layer_case(cfg, **kw)
    world = L.LayerWorld(case, device)
    world.run_interleaved()
    torch.cuda.synchronize()
    golden = torch.load(golden_dir / f"{name}.pt")
    check_world(world, sorted({0, cfg.tp - 1}), golden=golden)


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
