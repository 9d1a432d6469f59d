"""The C-ABI library without a GPU: it loads, exports every symbol the header declares, computes buffer extents and
validates binds (pack-only records, as the reference's CPU parameter-block tests use them: test_param_blocks.py)."""

import ctypes
import re

import pytest
import torch

from golden_cases import CASES, small_cfg
from sgl_muse_mega_b200.common import host
from sgl_muse_mega_b200.muse_spark.b200 import layer as L
from sgl_muse_mega_b200.muse_spark.b200 import synthetic
from sgl_muse_mega_b200.muse_spark.config import Config


@pytest.fixture(scope="module")
def lib():
    return host.library()


def declared_functions():
    text = host.HEADER.read_text()
    return sorted(set(re.findall(r"^(?:int|void|const char\*)\s+(mk_\w+)\s*\(", text, re.M)))


def test_exports_every_declared_symbol(lib):
    names = declared_functions()
    assert set(names) == set(host.EXPORTS), (names, host.EXPORTS)
    for n in names:
        assert getattr(lib.dll, n) is not None, n


def test_struct_mirrors_have_only_abi_scalars():
    for name, cls in host.STRUCTS.items():
        assert ctypes.sizeof(cls) % 8 == 0, name
        assert cls._fields_, name


def test_make_demands_every_field():
    with pytest.raises(ValueError, match="missing"):
        host.make("MkLayerShape", rows=16)


def test_constants_full_shape(lib):
    cfg = Config()
    shape = host.make(
        "MkLayerShape", rows=16, hidden=cfg.hidden, moe_hidden=cfg.moe_hidden, q_heads=cfg.q_heads_rank,
        kv_heads=cfg.kv_heads_rank, experts=cfg.experts, topk=cfg.topk, inter=cfg.moe_inter, ranks=8, node_ranks=4,
        rank=3, window=2047, bf16=0, tail=0, next_rope=1,
    )  # fmt: skip
    c = lib.layer_constants(shape)
    assert c.stages == host.MACROS["MKH_LAYER_STAGES"]
    assert (c.slots, c.qkv_row, c.kv_row_bytes, c.inter_rank, c.hidden_rank) == (128, 2304, 256, 512, 512)
    assert c.ar_bytes == 8 * 16 * 8192 * 2 and c.zb_bytes == 128 * 4096 * 2 and c.z_bytes == 128 * 2048
    assert c.ws_bytes > 0 and c.ws_bytes % 256 == 0


@pytest.mark.parametrize("field,value,msg", [("rows", 17, "rows"), ("ranks", 3, "ranks"), ("hidden", 100, "hidden")])
def test_bad_shapes_are_refused(lib, field, value, msg):
    kw = dict(rows=16, hidden=1024, moe_hidden=1024, q_heads=8, kv_heads=1, experts=16, topk=8, inter=1024, ranks=8,
              node_ranks=4, rank=0, window=7, bf16=0, tail=0, next_rope=1)  # fmt: skip
    kw[field] = value
    shape = host.make("MkLayerShape", **kw)
    c = host.STRUCTS["MkLayerConstants"]()
    assert lib.dll.mk_layer_constants(ctypes.byref(shape), ctypes.byref(c)) == -1
    assert msg in lib.dll.mk_last_error().decode()


def test_pack_only_bind_and_refusals(lib):
    """A bind without a module validates every operand and yields a record that reports its geometry but cannot launch."""
    cfg, kw = CASES["small_fp4_swa_tp2"]
    case = synthetic.layer_case(cfg, **kw)
    rank = L.LayerRank(lib, None, case, 0, torch.device("cpu"), packed=0)
    rec = rank.bind(fused=2)
    info = rec.info()
    # 17 stage slots; top-k + tables + nq share a launch, the row ops ride the qkv GEMM, the h-row view the tensor-core g2
    assert info.kernels == 13 and info.grid > 0 and info.smem > 0
    # the fused form on request: attention x 2, segment A, g1, h row, g2, segment B
    # default: the GEMMs on the item engine, pooler + router in one launch
    assert rank.bind().info().kernels == 12 and rank.bind(fused=1).info().kernels == 6
    plain = L.LayerRank(lib, None, case, 0, torch.device("cpu"), packed=0, tensor_cores=False)
    assert plain.bind().info().kernels == 13  # CUDA-core experts keep the h-row kernel
    with pytest.raises(RuntimeError, match="pack-only"):
        rec(0, False)
    # a missing operand is named
    rank.w["o_proj"] = None
    with pytest.raises(RuntimeError, match="w_o"):
        rank.bind()


def test_tile_images_bind_on_the_tensor_core_engine_only(lib):
    """The default layout of the dense weights is the tile image of the tensor-core engine (dense_packed 2): it binds the
    per-stage launch list (12 kernels) or the two fused kernels (6), and refuses the cluster split-K form."""
    cfg, kw = CASES["small_fp4_swa_tp2"]
    case = synthetic.layer_case(cfg, **kw)
    rank = L.LayerRank(lib, None, case, 0, torch.device("cpu"))
    assert rank.packed == 2 and rank.w["o_proj"].dtype == torch.uint8 and rank.w["o_proj"].shape[2:] == (2, 128, 128)
    assert rank.bind().info().kernels == 12
    assert rank.bind(fused=1).info().kernels == 6  # the two fused tensor-core kernels around the experts
    with pytest.raises(RuntimeError, match="dense_packed 2"):
        rank.bind(fused=2)


def test_expert_range_binds_whole_experts_only(lib):
    """Expert parallelism of the expert block: a lone-rank shape keeps its experts [lo, hi) (sliced and packed on their
    own, bound by pointers moved back by lo experts); bad ranges and tensor-parallel shapes are refused."""
    from sgl_muse_mega_b200.muse_spark.b200 import expert_block as X

    cfg = X.block_config(experts=16, moe_hidden=1024, moe_inter=1024)
    case = synthetic.layer_case(cfg, rows=4, ctx=8, seed=5)
    rank = L.LayerRank(lib, None, case, 0, torch.device("cpu"), expert_range=(4, 8))
    assert rank.w["gate_q"].shape[0] == 4 and rank.w1_pack.shape[0] == 4 and rank.w["expert_bias"].shape[0] == 16
    rec = rank.bind()
    assert rec.info().kernels == 12
    for lo, hi in ((4, 4), (8, 4), (0, 17), (-1, 4)):
        rank.expert_lo, rank.expert_hi = lo, hi
        with pytest.raises(RuntimeError, match="expert range"):
            rank.bind()
    tp2 = synthetic.layer_case(small_cfg(2), rows=4, ctx=8, seed=6)
    r2 = L.LayerRank(lib, None, tp2, 0, torch.device("cpu"), expert_range=(0, 8))
    with pytest.raises(RuntimeError, match="whole experts"):
        r2.bind()


def test_expert_parallel_world_binds_every_ranks_zb_and_flags(lib):
    """One process per GPU with whole experts per rank: the bind takes every rank's zb rows and flag block (here: device
    addresses of a peer's mapped arena) and refuses a world with a missing peer, without an expert range or without the
    packed images."""
    from types import SimpleNamespace as NS

    from sgl_muse_mega_b200.muse_spark.b200 import expert_block as X

    cfg = X.block_config(experts=16, moe_hidden=1024, moe_inter=1024)
    case = synthetic.layer_case(cfg, rows=4, ctx=8, seed=5)
    rank = L.LayerRank(lib, None, case, 0, torch.device("cpu"), expert_range=(8, 16))
    peer = NS(zb=0x7F0000001000, flags=0x7F0000002000)
    assert rank.bind(ep_peers=[peer, None], ep_rank=1).info().kernels == 12
    with pytest.raises(RuntimeError, match="zb_peer\\[0\\] or flags_peer\\[0\\]"):
        rank.bind(ep_peers=[NS(zb=0, flags=0), None], ep_rank=1)
    with pytest.raises(ValueError, match="exceed 8"):
        rank.bind(ep_peers=[peer] * 9, ep_rank=1)
    plain = L.LayerRank(lib, None, case, 0, torch.device("cpu"), expert_range=(8, 16), tensor_cores=False)
    with pytest.raises(RuntimeError, match="expert-parallel world needs"):
        plain.bind(ep_peers=[peer, None], ep_rank=1)
    lay = X.ep_layout(4096)
    assert lay.offset("flags") == 0 and lay.offset("zb") >= 256


def test_packet_mode_binds_and_marks_the_exchange_rows(lib):
    """``packets``: the bind fills this rank's four bf16 exchange buffers with the "not arrived" mark, keeps the kernel
    count, and refuses the fused form; an expert-parallel world in packet mode needs no peer flag block."""
    from types import SimpleNamespace as NS

    from sgl_muse_mega_b200.muse_spark.b200 import expert_block as X

    cfg, kw = CASES["small_fp4_swa_tp2"]
    case = synthetic.layer_case(cfg, **kw)
    rank = L.LayerRank(lib, None, case, 0, torch.device("cpu"))
    assert not bool((rank.ar.view(torch.uint8) == 0xFF).any())
    assert rank.bind(packets=True).info().kernels == rank.bind().info().kernels
    for t in (rank.ar, rank.pool_ag, rank.zb, rank.unpool_ag):
        assert bool((t.view(torch.uint8) == 0xFF).all())
    with pytest.raises(RuntimeError, match="fused"):
        rank.bind(fused=1, packets=True)
    ecfg = X.block_config(experts=16, moe_hidden=1024, moe_inter=1024)
    ecase = synthetic.layer_case(ecfg, rows=4, ctx=8, seed=5)
    ep = L.LayerRank(lib, None, ecase, 0, torch.device("cpu"), expert_range=(8, 16))
    assert ep.bind(ep_peers=[NS(zb=0x7F0000001000, flags=0), None], ep_rank=1, packets=True).info().kernels == 12


def test_launch_params_show_the_exchange_wiring(lib):
    """``mk_launch_params`` on pack-only records: a lone rank's binds, a two-rank world with counter words and with
    packets, and ranks 0 / 1 of an eight-rank world alone (a slice: absent sources read as zero, present ones are polled)."""
    from types import SimpleNamespace as NS

    cfg, kw = CASES["small_fp4_swa_tp2"]
    case = synthetic.layer_case(cfg, **kw)
    a, b = (L.LayerRank(lib, None, case, r, torch.device("cpu")) for r in range(2))
    p = a.bind([a, b]).params()
    assert p["stages"]["fused"] == 0
    # counter words: every producer signals both ranks, every consumer counts two contributors
    for name in ("o_proj", "pooler", "g1", "g2", "unpooler"):
        assert p[f"{name}.signal"]["signal"] == 2 and p[f"{name}.signal"]["remote"] == 1, name
    for name in ("post_norm", "nq", "g2", "combine", "cross_norm"):
        assert p[f"{name}.wait"]["wait"] == "counter" and p[f"{name}.wait"]["contributors"] == 2, name
    # packets: the four bf16 exchanges neither signal nor count; the h planes keep their counter word, g1 announces its epoch
    p = a.bind([a, b], packets=True).params()
    for name in ("o_proj", "pooler", "g2", "unpooler"):
        assert p[f"{name}.signal"]["signal"] == 0, name
    assert p["g1.signal"] == {"signal": 2, "remote": 1, "target": 1}
    assert p["g2.wait"]["wait"] == "counter" and p["g2.wait"]["target"] == 1
    P, H = cfg.moe_hidden, cfg.hidden
    assert p["post_norm.wait"] == {"wait": "packets", "present": 3, "band": 0, "contributors": 0, "target": 0}
    assert p["nq.wait"]["present"] == 3 and p["nq.wait"]["band"] == P // 2
    assert p["combine.wait"]["present"] == 3 and p["combine.wait"]["band"] == P // 2
    assert p["cross_norm.wait"]["present"] == 3 and p["cross_norm.wait"]["band"] == H // 2
    # a lone rank with packets: the rows are handed over inside the rank
    p = a.bind(packets=True).params()
    assert p["post_norm.wait"]["wait"] == "packets" and p["post_norm.wait"]["present"] == 1 and p["o_proj.signal"]["signal"] == 0
    # ranks 0 and 1 of an eight-rank world (node groups of four): the absent ranks' parts are not polled
    cfg8, kw8 = CASES["small_fp4_swa_tp8"]
    case8 = synthetic.layer_case(cfg8, **kw8)
    r0, r1 = (L.LayerRank(lib, None, case8, r, torch.device("cpu")) for r in range(2))
    p = r1.bind([r0, r1] + [None] * 6, packets=True).params()
    assert p["post_norm.wait"]["present"] == 0b11 and p["combine.wait"]["present"] == 0b11
    assert p["combine.wait"]["band"] == cfg8.moe_hidden // 8
    assert p["nq.wait"]["present"] == 0b11 and p["nq.wait"]["band"] == cfg8.moe_hidden // 4  # the node group's bands
    assert p["cross_norm.wait"]["band"] == cfg8.hidden // 4
    assert p["g1.signal"]["signal"] == 2  # the h planes go to the present ranks


def test_module_load_needs_builtin_image(lib):
    out = ctypes.c_void_p()
    assert lib.dll.mk_module_load(b"xx", 2, None, ctypes.byref(out)) == -1
    assert "image NULL" in lib.dll.mk_last_error().decode()


def test_tail_and_bf16_variants_drop_stages(lib):
    cfg, kw = CASES["small_bf16_tail_tp4"]
    case = synthetic.layer_case(cfg, **kw)
    rank = L.LayerRank(lib, None, case, 1, torch.device("cpu"), packed=0)
    assert rank.bind(fused=2).info().kernels == 14 - 2  # no h-row view (bf16), no successor qkv (tail)
    assert rank.bind(fused=0).info().kernels == 13 - 2
    assert rank.bind(fused=1).info().kernels == 7 - 1  # the fused form: no h-row view either


def test_bf16_layers_bind_tile_images_of_their_experts(lib):
    """A bf16 layer with whole tiles packs one tile image per expert (gate and up rows of a feature block in one tile) and
    binds the grouped tensor-core GEMM; the image inverts to the shards."""
    from sgl_muse_mega_b200.muse_spark.b200 import weights as W

    cfg, kw = CASES["small_bf16_global_tp8"]
    case = synthetic.layer_case(cfg, **kw)
    rank = L.LayerRank(lib, None, case, 3, torch.device("cpu"))
    assert rank.tensor_cores_bf16 and not rank.tensor_cores
    e, i_s, p = rank.w["gate"].shape
    h_s, inter = rank.w["w2"].shape[1:]
    assert rank.w1_pack.shape == (e * 2 * i_s // 128, p * 2 // 256, 2, 128, 128)
    assert rank.w2_pack.shape == (e * h_s // 128, inter * 2 // 256, 2, 128, 128)
    w1 = W.unpack_umma(rank.w1_pack, e * 2 * i_s, torch.bfloat16).view(e, 2 * i_s // 128, 2, 64, p)
    assert torch.equal(w1[:, :, 0].reshape(e, i_s, p), rank.w["gate"]) and torch.equal(w1[:, :, 1].reshape(e, i_s, p), rank.w["up"])
    assert torch.equal(W.unpack_umma(rank.w2_pack, e * h_s, torch.bfloat16).view(e, h_s, inter), rank.w["w2"])
    assert rank.bind().info().kernels == 12  # a bf16 layer has no h-row view on either expert path
    plain = L.LayerRank(lib, None, case, 3, torch.device("cpu"), tensor_cores=False)
    assert not plain.tensor_cores_bf16 and plain.w1_pack is None and plain.bind().info().kernels == 12


def test_weight_images_round_trip_and_layout():
    """The tensor-core weight images invert exactly, and a byte lands where the kernel's descriptors expect it."""
    from sgl_muse_mega_b200.muse_spark.b200 import weights as W

    g = torch.Generator().manual_seed(5)
    e, i_s, p, h_s, i = 3, 256, 512, 128, 768
    gq, uq = (torch.randint(0, 256, (e, i_s, p // 2), generator=g, dtype=torch.uint8) for _ in range(2))
    gs, us = (torch.randint(0, 127, (e, i_s, p // 16), generator=g, dtype=torch.uint8) for _ in range(2))
    pack = W.pack_w1_fp4(gq, gs, uq, us)
    assert pack.shape == (e, i_s // 128, p // 256, W.W1_STAGE)
    for a, b in zip(W.unpack_w1_fp4(pack), (gq, gs, uq, us)):
        assert torch.equal(a, b)
    wq = torch.randint(0, 256, (e, h_s, i // 2), generator=g, dtype=torch.uint8)
    ws = torch.randint(0, 127, (e, h_s, i // 16), generator=g, dtype=torch.uint8)
    p2 = W.pack_w2_fp4(wq, ws)
    assert p2.shape == (e, 1, 3, W.W2_STAGE)
    for a, b in zip(W.unpack_w2_fp4(p2), (wq, ws)):
        assert torch.equal(a, b)
    # spot checks of the byte addresses: expert 1, block 1, K chunk 1; tile row r, logical 16-byte chunk j, byte t
    ex, blk, kc, r, j, t = 1, 1, 1, 77, 5, 9
    off = (r // 8) * 1024 + (r % 8) * 128 + ((j ^ (r % 8)) * 16) + t
    assert pack[ex, blk, kc, off] == gq[ex, blk * 128 + r, kc * 128 + j * 16 + t]
    assert pack[ex, blk, kc, W.TILE_BYTES + off] == uq[ex, blk * 128 + r, kc * 128 + j * 16 + t]
    block, grp = 2, 3  # K64 block of the chunk, 16-element group inside it
    n, gq4 = r % 32, r // 32
    sf_off = 2 * W.TILE_BYTES + block * 512 + n * 16 + gq4 * 4 + grp
    assert pack[ex, blk, kc, sf_off] == gs[ex, blk * 128 + r, kc * 16 + block * 4 + grp]
