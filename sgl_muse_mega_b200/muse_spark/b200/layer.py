"""Device state and binding of one decoder-layer launch per rank.

Counterpart of the reference's ``sm103/buffers.py:42-399`` (device + symmetric state) and of ``Stack.layer_bind`` in
``sm103/verify.py:246-386``: every buffer a layer launch reads or writes is allocated here once, the bind struct is
filled by field name and the launch record is bound once; ``LayerRank.launch`` is then the only per-step call.

``LayerWorld`` holds every rank of a tensor-parallel world on ONE device and wires their exchange buffers to each other
as peers. It serves the parity tests (the ranks' stages are interleaved with ``Launch.step`` so that every exchange has
all its contributions) and the single-GPU benchmark of one rank's slice (the other ranks' contributions stay in place
from a first interleaved pass). On a multi-GPU world the same bind takes the peers' mapped pointers instead.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ...common import host
from ..config import Config
from . import weights

# stage groups between which every rank must have finished before any rank continues (the exchanges)
STAGE_GROUPS = ((0, 3), (3, 2), (5, 5), (10, 2), (12, 2), (14, 3))
EXPERT_FIELDS = ("gate_q", "gate_sf", "up_q", "up_sf", "w2_q", "w2_sf", "g1_alphas", "g1_scale_c", "g2_alphas", "gate", "up", "w2")
STAGE_NAMES = (
    "attn_split", "attn_combine", "o_proj", "post_norm", "pooler", "router", "topk", "nq", "route_tables", "g1",
    "h_row", "g2", "combine", "unpooler", "cross_norm", "qkv", "rowops",
)  # fmt: skip


def layer_shape(cfg: Config, case, rank: int):
    return host.make(
        "MkLayerShape",
        rows=case.rows, hidden=cfg.hidden, moe_hidden=cfg.moe_hidden, q_heads=cfg.q_heads_rank,
        kv_heads=cfg.kv_heads_rank, experts=cfg.experts, topk=cfg.topk, inter=cfg.moe_inter, ranks=cfg.tp,
        node_ranks=cfg.node_ranks, rank=rank, window=0 if case.global_attn else cfg.swa_window,
        bf16=int(case.bf16), tail=int(case.tail), next_rope=int(not (case.next_global or case.tail)),
    )  # fmt: skip


class LayerRank:
    """One rank's weights (moved to the device), buffers and bound launch of one layer."""

    def __init__(self, lib: host.Library, module, case, rank: int, device, kv_rows: Optional[int] = None, tensors=None,
                 tensor_cores: bool = True, keep_plain_experts: bool = True, io: Optional[dict] = None,
                 packed: Optional[int] = None, expert_range: Optional[tuple] = None):  # fmt: skip
        """``io`` replaces buffers this layer would allocate with ones it shares with its neighbours in a stack: inputs
        ``qkv_in`` / ``stream_in`` (the predecessor's outputs), ``k_cache`` / ``v_cache`` (the pools the predecessor
        appended to), the step's feeds ``page_table`` / ``kv_len`` / ``cache_loc`` / ``next_cos_sin`` and the
        successor's pools ``next_k`` / ``next_v``, and the exchange buffers one rank's layers share (``ar``, ``z``,
        ``z_sf``, ``z_ex``, ``zb``: byte tensors at least as large as this layer needs; ``pool_ag``, ``unpool_ag``,
        ``flags``), and ``status`` (one status block shared by the launches of a stack).
        ``tensor_cores``: bind the packed NVFP4 images when the shape has whole 128-row tiles (the tcgen05 expert
        kernels); otherwise, or when False, the experts run on the general CUDA-core kernels from the plain tensors.
        ``keep_plain_experts`` False drops the plain expert tensors once the images exist (halves the expert memory).
        ``expert_range`` (lo, hi): expert parallelism of a lone-rank shape (``MkLayerBind.expert_lo`` / ``expert_hi``):
        this object keeps and packs the experts [lo, hi) only and runs the routed slots that fall on them; the ranks of
        such a world share ``zb`` (``io``) and any one of them runs combine once all have run their experts."""
        cfg = case.cfg
        self.lib, self.case, self.rank, self.device = lib, case, rank, device
        self.shape = layer_shape(cfg, case, rank)
        self.consts = c = lib.layer_constants(self.shape)
        t = tensors if tensors is not None else case.ranks[rank]
        dev = lambda x: None if x is None else x.to(device).contiguous()  # noqa: E731
        io = dict(io or {})
        skip = set(io) | ({"k_ctx", "v_ctx"} if "k_cache" in io else set())
        self.expert_lo, self.expert_hi = expert_range or (0, 0)
        per_expert = lambda k, v: v if v is None or not self.expert_hi or k not in EXPERT_FIELDS else v[self.expert_lo : self.expert_hi]  # noqa: E731
        self.w = {k: (None if k in skip else dev(per_expert(k, v))) for k, v in vars(t).items()}
        for k in ("qkv_in", "stream_in", "next_cos_sin"):
            if k in io:
                self.w[k] = io[k]
        M, H, P, E, K = case.rows, cfg.hidden, cfg.moe_hidden, cfg.experts, cfg.topk
        whole_tiles = (cfg.inter_rank % 128 == 0 and cfg.moe_hidden_rank % 128 == 0 and P % 256 == 0
                       and cfg.moe_inter % 256 == 0 and P <= 4096 and cfg.moe_inter <= 4096)  # fmt: skip
        self.tensor_cores = bool(tensor_cores and not case.bf16 and whole_tiles)
        # a bf16 layer's experts as a grouped GEMM on the tensor-core dense pipeline (one tile image per expert)
        self.tensor_cores_bf16 = bool(tensor_cores and case.bf16 and cfg.inter_rank % 64 == 0 and cfg.moe_hidden_rank % 128 == 0
                                      and P % 128 == 0 and cfg.moe_inter % 128 == 0 and self.w["gate"] is not None)  # fmt: skip
        self.w1_pack = self.w2_pack = None
        if self.tensor_cores_bf16:
            w = self.w
            self.w1_pack, self.w2_pack = weights.pack_bf16_experts(w["gate"], w["up"], w["w2"])
            if not keep_plain_experts:
                for k in ("gate", "up", "w2"):
                    w[k] = None
        if self.tensor_cores:
            w = self.w
            self.w1_pack = weights.pack_w1_fp4(w["gate_q"], w["gate_sf"], w["up_q"], w["up_sf"])
            self.w2_pack = weights.pack_w2_fp4(w["w2_q"], w["w2_sf"])
            if not keep_plain_experts:
                for k in ("gate_q", "gate_sf", "up_q", "up_sf", "w2_q", "w2_sf"):
                    w[k] = None
        # the dense weights in the layout of the dense engine (``MkLayerBind.dense_packed``): 2 (the default where every K is
        # a multiple of 128) the tile images of the tensor-core engine, 1 / True the item images of the mma.sync item
        # engine, 0 / False row-major (item engine with one copy per weight row, or the cluster split-K GEMMs with
        # ``bind(fused=2)``). Packed forms keep this rank's node block of the pooler and the unpooler only.
        tiles_ok = cfg.oproj_k % 128 == 0 and H % 128 == 0 and P % 128 == 0
        self.packed = (2 if tiles_ok else 0) if packed is None else int(packed)
        if self.packed:
            w, nr = self.w, cfg.node_ranks
            j = rank % nr
            pk = lambda t: weights.pack_dense(t, self.packed)  # noqa: E731
            w["o_proj"] = pk(w["o_proj"])
            w["pooler"] = pk(w["pooler"][j * (P // nr) : (j + 1) * (P // nr)])
            w["router"] = pk(w["router"])
            w["unpooler"] = pk(w["unpooler"][j * (H // nr) : (j + 1) * (H // nr)])
            if w.get("next_qkv") is not None:
                w["next_qkv"] = pk(w["next_qkv"])
        bf, f32, u8, i32 = torch.bfloat16, torch.float32, torch.uint8, torch.int32

        def z(shape, dtype):
            return torch.zeros(shape, dtype=dtype, device=device)

        def raw(nbytes):
            return z((int(nbytes),), u8)

        # KV pools of this layer (context rows then the window's rows, identity slots) and of the successor
        kv_rows = kv_rows or (case.ctx + M + 127) // 128 * 128
        kvw = cfg.kv_heads_rank * cfg.head_dim
        if "k_cache" in io:
            self.k_cache, self.v_cache = io["k_cache"], io["v_cache"]
            kv_rows = self.k_cache.shape[0]
        else:
            self.k_cache, self.v_cache = z((kv_rows, kvw), bf), z((kv_rows, kvw), bf)
            self.k_cache[: case.ctx] = self.w["k_ctx"].reshape(case.ctx, kvw)
            self.v_cache[: case.ctx] = self.w["v_ctx"].reshape(case.ctx, kvw)
            if "qkv_in" not in io:
                qo, ko = cfg.q_heads_rank * 64, (cfg.q_heads_rank + cfg.kv_heads_rank) * 64
                self.k_cache[case.ctx : case.ctx + M] = self.w["qkv_in"][:, qo:ko]
                self.v_cache[case.ctx : case.ctx + M] = self.w["qkv_in"][:, ko : ko + kvw]
        if "next_k" in io:
            self.next_k, self.next_v = io["next_k"], io["next_v"]
        else:
            self.next_k, self.next_v = z((kv_rows, kvw), bf), z((kv_rows, kvw), bf)
        self.next_kv_rows = self.next_k.shape[0]
        self.page_table = io.get("page_table")
        if self.page_table is None:
            self.page_table = torch.arange(kv_rows, dtype=torch.int64, device=device) * c.kv_row_bytes
        self.kv_len = io.get("kv_len")
        if self.kv_len is None:
            self.kv_len = torch.tensor([case.ctx + M], dtype=i32, device=device)
        self.cache_loc = io.get("cache_loc")
        if self.cache_loc is None:
            self.cache_loc = torch.arange(case.ctx, case.ctx + M, dtype=i32, device=device)
        self.kv_rows = kv_rows
        # outputs
        self.o = dict(
            x_attn=z((M, cfg.q_heads_rank * 64), bf), branch=z((M, H), bf), stream_mid=z((M, H), f32), h3=z((M, H), bf),
            h3f=z((M, H), f32), logits=z((M, E), f32), ids=z((M, K), i32), w=z((M, K), f32),
            xq=z((M, P), bf) if case.bf16 else z((M, P // 2), u8), x_sf=z((M, P // 16), u8), x_scale=z((M,), f32),
            y=z((M, P), bf), stream_out=z((M, H), f32), h3_next=z((M, H), bf), qkv_next=z((M, c.qkv_row), bf),
        )  # fmt: skip
        # exchange buffers (symmetric across the ranks)
        def shared(name, nbytes):
            return io[name][: int(nbytes)] if name in io else raw(nbytes)

        self.ar = shared("ar", c.ar_bytes)
        self.pool_ag = io["pool_ag"] if "pool_ag" in io else z((M, P), bf)
        self.unpool_ag = io["unpool_ag"] if "unpool_ag" in io else z((M, H), bf)
        # a stack keeps the bf16 layers' h rows apart from the NVFP4 layers' code planes ("z16"): a column band that an
        # absent rank never writes then stays zero in both, instead of holding the other kind's bytes
        self.z_name = "z16" if case.bf16 and "z16" in io else "z"
        self.z, self.z_sf = shared(self.z_name, c.z_bytes), shared("z_sf", c.z_sf_bytes)
        self.z16 = self.z
        self.z_ex, self.zb = shared("z_ex", c.z_ex_bytes), shared("zb", c.zb_bytes)
        self.flags = io["flags"] if "flags" in io else z((c.flag_words,), i32)
        self.ws = raw(c.ws_bytes)
        self.status = io["status"] if "status" in io else raw(c.status_bytes)
        self.module = module
        self.launch_record = None

    def bind(self, peers: Optional[list] = None, b_live: int = 0, wait_budget: int = 0, fused: Optional[bool] = None,
             ep_peers: Optional[list] = None, ep_rank: int = 0, tree: Optional[torch.Tensor] = None, packets: bool = False):
        """Binds the launch; ``peers`` = per rank an object whose attributes ``ar``, ``pool_ag``, ``unpool_ag``, ``z``,
        ``z_sf``, ``z_ex``, ``zb``, ``flags`` are that rank's exchange buffers (tensors, or device addresses of buffers
        mapped from another process): every rank's ``LayerRank`` (own included), or None for a lone rank.
        ``fused``: the form of the dense stages (``MkLayerBind.fused``): 0 / False / None = one launch per stage with
        the GEMMs on the engine the weights are packed for (13 kernels a layer), 1 / True = two persistent kernels around the
        experts (7 kernels a layer): on tile images (``packed`` 2) the fused tensor-core kernels, on ``packed`` 0 or 1 the
        segment kernels of the item engine (
        measured slower on the full shape, and never for peers launched one after the other on one GPU: its exchange
        waits poll for ranks that run at the same time), 2 = one launch per stage with the cluster split-K GEMMs (14).
        ``ep_peers`` / ``ep_rank``: an expert-parallel world of one process per GPU (``expert_range`` given): per rank an
        object with ``zb`` and ``flags`` (this rank's own entry may be None); g2 writes its zb rows into every rank's zb
        and the combine waits for all ranks. ``tree``: the token tree's table (``dflash/tree.py``): the attention masks
        the window's own keys by the rows' ancestor masks and places the rows by depth.
        ``packets``: the four bf16 exchanges carry their own validity (``MkLayerBind.packets``): this rank's ``ar``,
        ``pool_ag``, ``zb`` and ``unpool_ag`` are filled with the "not arrived" mark here, the consumers put it back after
        every use, so these four read as marks after a launch (``values()`` of such a rank has no pooled / zb rows). The
        router's f32 logits travel the same way inside the rank (marked, polled by the routing rows, wiped), and the
        consuming row kernels do not wait for the producing grid to end: they start on the rows as they arrive."""
        fused = int(fused or 0)
        if packets:
            if fused == 1:
                raise RuntimeError("packets is not available with the fused form")
            for t in (self.ar, self.pool_ag, self.zb, self.unpool_ag, self.o["logits"]):
                t.view(torch.uint8).fill_(0xFF)
        if fused == 2 and self.packed == 2:
            raise RuntimeError("dense_packed 2 (tile images) has no cluster split-K form: build the rank with packed=0 for fused=2")
        cfg, case, w, o = self.case.cfg, self.case, self.w, self.o
        n = cfg.tp

        def peer(attr):
            if peers is None:
                return [getattr(self, attr) if r == self.rank else None for r in range(n)]
            return [getattr(p, attr) if p is not None else None for p in peers]

        fp4 = not case.bf16
        zb_peer, flags_peer, ep_world = peer("zb"), peer("flags"), 0
        if ep_peers is not None:
            assert self.expert_hi and peers is None, "an expert-parallel world binds a lone-rank shape with an expert range"
            ep_world = len(ep_peers)
            zb_peer = [self.zb if r == ep_rank else getattr(ep_peers[r], "zb") for r in range(ep_world)]
            flags_peer = [self.flags if r == ep_rank else getattr(ep_peers[r], "flags") for r in range(ep_world)]

        def ex(t):
            """A per-expert array's address as the kernels index it (by the global expert id)."""
            if t is None or not self.expert_hi:
                return t
            return t.data_ptr() - self.expert_lo * t[0].numel() * t.element_size()

        bind = host.make(
            "MkLayerBind",
            qkv_in=w["qkv_in"], k_cache=self.k_cache, v_cache=self.v_cache, kv_rows=self.kv_rows,
            page_table=self.page_table, kv_len=self.kv_len, page_stride=self.page_table.numel(), x_attn=o["x_attn"],
            w_o=w["o_proj"], ar=self.ar, ar_peer=peer("ar"), branch=o["branch"], stream_in=w["stream_in"],
            alpha=w["post_alpha"], beta=w["post_beta"], prenorm_w=w["post_pre_w"], stream_out=o["stream_mid"],
            h3=o["h3"], h3f=o["h3f"], w_p=w["pooler"], pool_ag=self.pool_ag, pool_ag_peer=peer("pool_ag"),
            w_r=w["router"], logits=o["logits"], router_mult=case.router_mult, expert_bias=w["expert_bias"],
            topk_idx32=o["ids"], topk_w=o["w"], route_scale=cfg.route_scale, gamma=w["pre_gamma"], eps=case.pre_eps,
            q=o["xq"], sf=o["x_sf"], x_scale=o["x_scale"],
            w1_gate=ex(w["gate_q"] if fp4 else w["gate"]), w1_gate_sf=ex(w["gate_sf"]),
            w1_up=ex(w["up_q"] if fp4 else w["up"]), w1_up_sf=ex(w["up_sf"]), w2=ex(w["w2_q"] if fp4 else w["w2"]),
            w2_sf=ex(w["w2_sf"]), w1_pack=ex(self.w1_pack), w2_pack=ex(self.w2_pack), g1_alphas=ex(w["g1_alphas"]),
            g1_scale_c=ex(w["g1_scale_c"]), g2_alphas=ex(w["g2_alphas"]), z=self.z, z_sf=self.z_sf, z_ex=self.z_ex, zb=self.zb,
            z_peer=peer(self.z_name), zsf_peer=peer("z_sf"), zex_peer=peer("z_ex"), zb_peer=zb_peer,
            gamma_p1=w["gamma_p1"], y=o["y"], w_up=w["unpooler"], unpool_ag=self.unpool_ag,
            unpool_ag_peer=peer("unpool_ag"), c_alpha=w["cross_alpha"], c_beta=w["cross_beta"], c_pre_w=w["cross_pre_w"],
            c_post_w=w["cross_post_w"], c_stream_out=o["stream_out"], h3q=o["h3_next"], w_qkv=w["next_qkv"],
            qkv_out=o["qkv_next"], cos_sin=w["next_cos_sin"], cache_loc=self.cache_loc, next_k_cache=self.next_k,
            next_v_cache=self.next_v, next_kv_rows=self.next_kv_rows, q_scale=cfg.q_scale, qkv_eps=cfg.rms_eps,
            flags=self.flags, flags_peer=flags_peer, ws=self.ws, status=self.status, b_live=b_live, wait_budget=wait_budget, fused=fused, dense_packed=int(self.packed),
            expert_lo=self.expert_lo, expert_hi=self.expert_hi, ep_rank=ep_rank if ep_world else 0, ep_world=ep_world, tree=tree, packets=int(packets),
        )  # fmt: skip
        self.launch_record = self.lib.layer_bind(self.module, self.shape, bind)
        return self.launch_record

    def launch(self, stream: int, pdl: bool = False) -> None:
        self.launch_record(stream, pdl)

    # ---- gathered views (what the oracle calls pooled / zb / ffn_out / the h planes) ----
    def values(self) -> dict:
        """The layer's named values as the oracle names them (device tensors)."""
        cfg, case, c = self.case.cfg, self.case, self.consts
        M, K, P, I = case.rows, cfg.topk, cfg.moe_hidden, cfg.moe_inter
        out = dict(self.o)
        out["pooled"] = self.pool_ag
        out["ffn_out"] = self.unpool_ag
        out["zb"] = self.zb.view(torch.bfloat16).view(M, K, P)
        if case.bf16:
            out["x"] = out.pop("xq")
            out.pop("x_sf"), out.pop("x_scale")
        if case.tail:
            out.pop("qkv_next")
        out.pop("h3f")
        return out

    def h_planes(self):
        cfg, case = self.case.cfg, self.case
        M, K, I = case.rows, cfg.topk, cfg.moe_inter
        return (
            self.z.view(M, K, I // 2),
            self.z_sf.view(M, K, I // 16),
            self.z_ex.view(torch.int8).view(M, K, I // 16).to(torch.int32),
        )


class LayerWorld:
    """Every rank of the world on one device, exchange buffers wired as peers (see the module docstring)."""

    def __init__(self, case, device, lib: Optional[host.Library] = None, ranks: Optional[list] = None, b_live: int = 0,
                 tensor_cores: bool = True, packed: Optional[int] = None):  # fmt: skip
        self.lib = lib or host.library()
        self.case, self.device = case, device
        with torch.cuda.device(device):
            self.module = self.lib.load()
        n = case.cfg.tp
        self.ranks = [LayerRank(self.lib, self.module, case, r, device, tensor_cores=tensor_cores, packed=packed) for r in range(n)]
        for r in self.ranks:
            r.bind(self.ranks, b_live)

    def run_interleaved(self, stream: Optional[int] = None) -> None:
        """All ranks, stage group by stage group: every exchange sees every rank's contribution."""
        s = torch.cuda.current_stream(self.device).cuda_stream if stream is None else stream
        for first, count in STAGE_GROUPS:
            for r in self.ranks:
                r.launch_record.step(s, first, count)
