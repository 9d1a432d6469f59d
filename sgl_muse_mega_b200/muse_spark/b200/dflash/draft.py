"""One rank's DFlash2 draft step on the device: buffers, bind-once launch records, the launch list.

Mirrors the reference's ``sm103/dflash/iteration.py`` (``Iteration.launches`` :670-684: draft_entry, draft_qkv, the draft
layers, draft_head) and ``sm103/dflash/head.py`` / ``layer.py`` binds with this library's entry points::

    mk_dflash_entry_bind        feats, fc (gathered), ctx norm, context k / v rows, their head norm + RoPE into the pools,
                                the block's embedding rows + layer 0's input norm                              6 kernels
    mk_dflash_layer_bind x L    conv, qkv, attention, o_proj + all-reduce, conv, SwiGLU MLP + all-reduce       10 kernels
    mk_lm_head_bind             the target lm_head over y rows 1.., f32 logits gathered on every rank           1 kernel
    mk_dflash_draft_head_bind   W_P y, top-16, lattice, walk, the verify window's ids                           3 kernels

The step is driven by the step words on the device (position, anchor, last commit): a CUDA graph of the list replays
without host input. ``DraftWorld`` holds every rank of a world on one device (the tests' form: launches interleaved kernel
by kernel, the stream orders the exchanges); with one process per GPU the exchange buffers sit in a shared arena and the
kernels signal through the draft's flag block.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from ....common import host
from .. import headtail as HT
from .. import weights as W
from .weights import DraftConfig, DraftWeights, TargetShared, rope_table

BF = torch.bfloat16


def shape_of(cfg: DraftConfig, ranks: int, rank: int, rows: int):
    return host.make(
        "MkDflashShape", rows=rows, hidden=cfg.hidden, layers=cfg.layers, q_heads=cfg.q_rank(ranks), kv_heads=cfg.kv_rank(ranks),
        inter=cfg.inter // ranks, features=cfg.features, ranks=ranks, rank=rank, window_left=cfg.window_left,
        conv_groups=cfg.conv_groups, vocab=cfg.vocab, selector_rank=cfg.selector_rank,
    )  # fmt: skip


class Exchange:
    """The buffers a rank's peers write into: gathered fc rows, the two all-reduce workspaces, the gathered draft logits,
    plus its vocab shard of the embedding and its flag block. Tensors here; a peer process passes the same names as device
    addresses (any object with these attributes serves)."""

    def __init__(self, cfg: DraftConfig, ranks: int, rows: int, device, embed: torch.Tensor, flags: bool):
        z = lambda *s, dt=BF: torch.zeros(*s, dtype=dt, device=device)  # noqa: E731
        self.ctx_raw = z(rows, cfg.hidden)
        self.ar_attn = z(ranks, 16, cfg.hidden)
        self.ar_mlp = z(ranks, 16, cfg.hidden)
        self.gathered = z(rows - 1, cfg.vocab, dt=torch.float32)
        self.embed = embed
        self.flags = z(32, dt=torch.int32) if flags else None


class DraftRank:
    def __init__(self, cfg: DraftConfig, w: DraftWeights, t: TargetShared, rank: int, ranks: int, device, *, rows: int,
                 pool_rows: int, rope_rows: int, lib: Optional[host.Library] = None, module=None, words: Optional[torch.Tensor] = None,
                 caps: Optional[Sequence[torch.Tensor]] = None, verify_ids: Optional[torch.Tensor] = None, exchange=None,
                 flags: bool = False, wait_budget: int = 0, packed: Optional[int] = None, lm_head_packed: Optional[int] = None,
                 samp: Optional[torch.Tensor] = None, cand: Optional[torch.Tensor] = None,
                 walk_q: Optional[torch.Tensor] = None, sample_too: bool = False):  # fmt: skip
        """``samp`` (the sampling words on the device) selects the sampled walk; ``cand`` / ``walk_q``: buffers a sampled
        accept was bound to (default: allocated here). ``sample_too``: the greedy head stays bound beside the sampled one
        (``launch_all(sample=False)`` runs it), for a server that takes greedy and sampled requests.
        ``packed``: the layout the draft's GEMM weights are uploaded in (``weights.pack_dense``): 2 tile images for the
        tensor-core engine (the default where the shapes tile), 1 / True item images, 0 / False row-major.
        ``lm_head_packed``: the layout ``t.lm_head`` already has (a target stack's packed lm_head); default: packed here."""
        self.cfg, self.rank, self.ranks, self.rows, self.device = cfg, rank, ranks, rows, device
        tiles_ok = cfg.conv_groups % 32 == 0 and (cfg.inter // ranks) % 64 == 0 and cfg.hidden % 128 == 0
        self.packed = (2 if tiles_ok else 0) if packed is None else int(packed)
        pk = lambda x, perm=None: W.pack_dense(x, self.packed, perm)  # noqa: E731
        self.lm_head_packed = int(lm_head_packed or 0) or self.packed
        self.lib = lib or host.library()
        self.module = module or self.lib.load()
        self.shape = shape_of(cfg, ranks, rank, rows)
        self.consts = self.lib.dflash_constants(self.shape)
        self.pool_rows, self.rope_rows, self.wait_budget = pool_rows, rope_rows, wait_budget
        dev = device
        z = lambda *s, dt=BF: torch.zeros(*s, dtype=dt, device=dev)  # noqa: E731
        d = lambda x: x.to(dev).contiguous()  # noqa: E731
        H, c, gamma = cfg.hidden, self.consts, rows - 1
        kvh, qh = cfg.kv_rank(ranks), cfg.q_rank(ranks)
        # weights
        self.w = dict(
            fc=pk(d(w.fc)), hid_norm=d(w.hidden_norm), norm=d(w.norm), pred=d(w.pred_codebook), succ=d(w.succ_codebook),
            hproj=pk(d(w.hidden_proj)),
            lm_head=d(t.lm_head) if lm_head_packed else pk(d(t.lm_head)),
            w_kv=pk(d(torch.cat([lw.qkv[qh * cfg.head_dim :] for lw in w.layers]))),
        )  # fmt: skip
        self.lw = [
            dict(in_norm=d(lw.input_norm), post_norm=d(lw.post_norm), q_norm=d(lw.q_norm), k_norm=d(lw.k_norm), qkv=pk(d(lw.qkv)),
                 o=pk(d(lw.o)), gate_up=pk(d(lw.gate_up), W.silu_perm(cfg.inter // ranks)), down=pk(d(lw.down)),
                 attn_proj=pk(d(lw.attn_conv.proj), W.conv_perm(cfg.conv_groups)), attn_base=d(lw.attn_conv.base),
                 mlp_proj=pk(d(lw.mlp_conv.proj), W.conv_perm(cfg.conv_groups)), mlp_base=d(lw.mlp_conv.base))
            for lw in w.layers
        ]  # fmt: skip
        self.rope = d(rope_table(rope_rows, cfg.head_dim, cfg.rope_theta))
        # state and pools
        self.words = words if words is not None else z(8, dt=torch.int64)
        self.caps = list(caps) if caps is not None else [z(rows, H, dt=torch.float32) for _ in range(cfg.features)]
        self.k_pool = [z(pool_rows, kvh, cfg.head_dim) for _ in range(cfg.layers)]
        self.v_pool = [z(pool_rows, kvh, cfg.head_dim) for _ in range(cfg.layers)]
        self.x = exchange or Exchange(cfg, ranks, rows, dev, d(t.embed), flags)
        # private buffers
        self.ws = torch.zeros(c.ws_bytes, dtype=torch.uint8, device=dev)
        self.feats, self.ctx, self.kv = z(rows, cfg.features * H), z(rows, H), z(rows, c.kv_rows_n)
        self.emb = z(rows, H)
        self.h = [z(rows, H) for _ in range(cfg.layers + 1)]  # h[l]: layer l's normed input; h[L] = y
        self.res = [self.emb] + [z(rows, H) for _ in range(cfg.layers - 1)]
        self.f = dict(c_att=z(rows, c.coeffs), xa=z(rows, H), qkv=z(rows, c.qkv_row), q=z(rows, qh * cfg.head_dim),
                      attn_ws=torch.zeros(c.attn_ws_bytes // 4, dtype=torch.float32, device=dev), o=z(rows, qh * cfg.head_dim),
                      a=z(rows, H), h_post=z(rows, H), res_post=z(rows, H), c_mlp=z(rows, c.coeffs), xm=z(rows, H),
                      m=z(rows, cfg.inter // ranks), x_out=z(rows, H))  # fmt: skip
        self.hid = z(gamma, cfg.selector_rank)
        self.keys = torch.zeros(gamma, c.topk_chunks + 1, 16, dtype=torch.int64, device=dev)
        self.cand = cand if cand is not None else torch.zeros(gamma, 16, dtype=torch.int64, device=dev)
        self.unary = z(gamma, 16, dt=torch.float32)
        self.scores = z(gamma, 16, 16, dt=torch.float32)
        self.pick = z(gamma, dt=torch.int32)
        self.drafts = z(gamma, dt=torch.int64)
        self.verify_ids = verify_ids if verify_ids is not None else z(rows, dt=torch.int64)
        self.samp = samp  # i64 [4] sampling words on the device (``sampling_words``), or None: the greedy walk
        self.sample_too = sample_too and samp is not None
        self.walk_q = walk_q if walk_q is not None else z(gamma, 16, dt=torch.float32)
        self.status = z(16, dt=torch.int32)
        self.launches: list = []

    @property
    def y(self) -> torch.Tensor:
        return self.h[-1]

    def bind(self, peers: Optional[Sequence] = None) -> None:
        """``peers``: every rank's exchange (``Exchange`` or an object with the same attributes as tensors / addresses),
        None where a rank is absent; this rank's own entry may be None too."""
        cfg, lib, mod, r = self.cfg, self.lib, self.module, self.rank
        peers = list(peers) if peers is not None else [None] * self.ranks
        peers[r] = self.x
        of = lambda name: [None if p is None else getattr(p, name) for p in peers]  # noqa: E731
        flags = self.x.flags
        fpeer = of("flags") if flags is not None else []
        # a slice of a larger world (absent ranks): an id owned by an absent rank reads a present rank's shard instead, the
        # same one on every present rank (present rank number r mod present)
        shards = of("embed")
        here = [i for i, e in enumerate(shards) if e is not None]
        embed = [shards[here[i % len(here)]] if e is None else e for i, e in enumerate(shards)]
        common = dict(ws=self.ws, flags=flags, flags_peer=fpeer, status=self.status, wait_budget=self.wait_budget, eps=cfg.rms_eps,
                      packed=int(self.packed))
        entry = host.make(
            "MkDflashEntryBind", cap=self.caps, words=self.words, embed_peer=embed, shard_rows=cfg.vocab // self.ranks,
            mask_id=cfg.mask_id, w_fc=self.w["fc"], hid_norm=self.w["hid_norm"], in_norm=self.lw[0]["in_norm"], w_kv=self.w["w_kv"],
            k_norm=[l["k_norm"] for l in self.lw], k_pool=self.k_pool, v_pool=self.v_pool, pool_rows=self.pool_rows, rope=self.rope,
            rope_rows=self.rope_rows, feats=self.feats, ctx_raw_peer=of("ctx_raw"), ctx=self.ctx, kv=self.kv, x=self.emb, h=self.h[0],
            **common,
        )  # fmt: skip
        self.entry = lib.dflash_bind("mk_dflash_entry_bind", mod, self.shape, entry)
        self.layers = []
        f = self.f
        for li, l in enumerate(self.lw):
            last = li == cfg.layers - 1
            b = host.make(
                "MkDflashLayerBind", h_in=self.h[li], res_in=self.res[li], words=self.words, attn_proj=l["attn_proj"],
                attn_base=l["attn_base"], mlp_proj=l["mlp_proj"], mlp_base=l["mlp_base"], w_qkv=l["qkv"], q_norm=l["q_norm"],
                k_norm=l["k_norm"], w_o=l["o"], post_norm=l["post_norm"], w_gate_up=l["gate_up"], w_down=l["down"],
                next_norm=self.w["norm"] if last else self.lw[li + 1]["in_norm"], k_pool=self.k_pool[li], v_pool=self.v_pool[li],
                pool_rows=self.pool_rows, rope=self.rope, rope_rows=self.rope_rows, c_att=f["c_att"], xa=f["xa"], qkv=f["qkv"],
                q=f["q"], attn_ws=f["attn_ws"], o=f["o"], ar_attn_peer=of("ar_attn"), a=f["a"], h_post=f["h_post"],
                res_post=f["res_post"], c_mlp=f["c_mlp"], xm=f["xm"], m=f["m"], ar_mlp_peer=of("ar_mlp"), x_out=f["x_out"],
                h_out=self.h[li + 1], res_out=None if last else self.res[li + 1], **common,
            )  # fmt: skip
            self.layers.append(lib.dflash_bind("mk_dflash_layer_bind", mod, self.shape, b))
        present = sum(p is not None for p in peers)
        self.lm_head = HT.LmHead(lib, mod, w=self.w["lm_head"], x=self.y[1:], gathered=of("gathered"), rank=r, flags=flags,
                                 flags_peer=fpeer, v_total=cfg.vocab, w_packed=self.lm_head_packed, n_out=cfg.vocab // self.ranks,
                                 hidden=cfg.hidden)  # fmt: skip
        def head_bind(samp):
            return host.make(
                "MkDflashDraftHeadBind", y=self.y, w_hproj=self.w["hproj"], hid=self.hid, logits=self.x.gathered,
                pred_codebook=self.w["pred"], succ_codebook=self.w["succ"], words=self.words, keys=self.keys, cand=self.cand,
                unary=self.unary, scores=self.scores, pick=self.pick, drafts=self.drafts, verify_ids=self.verify_ids,
                mult=cfg.output_multiplier, cap=cfg.softcap, ws=self.ws, flags=flags, contributors=present if flags is not None else 0,
                status=self.status, wait_budget=self.wait_budget, packed=int(self.packed), samp=samp,
                walk_q=self.walk_q if samp is not None else None,
            )  # fmt: skip

        self.head = lib.dflash_bind("mk_dflash_draft_head_bind", mod, self.shape, head_bind(self.samp))
        self.launches = [self.entry, *self.layers, self.lm_head.launch, self.head]
        self.launches_greedy = self.launches
        if self.sample_too:
            self.head_greedy = lib.dflash_bind("mk_dflash_draft_head_bind", mod, self.shape, head_bind(None))
            self.launches_greedy = [*self.launches[:-1], self.head_greedy]

    def kernels(self) -> int:
        return sum(l.info().kernels for l in self.launches)

    def launch_all(self, s: int, pdl: bool = True, sample: Optional[bool] = None) -> None:
        """``sample`` False: the greedy walk of a rank bound with ``sample_too``; default: the walk the rank was built for."""
        for l in self.launches_greedy if sample is False else self.launches:
            l(s, pdl)

    def set_state(self, pos: int, anchor: int, commit: int, caps: Optional[torch.Tensor] = None) -> None:
        """The step words and, optionally, the captured residuals [features, rows, H] the step starts from."""
        w = torch.zeros(8, dtype=torch.int64)
        w[HT.WORDS["P"]], w[HT.WORDS["ANCHOR"]], w[HT.WORDS["COMMIT"]] = pos, anchor, commit
        self.words.copy_(w)
        if caps is not None:
            for dst, src in zip(self.caps, caps):
                dst.copy_(src)

    def load_history(self, k: Sequence[torch.Tensor], v: Sequence[torch.Tensor]) -> None:
        """Earlier positions' context rows, per layer [n, kv heads (whole model), D], into this rank's pools."""
        kvh = self.cfg.kv_rank(self.ranks)
        for li in range(self.cfg.layers):
            n = k[li].shape[0]
            self.k_pool[li][:n] = k[li][:, self.rank * kvh : (self.rank + 1) * kvh].to(self.device)
            self.v_pool[li][:n] = v[li][:, self.rank * kvh : (self.rank + 1) * kvh].to(self.device)

    def statuses(self) -> list:
        st = self.entry.status(torch.cuda.current_stream(self.device).cuda_stream)
        out = [("draft", st.code, st.stage, st.observed)] if st.code else []
        st = self.lm_head.launch.status(torch.cuda.current_stream(self.device).cuda_stream)
        return out + ([("draft_lm_head", st.code, st.stage, st.observed)] if st.code else [])


def sampling_words(seed: int, stream: int, temperature: float, top_k: int = 1 << 30, top_p: float = 1.0) -> torch.Tensor:
    """The sampled step's words (reference ``sm103/dflash/head.py:56-59``): seed, stream, top_k, f32 temperature bits |
    f32 top_p bits << 32, as i64 [4] on the host."""
    import struct

    t = struct.unpack("<I", struct.pack("<f", temperature))[0]
    p = struct.unpack("<I", struct.pack("<f", top_p))[0]
    seed &= 2**64 - 1
    return torch.tensor([seed - 2**64 if seed >= 2**63 else seed, stream, top_k, t | (p << 32)], dtype=torch.int64)


class DraftWorld:
    """Every rank of a draft case on one device; the launches run kernel by kernel across the ranks, so the stream orders
    each exchange (no flags)."""

    def __init__(self, case, device, lib: Optional[host.Library] = None, **kw):
        self.case, self.device = case, device
        lib = lib or host.library()
        mod = lib.load()
        cfg = case.cfg
        pool_rows = kw.pop("pool_rows", max(case.pos, cfg.window_left) + case.rows + 8)
        self.ranks = [
            DraftRank(cfg, w, t, r, case.ranks, device, rows=case.rows, pool_rows=pool_rows, rope_rows=pool_rows, lib=lib,
                      module=mod, **kw)
            for r, (w, t) in enumerate(case.shards)
        ]  # fmt: skip
        for dr in self.ranks:
            dr.bind([p.x for p in self.ranks])
            dr.set_state(case.pos, case.anchor, case.commit, case.caps)
            dr.load_history(case.hist_k, case.hist_v)

    def run_interleaved(self, after=None) -> None:
        """``after(launch index)`` is called when every rank has finished that launch (entry = 0, layer l = 1 + l, ...)."""
        s = torch.cuda.current_stream(self.device).cuda_stream
        for li in range(len(self.ranks[0].launches)):
            n = self.ranks[0].launches[li].info().kernels
            for k in range(n):
                for dr in self.ranks:
                    l = dr.launches[li]
                    if l.info().kernels == 1 and li == len(dr.launches) - 2:
                        l(s, False)  # the lm_head: a single-kernel record without stage addressing
                    else:
                        l.step(s, k, 1)
            if after is not None:
                after(li)


# ---- a world of one process per GPU -------------------------------------------------------------------------------------

EXCHANGE = ("flags", "ctx_raw", "ar_attn", "ar_mlp", "gathered")


def exchange_layout(cfg: DraftConfig, ranks: int, rows: int, with_embed: bool = False):
    """The draft's exchange arena of one rank (depends on the model and the block only: every rank carves the same).
    ``with_embed``: room for the rank's vocab shard of the embedding too (a draft that runs without a target stack, whose
    arena otherwise holds it)."""
    from ....common import symm

    lay = symm.Layout()
    lay.add("flags", (64,), torch.int32)
    lay.add("ctx_raw", (rows, cfg.hidden), BF)
    lay.add("ar_attn", (ranks, 16, cfg.hidden), BF)
    lay.add("ar_mlp", (ranks, 16, cfg.hidden), BF)
    lay.add("gathered", (rows - 1, cfg.vocab), torch.float32)
    if with_embed:
        lay.add("embed", (cfg.vocab // ranks, cfg.hidden), BF)
    return lay


class ArenaExchange:
    """This rank's exchange buffers inside its arena (tensors), plus its embedding shard (the target stack's)."""

    def __init__(self, arena, embed):
        self.arena, self.embed = arena, embed
        for name in EXCHANGE:
            setattr(self, name, arena.tensor(name))
        if "embed" in arena.layout.items:  # the shard moves into the arena, where the peers can read it
            self.embed = arena.tensor("embed")
            self.embed.copy_(embed)


class PeerExchange:
    """A peer's exchange buffers by device address (its arena, mapped) and the address of its embedding shard."""

    def __init__(self, arena, embed_ptr: Optional[int]):
        self.arena, self.embed = arena, embed_ptr if embed_ptr is not None else arena.ptr("embed")
        for name in EXCHANGE:
            setattr(self, name, arena.ptr(name))


def connect_exchange(arena, embed, peer_embed_ptrs: Optional[Sequence[Optional[int]]], rank: int, ranks: int, group=None) -> tuple:
    """Swaps the draft arenas' handles over ``torch.distributed`` -> (own ``ArenaExchange``, the peer list for
    ``DraftRank.bind``: own entry included, None for ranks beyond the present world)."""
    import torch.distributed as dist

    from ....common import symm

    n = dist.get_world_size(group)
    arenas = symm.connect(arena, rank, n, group)
    own = ArenaExchange(arena, embed)
    ptrs = peer_embed_ptrs if peer_embed_ptrs is not None else [None] * n
    peers = [own if i == rank else PeerExchange(a, ptrs[i]) for i, a in enumerate(arenas)] + [None] * (ranks - n)
    return own, peers
