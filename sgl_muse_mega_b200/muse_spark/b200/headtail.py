"""The launches of a verify step that sit around the 62 decoder layers: window feeds, the fused entry, the lm_head
shard GEMM, the soft cap, and the greedy accept that closes a DFlash2 iteration.

Each class owns its outputs, binds once and launches on a stream, like the reference's ``Stack`` members
(``sm103/verify.py:120-160`` feeds, ``:400-433`` entry and qkv head, ``:436-470`` lm_head and soft cap) and its
``sm103/dflash/head.py`` accept. All of them are plain launches of the C-ABI library; none computes on the host.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from ...common import host

WORDS = {"P": 0, "ANCHOR": 1, "ACCEPT": 2, "COMMIT": 3, "ITER": 4, "OUT_COUNT": 5}
N_WORDS = 8


def _z(*shape, dtype, device):
    return torch.zeros(*shape, dtype=dtype, device=device)


class WindowFeeds:
    """The step's feeds from the serving framework's batch tensors (positions, out_cache_loc, seq_lens,
    req_pool_indices, req_to_token, full_to_swa): rope rows, int32 cache slots, kv_len and the position -> byte-offset
    tables."""

    def __init__(self, lib: host.Library, module, *, positions, cos_sin_cache, out_cache_loc, swa_out_cache_loc, seq_lens,
                 req_pool_indices, req_to_token, full_to_swa, kv_row_bytes: int):  # fmt: skip
        dev, rows = positions.device, positions.shape[0]
        hd = cos_sin_cache.shape[1]
        self.cos_sin = _z(rows, hd, dtype=torch.float32, device=dev)
        self.loc_full = _z(rows, dtype=torch.int32, device=dev)
        self.loc_swa = _z(rows, dtype=torch.int32, device=dev) if swa_out_cache_loc is not None else None
        self.kv_len = _z(1, dtype=torch.int32, device=dev)
        self.pt_full = _z(req_to_token.shape[1], dtype=torch.int64, device=dev)
        self.pt_swa = _z(req_to_token.shape[1], dtype=torch.int64, device=dev) if full_to_swa is not None else None
        self.status = _z(16, dtype=torch.int32, device=dev)
        self.keep = (positions, cos_sin_cache, out_cache_loc, swa_out_cache_loc, seq_lens, req_pool_indices, req_to_token,
                     full_to_swa)  # fmt: skip
        self.bind = host.make(
            "MkFeedsBind", positions=positions, cos_sin_cache=cos_sin_cache, cos_sin_rows=cos_sin_cache.shape[0],
            out_cache_loc=out_cache_loc, swa_out_cache_loc=swa_out_cache_loc, seq_lens=seq_lens,
            req_pool_indices=req_pool_indices, req_to_token=req_to_token, r2t_rows=req_to_token.shape[0],
            r2t_width=req_to_token.shape[1], full_to_swa=full_to_swa,
            swa_map_len=0 if full_to_swa is None else full_to_swa.shape[0], cos_sin=self.cos_sin, loc_full=self.loc_full,
            loc_swa=self.loc_swa, kv_len=self.kv_len, pt_full=self.pt_full, pt_swa=self.pt_swa, rows=rows, head_dim=hd,
            kv_row_bytes=kv_row_bytes, status=self.status,
        )  # fmt: skip
        self.launch = lib.bind("mk_feeds_bind", module, self.bind)


class Entry:
    """ids -> residual (f32) and layer 0's normed input (bf16); ``embed_shards`` are every rank's vocab rows (this
    rank's own tensor and its peers' mapped buffers)."""

    def __init__(self, lib: host.Library, module, *, ids, embed_shards: Sequence, pre_w, eps_embed: float = 1e-5,
                 eps_pre: float = 1e-5, shard_rows: Optional[int] = None, hidden: Optional[int] = None,
                 residual=None, normed=None):  # fmt: skip
        """``embed_shards``: tensors, or device addresses (then ``shard_rows`` and ``hidden`` say their shape).
        ``residual`` / ``normed``: the outputs, when the caller has already bound other launches to them."""
        dev, rows = ids.device, ids.shape[0]
        if shard_rows is None:
            shard_rows, hidden = embed_shards[0].shape
        self.residual = residual if residual is not None else _z(rows, hidden, dtype=torch.float32, device=dev)
        self.normed = normed if normed is not None else _z(rows, hidden, dtype=torch.bfloat16, device=dev)
        self.keep = (ids, list(embed_shards), pre_w)
        self.bind = host.make(
            "MkEntryBind", ids=ids, embed_peer=list(embed_shards), shard_rows=shard_rows, ranks=len(embed_shards),
            pre_w=pre_w, residual=self.residual, normed=self.normed, rows=rows, hidden=hidden, eps_embed=eps_embed,
            eps_pre=eps_pre,
        )  # fmt: skip
        self.launch = lib.bind("mk_entry_bind", module, self.bind)


class LmHead:
    """One rank's vocab shard against the final hidden rows, f32, stored at column ``rank * n_out`` of every rank's
    gathered logits (``gathered[r]`` is rank r's [rows, v_total] buffer; absent ranks are None)."""

    def __init__(self, lib: host.Library, module, *, w, x, gathered: Sequence[Optional[torch.Tensor]], rank: int,
                 flags=None, flags_peer: Sequence = (), v_total: Optional[int] = None, engine: bool = True,
                 w_packed: int = 0, n_out: Optional[int] = None, hidden: Optional[int] = None):  # fmt: skip
        """``gathered``: tensors, or device addresses (then ``v_total`` is their row length). ``flags`` /
        ``flags_peer``: this rank's flag block and the peers' (present exactly where ``gathered`` is): the GEMM then
        signals the logits exchange on every rank it stored to."""
        w_packed = int(w_packed)
        if w_packed:  # item images (1, weights.pack_items) or tile images (2, weights.pack_umma): the shape comes from the caller
            assert n_out is not None and hidden is not None and engine
        else:
            n_out, hidden = w.shape
        if v_total is None:
            v_total = gathered[rank].shape[1]
        self.status = _z(16, dtype=torch.int32, device=x.device)
        # private scratch of the item engine (partial sums per 512-k chunk and its barrier word); shapes it does not tile
        # run on the cluster split-K GEMM without scratch
        ws_bytes = (hidden // 256) * 16 * n_out * 4 + 512 if engine and hidden % 512 == 0 else 0
        if w_packed == 2:  # the tensor-core engine: stream-K partial sums and one ticket per 128-row tile
            tiles = (n_out + 127) // 128
            ws_bytes = max(ws_bytes, (2 * 148 + 2 * tiles) * 2048 * 4 + (tiles * 4 + 255) // 256 * 256 + 512)
        self.ws = _z(ws_bytes, dtype=torch.uint8, device=x.device) if ws_bytes else None
        self.keep = (w, x, list(gathered))
        self.bind = host.make(
            "MkLmHeadBind", w=w, x=x, out_peer=list(gathered), rank=rank, v_total=v_total, col0=rank * n_out,
            n_out=n_out, hidden=hidden, rows=x.shape[0], status=self.status, flags=flags, flags_peer=list(flags_peer),
            ws=self.ws, ws_bytes=ws_bytes, w_packed=int(w_packed),
        )  # fmt: skip
        self.launch = lib.bind("mk_lm_head_bind", module, self.bind)


class Softcap:
    """cap tanh(x scale / cap) over the gathered logits, into ``out`` (the serving framework's logits tensor)."""

    def __init__(self, lib: host.Library, module, *, x, out, scale: float, cap: float, flags=None, contributors: int = 0,
                 wait_budget: int = 0):  # fmt: skip
        self.status = _z(16, dtype=torch.int32, device=x.device)
        self.keep = (x, out, flags)
        self.bind = host.make("MkSoftcapBind", x=x, out=out, numel=x.numel(), scale=scale, cap=cap, flags=flags,
                              contributors=contributors, wait_budget=wait_budget, status=self.status)  # fmt: skip
        self.launch = lib.bind("mk_softcap_bind", module, self.bind)


class Accept:
    """The greedy accept over the gathered (pre-cap) logits. Owns the step words, the committed-token ring and the
    per-row arg-max; writes the next iteration's target feeds into ``feeds`` (cos_sin, loc_full, loc_swa, kv_len: the
    buffers the layers were bound to) and the draft feeds it allocates when ``dcos_sin_cache`` is given."""

    def __init__(self, lib: host.Library, module, *, logits, tokens, b_live: int, scale: float, cap: float, ring: int = 64,
                 accept_override: Optional[torch.Tensor] = None, cos_sin_cache=None, cos_sin=None, loc_full=None,
                 loc_swa=None, kv_len=None, dcos_sin_cache=None, dring: int = 0, flags=None, contributors: int = 0,
                 wait_budget: int = 0, pool_rows: int = 0, samp=None, cand=None, walk_q=None, block_verify: bool = True,
                 share: Optional["Accept"] = None, tree: Optional[torch.Tensor] = None):  # fmt: skip
        """``samp`` (the sampling words on the device, ``dflash.draft.sampling_words``) with the draft head's ``cand`` and
        ``walk_q`` binds the sampled accept instead of the greedy one (``sample_out``: the residual's scale and mass).
        ``share``: another accept of the same step (the greedy one beside the sampled one) whose step words, token ring,
        counter and draft feeds this one advances too: a request may then alternate between the two launches.
        ``tree``: the token tree's table (``dflash/tree.py`` ``TreeWalk.table``): the greedy accept then follows the
        tree's matching path instead of the chain's prefix and leaves the path in the table."""
        dev = logits.device
        rows, vocab = logits.shape
        self.sample_ws = self.sample_out = None
        if samp is not None:
            ys = (rows * vocab * 4 + 255) // 256 * 256
            self.sample_ws = _z(ys + rows * vocab * 8 + 256, dtype=torch.uint8, device=dev)
            self.sample_out = _z(16, dtype=torch.float64, device=dev)  # [0:2] scale, mass; the rest: trace builds
        draft = dcos_sin_cache is not None
        if share is not None:
            assert share.out_ring.numel() == ring, "accepts that share their state have one token ring"
            self.words, self.out_ring, self.top1, self.counter = share.words, share.out_ring, share.top1, share.counter
            self.dcos_sin, self.dslot, self.dkv_len = share.dcos_sin, share.dslot, share.dkv_len
        else:
            self.words = _z(N_WORDS, dtype=torch.int64, device=dev)
            self.out_ring = _z(ring, dtype=torch.int32, device=dev)
            self.top1 = _z(rows, dtype=torch.int32, device=dev)
            self.counter = _z(512, dtype=torch.int32, device=dev)  # arrival counters and the row chunks' winners
            self.dcos_sin = _z(2 * b_live, 128, dtype=torch.float32, device=dev) if draft else None
            self.dslot = _z(2 * b_live, dtype=torch.int32, device=dev) if draft else None
            self.dkv_len = _z(1, dtype=torch.int32, device=dev) if draft else None
        self.status = _z(16, dtype=torch.int32, device=dev)
        self.keep = (logits, tokens, accept_override, cos_sin_cache, cos_sin, loc_full, loc_swa, kv_len, dcos_sin_cache, samp, cand, walk_q)
        self.bind = host.make(
            "MkAcceptBind", logits=logits, vocab=vocab, rows=rows, b_live=b_live, scale=scale, cap=cap, tokens=tokens,
            accept_override=accept_override, n_override=0 if accept_override is None else accept_override.numel(),
            words=self.words, out_ring=self.out_ring, ring=ring, top1=self.top1, counter=self.counter,
            cos_sin_cache=cos_sin_cache, cos_sin_rows=0 if cos_sin_cache is None else cos_sin_cache.shape[0],
            cos_sin=cos_sin, loc_full=loc_full, loc_swa=loc_swa, kv_len=kv_len, dcos_sin_cache=dcos_sin_cache,
            dcos_sin_rows=0 if dcos_sin_cache is None else dcos_sin_cache.shape[0], dcos_sin=self.dcos_sin,
            dslot=self.dslot, dkv_len=self.dkv_len, dring=dring, flags=flags, contributors=contributors,
            wait_budget=wait_budget, status=self.status, pool_rows=pool_rows, samp=samp, cand=cand, walk_q=walk_q,
            block_verify=int(block_verify), sample_ws=self.sample_ws,
            sample_ws_bytes=0 if self.sample_ws is None else self.sample_ws.numel(), sample_out=self.sample_out, tree=tree,
        )  # fmt: skip
        self.launch = lib.bind("mk_accept_bind", module, self.bind)
