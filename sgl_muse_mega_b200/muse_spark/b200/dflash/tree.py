"""The DFlash2 token tree's launches (``csrc/tree.cu``): the draft head's tree walk over its lattice and the compaction of the
accepted path's rows. Counterparts of the reference's tree variants of the draft head and ``mk_dflash_tree_compact``
(``kernels/dflash/tree.cuh``); the tree accept is ``headtail.Accept(tree=...)``.

``TreeWalk`` turns the lattice (candidates and pair scores of the draft head) into the verify window's rows as a tree:
``table`` (i32 [96]: parent, depth, ancestor mask, the accept's path, the window rows' pool slots) and ``verify_ids`` (the
rows' tokens in preorder). ``TreeCompact`` moves, after the accept, the accepted path's K / V and captured rows to the
places of a chain's rows 1 .. accept, so that the next iteration finds the committed positions where a chain leaves them.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from ....common import host

TABLE_WORDS = 96
PARENT, DEPTH, MASK, PATH, SLOT_FULL, SLOT_SWA = 0, 16, 32, 48, 64, 80


class TreeWalk:
    def __init__(self, lib: host.Library, module, *, cand: torch.Tensor, scores: torch.Tensor, words: torch.Tensor,
                 verify_ids: torch.Tensor, loc_full: Optional[torch.Tensor] = None, loc_swa: Optional[torch.Tensor] = None,
                 table: Optional[torch.Tensor] = None, cos_sin_cache: Optional[torch.Tensor] = None,
                 cos_sin: Optional[torch.Tensor] = None):  # fmt: skip
        """``cos_sin_cache`` / ``cos_sin``: the target's rope cache and its window feeds: rewritten by depth (the accept of
        the previous iteration wrote a chain's rows)."""
        rows = verify_ids.numel()
        assert cand.shape == (rows - 1, 16) and scores.shape == (rows - 1, 16, 16)
        self.table = table if table is not None else torch.zeros(TABLE_WORDS, dtype=torch.int32, device=cand.device)
        self.keep = (cand, scores, words, verify_ids, loc_full, loc_swa, cos_sin_cache, cos_sin)
        bind = host.make("MkDflashTreeBind", cand=cand, scores=scores, words=words, table=self.table, verify_ids=verify_ids,
                         loc_full=loc_full, loc_swa=loc_swa, rows=rows, cos_sin_cache=cos_sin_cache,
                         cos_sin_rows=0 if cos_sin_cache is None else cos_sin_cache.shape[0], cos_sin=cos_sin)  # fmt: skip
        self.launch = lib.bind("mk_dflash_tree_bind", module, bind)

    def rows(self) -> dict:
        t = self.table.cpu().tolist()
        return dict(parent=t[PARENT:DEPTH], depth=t[DEPTH:MASK], mask=t[MASK:PATH], path=t[PATH:SLOT_FULL])


class TreeCompact:
    def __init__(self, lib: host.Library, module, *, table: torch.Tensor, swa: Sequence[torch.Tensor] = (),
                 full: Sequence[torch.Tensor] = (), caps: Sequence[torch.Tensor] = ()):
        """``swa`` / ``full``: the K and V pools of the sliding-window / full-attention layers ([slots, row] each, one row
        width); ``caps``: the captured rows ([window rows, width], one width)."""
        kv = list(swa) + list(full)
        assert len({t[0].numel() * t.element_size() for t in kv}) <= 1 and len({t[0].numel() * t.element_size() for t in caps}) <= 1
        dev = table.device
        self.keep = (table, kv, list(caps))
        self.ptrs = torch.tensor([t.data_ptr() for t in kv + list(caps)], dtype=torch.int64, device=dev)
        bind = host.make(
            "MkDflashTreeCompactBind", table=table, rows=self.ptrs, n_swa=len(swa), n_full=len(full), n_cap=len(caps),
            kv_row_bytes=kv[0][0].numel() * kv[0].element_size() if kv else 0,
            cap_row_bytes=caps[0][0].numel() * caps[0].element_size() if caps else 0,
        )  # fmt: skip
        self.launch = lib.bind("mk_dflash_tree_compact_bind", module, bind)
