"""Stand-alone launches around the decoder layers. ``QkvHead`` is layer 0's head: the qkv GEMM, the per-head qk norm,
RoPE and the K/V append, the same work a layer launch does for its successor (reference: ``Stack`` binds it as
``qkv_head``, ``sm103/verify.py:423-433``; kernel ``kernels/head.cu:308-315``)."""

from __future__ import annotations

from typing import Optional

import torch

from ...common import host


class QkvHead:
    def __init__(self, lib: host.Library, module, *, w, x, q_heads: int, kv_heads: int, q_scale: float, eps: float,
                 cos_sin: Optional[torch.Tensor], cache_loc, k_cache=None, v_cache=None):  # fmt: skip
        rows, hidden = x.shape
        self.out = torch.zeros(rows, 2 * (q_heads + kv_heads) * 64, dtype=torch.bfloat16, device=x.device)
        self.keep = (w, x, cos_sin, cache_loc, k_cache, v_cache)
        fields = dict(w=w, x=x, out=self.out, cos_sin=cos_sin, cache_loc=cache_loc, k_cache=k_cache, v_cache=v_cache,
                      q_scale=q_scale, eps=eps, hidden=hidden, rows=rows, q_heads=q_heads, kv_heads=kv_heads,
                      ws=None, ws_bytes=0)  # fmt: skip
        self.consts = lib.qkv_constants(host.make("MkQkvBind", **fields))
        self.ws = torch.zeros(self.consts.ws_bytes, dtype=torch.uint8, device=x.device)
        fields.update(ws=self.ws, ws_bytes=self.consts.ws_bytes)
        self.bind = host.make("MkQkvBind", **fields)
        self.launch_record = lib.qkv_bind(module, self.bind)

    def launch(self, stream: int, pdl: bool = False) -> None:
        self.launch_record(stream, pdl)
