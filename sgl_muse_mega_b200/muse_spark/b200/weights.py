"""Per-rank expert shards and the tensor-core weight images the B200 expert kernels stream (their ABI).

Same role as the reference's ``sm103/weights.py``: ``shard_*`` cut a checkpoint's expert stack to the rank's rows
(``weights.py:62-77``), ``pack_*`` build the kernel layout from the shards, ``unpack_*`` invert it exactly. The layout
itself is this library's own: one contiguous *stage* per (expert, 128-row block, 256-element K chunk), which the kernel
fetches with a single bulk copy and feeds to ``tcgen05.mma.kind::mxf4nvf4`` without touching a byte:

    stage = [tile 0][tile 1 (W1 only)][scales 0][scales 1 (W1 only)]
    tile   = 128 rows x 128 bytes (256 e2m1 codes), 8-row groups of 1024 bytes, the 16-byte chunk j of row r stored at
             chunk j ^ (r % 8)                                   (the 128-byte-swizzle K-major operand layout)
    scales = 4 K64 blocks x 512 bytes; byte n*16 + g*4 + k of a block = e4m3 scale of tile row 32 g + n, 16-element
             group k of that block                               (the 32 x 16 B image tcgen05.cp.32x128b.warpx4 copies)

W1 pairs the gate rows of a 128-feature block (tile 0) with the same features' up rows (tile 1), as the reference pairs
them (``weights.py:80-111``), so one thread of the epilogue sees both halves of a feature.
"""

from __future__ import annotations

import torch

TILE_ROWS = 128
K_CHUNK = 256  # elements per stage along K
TILE_BYTES = TILE_ROWS * K_CHUNK // 2
SF_BYTES = 4 * 512
W1_STAGE = 2 * (TILE_BYTES + SF_BYTES)
W2_STAGE = TILE_BYTES + SF_BYTES


def shard_w13(w13: torch.Tensor, rank: int, ranks: int, inter: int):
    """The rank's (gate, up) rows of a checkpoint w13 [E, 2 inter, ...] (gate rows first)."""
    i_s = inter // ranks
    return tuple(w13[:, h * inter + rank * i_s : h * inter + (rank + 1) * i_s] for h in (0, 1))


def shard_w2(w2: torch.Tensor, rank: int, ranks: int, hidden: int) -> torch.Tensor:
    """The rank's output rows of a checkpoint w2 [E, hidden, ...]."""
    h_s = hidden // ranks
    return w2[:, rank * h_s : (rank + 1) * h_s]


def _swizzle_index(device) -> torch.Tensor:
    """[8 rows, 8 chunks]: the source chunk that lands in physical chunk c of row r (XOR is its own inverse)."""
    r = torch.arange(8, device=device)[:, None]
    c = torch.arange(8, device=device)[None, :]
    return c ^ r


def _tiles(q: torch.Tensor) -> torch.Tensor:
    """codes [E, R, K/2] -> swizzled tiles [E, R/128, K/256, 16384]."""
    e, rows, kb = q.shape
    nb, kc = rows // TILE_ROWS, kb // 128
    t = q.reshape(e, nb, 16, 8, kc, 8, 16).permute(0, 1, 4, 2, 3, 5, 6)  # [e, nb, kc, group, row8, chunk, 16]
    idx = _swizzle_index(q.device)[None, None, None, None, :, :, None].expand(e, nb, kc, 16, 8, 8, 16)
    return torch.gather(t, 5, idx).reshape(e, nb, kc, TILE_BYTES)


def _untiles(t: torch.Tensor, rows: int, kb: int) -> torch.Tensor:
    e, nb, kc, _ = t.shape
    v = t.reshape(e, nb, kc, 16, 8, 8, 16)
    idx = _swizzle_index(t.device)[None, None, None, None, :, :, None].expand(e, nb, kc, 16, 8, 8, 16)
    v = torch.gather(v, 5, idx)
    return v.permute(0, 1, 3, 4, 2, 5, 6).reshape(e, rows, kb)


def _sf_images(sf: torch.Tensor) -> torch.Tensor:
    """scales [E, R, K/16] -> [E, R/128, K/256, 2048]: per K chunk four 512-byte blocks, byte n*16 + g*4 + k."""
    e, rows, ks = sf.shape
    nb, kc = rows // TILE_ROWS, ks // 16
    v = sf.reshape(e, nb, 4, 32, kc, 4, 4)  # [e, nb, g, n, kc, block, k]
    return v.permute(0, 1, 4, 5, 3, 2, 6).reshape(e, nb, kc, SF_BYTES)  # [e, nb, kc, block, n, g, k]


def _unsf_images(img: torch.Tensor, rows: int, ks: int) -> torch.Tensor:
    e, nb, kc, _ = img.shape
    v = img.reshape(e, nb, kc, 4, 32, 4, 4)
    return v.permute(0, 1, 5, 4, 2, 3, 6).reshape(e, rows, ks)


def _check(q: torch.Tensor, sf: torch.Tensor) -> None:
    assert q.dtype == torch.uint8 and sf.dtype == torch.uint8
    assert q.shape[1] % TILE_ROWS == 0, f"rows {q.shape[1]} are not whole 128-row tiles"
    assert (2 * q.shape[2]) % K_CHUNK == 0, f"K {2 * q.shape[2]} is not a multiple of {K_CHUNK}"
    assert sf.shape == (q.shape[0], q.shape[1], q.shape[2] // 8), (q.shape, sf.shape)


def pack_w1_fp4(gate_q, gate_sf, up_q, up_sf) -> torch.Tensor:
    """The rank's NVFP4 W1 (gate / up codes [E, I_s, P/2], scales [E, I_s, P/16]) -> [E, I_s/128, P/256, 36864] u8."""
    _check(gate_q, gate_sf)
    _check(up_q, up_sf)
    return torch.cat((_tiles(gate_q), _tiles(up_q), _sf_images(gate_sf), _sf_images(up_sf)), dim=-1).contiguous()


def unpack_w1_fp4(pack: torch.Tensor):
    """Exact inverse of ``pack_w1_fp4`` -> (gate_q, gate_sf, up_q, up_sf)."""
    e, nb, kc, stage = pack.shape
    assert stage == W1_STAGE
    rows, kb, ks = nb * TILE_ROWS, kc * 128, kc * 16
    g, u, gs, us = pack.split((TILE_BYTES, TILE_BYTES, SF_BYTES, SF_BYTES), dim=-1)
    return _untiles(g, rows, kb), _unsf_images(gs, rows, ks), _untiles(u, rows, kb), _unsf_images(us, rows, ks)


def pack_w2_fp4(w2_q, w2_sf) -> torch.Tensor:
    """The rank's NVFP4 W2 (codes [E, H_s, I/2], scales [E, H_s, I/16]) -> [E, H_s/128, I/256, 18432] u8."""
    _check(w2_q, w2_sf)
    return torch.cat((_tiles(w2_q), _sf_images(w2_sf)), dim=-1).contiguous()


def unpack_w2_fp4(pack: torch.Tensor):
    e, nb, kc, stage = pack.shape
    assert stage == W2_STAGE
    rows, kb, ks = nb * TILE_ROWS, kc * 128, kc * 16
    t, s = pack.split((TILE_BYTES, SF_BYTES), dim=-1)
    return _untiles(t, rows, kb), _unsf_images(s, rows, ks)


def pack_items(w: torch.Tensor) -> torch.Tensor:
    """A row-major GEMM weight [N, K] (bf16, or f32 for the router) -> the item images the item engine streams:
    [ceil(N / bn)][K / 512][bn rows][512 k + 64 bytes of padding], bn = 64 (bf16) or 16 (f32), rows past N zero. An item
    (one N block x one K chunk) is then contiguous and arrives by a few large bulk copies with its rows already at the
    padded stride the kernel's shared-memory reads want. K must be a multiple of 512."""
    n, k = w.shape
    f32 = w.dtype == torch.float32
    bn, kc, pad = (16, 512, 16) if f32 else (64, 512, 32)
    if k % kc:
        raise ValueError(f"K {k} is not a multiple of {kc}")
    nb = (n + bn - 1) // bn
    out = torch.zeros(nb, k // kc, bn, kc + pad, dtype=w.dtype, device=w.device)
    full = n // bn
    if full:
        out[:full, :, :, :kc] = w[: full * bn].view(full, bn, k // kc, kc).permute(0, 2, 1, 3)
    if n % bn:
        out[full, :, : n % bn, :kc] = w[full * bn :].view(n % bn, k // kc, kc).permute(1, 0, 2)
    return out


# ---- tile images of the tensor-core dense engine (csrc/dense.cu) ---------------------------------------------------------------

UMMA_ROWS = 128  # weight rows per tile (the M operand of tcgen05.mma)
UMMA_STAGE_BYTES = 256  # bytes of K per stage and row: two 128-byte swizzle atoms


def pack_umma(w: torch.Tensor, perm: torch.Tensor | None = None) -> torch.Tensor:
    """A row-major GEMM weight [N, K] (bf16, or f32 for the router) -> the tile images the tensor-core dense engine streams:
    u8 [ceil(N / 128)][K bytes / 256][2 atoms][128 rows][128 bytes], the 16-byte chunk j of row r of an atom stored at chunk
    j ^ (r % 8) (K-major 128-byte swizzle), rows past N zero. One (tile, K stage) is 32 KiB and arrives by two bulk copies.
    ``perm``: tile row i of the image holds row ``perm[i]`` of ``w`` (the epilogues that pair rows: SwiGLU, conv).
    f32 weights lose their low 13 mantissa bits here (the tf32 operand the reference's router defines, R1:123-125)."""
    if w.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"dtype {w.dtype} is not bf16 / f32")
    if perm is not None:
        w = w[perm.to(w.device)]
    n, k = w.shape
    row_bytes = k * w.element_size()
    if row_bytes % UMMA_STAGE_BYTES:
        raise ValueError(f"K {k} ({row_bytes} bytes) is not a whole number of {UMMA_STAGE_BYTES}-byte stages")
    if w.dtype == torch.float32:
        w = (w.contiguous().view(torch.int32) & ~0x1FFF).view(torch.float32)
    tiles, ks = (n + UMMA_ROWS - 1) // UMMA_ROWS, row_bytes // UMMA_STAGE_BYTES
    b = torch.zeros(tiles * UMMA_ROWS, row_bytes, dtype=torch.uint8, device=w.device)
    b[:n] = w.contiguous().view(torch.uint8).view(n, row_bytes)
    v = b.view(tiles, 16, 8, ks, 2, 8, 16).permute(0, 3, 4, 1, 2, 5, 6)  # [tile, stage, atom, group, row8, chunk, 16]
    idx = _swizzle_index(w.device)[None, None, None, None, :, :, None].expand(tiles, ks, 2, 16, 8, 8, 16)
    return torch.gather(v, 5, idx).reshape(tiles, ks, 2, UMMA_ROWS, 128).contiguous()


def unpack_umma(img: torch.Tensor, n: int, dtype: torch.dtype) -> torch.Tensor:
    """Exact inverse of ``pack_umma`` without ``perm`` (up to the router's cleared mantissa bits): -> [n, K]."""
    tiles, ks = img.shape[:2]
    v = img.reshape(tiles, ks, 2, 16, 8, 8, 16)
    idx = _swizzle_index(img.device)[None, None, None, None, :, :, None].expand(tiles, ks, 2, 16, 8, 8, 16)
    v = torch.gather(v, 5, idx).permute(0, 3, 4, 1, 2, 5, 6).reshape(tiles * UMMA_ROWS, ks * UMMA_STAGE_BYTES)
    return v[:n].contiguous().view(dtype)


def silu_perm(inter: int) -> torch.Tensor:
    """Row order of a [gate rows | up rows] weight ([2 inter, K]) for the SwiGLU epilogue: tile t holds gate rows
    64 t .. 64 t + 63, then the same features' up rows."""
    t = torch.arange(inter // 64)[:, None] * 64 + torch.arange(64)[None, :]
    return torch.cat((t, t + inter), 1).reshape(-1)


def pack_bf16_experts(gate: torch.Tensor, up: torch.Tensor, w2: torch.Tensor) -> tuple:
    """A bf16 layer's experts (this rank's shards: gate, up [E, I_s, P], w2 [E, H_s, I]) -> the tile images of the grouped
    tensor-core GEMM (``csrc/experts_bf16_umma.cu``): (w1 image, w2 image), each u8
    [E x tiles per expert][K bytes / 256][2][128][128]. w1's tiles hold 64 gate rows and the same features' up rows
    (``silu_perm`` inside every expert), w2's its rows in order. I_s must be a multiple of 64, H_s of 128."""
    e, i_s, p = gate.shape
    h_s = w2.shape[1]
    if i_s % 64 or h_s % 128:
        raise ValueError(f"I_s {i_s} is not a multiple of 64 or H_s {h_s} not of 128")
    perm = silu_perm(i_s).to(gate.device)
    w1 = torch.cat((gate, up), 1)[:, perm]  # [E, 2 I_s, P]: per expert, tile t = gate rows 64 t .., then up rows 64 t ..
    img1 = pack_umma(w1.reshape(e * 2 * i_s, p))
    del w1
    img2 = pack_umma(w2.reshape(e * h_s, w2.shape[2]))
    return img1, img2


def conv_perm(groups: int) -> torch.Tensor:
    """Row order of a conv projection ([4 groups, K], rows kind x groups + group) for the conv epilogue: tile t holds the four
    kinds' coefficients of groups 32 t .. 32 t + 31 (tile row kind 32 + group)."""
    t = torch.arange(groups // 32)[:, None, None] * 32
    kind = torch.arange(4)[None, :, None] * groups
    g = torch.arange(32)[None, None, :]
    return (t + kind + g).reshape(-1)


def pack_dense(w: torch.Tensor, packed: int, perm: torch.Tensor | None = None) -> torch.Tensor:
    """The weight in the layout of the dense engine ``packed`` names: 0 row-major, 1 item images, 2 tile images."""
    packed = int(packed)
    if packed == 2:
        return pack_umma(w, perm)
    return pack_items(w) if packed == 1 else w
