"""The allocation-free head entry point, mk_qkv_launch_static, against mk_qkv_bind.

Some callers of this library cannot allocate device memory when they launch: a serving process hands the whole device
to its own memory pool at start-up, so a cudaMalloc made later by a plugin fails or eats into the pool's headroom. For
them the library carries the GEMM's scratch inside its own device image; this test holds that path to the ordinary one,
bit for bit, on two calls in a row (the second call finds the first call's leftovers in the shared scratch).
The file name sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""

import ctypes

import pytest
import torch

from sgl_muse_mega_b200.common import host
from sgl_muse_mega_b200.muse_spark.b200.head import QkvHead

pytestmark = pytest.mark.gpu


def _case(rows, hidden, qh, kvh, seed, dev):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(2 * (qh + kvh) * 64, hidden, generator=g) / hidden**0.5).bfloat16().to(dev)
    x = torch.randn(rows, hidden, generator=g).bfloat16().to(dev)
    ang = torch.rand(rows, 32, generator=g) * 6.28
    cos_sin = torch.cat((ang.cos(), ang.sin()), 1).to(dev)
    loc = torch.arange(3, 3 + rows, dtype=torch.int32, device=dev)
    return w, x, cos_sin, loc


def test_static_head_matches_bound_head_twice():
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    lib = host.library()
    module = lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    # two different shapes back to back: the second call's K split, tile count and counters differ from the first's
    for seed, (rows, hidden, qh, kvh) in enumerate([(16, 8192, 16, 2), (7, 2048, 8, 1)]):
        w, x, cos_sin, loc = _case(rows, hidden, qh, kvh, 40 + seed, dev)
        kc = torch.zeros(32, kvh * 64, dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        bound = QkvHead(lib, module, w=w, x=x, q_heads=qh, kv_heads=kvh, q_scale=5.473, eps=1e-5, cos_sin=cos_sin,
                        cache_loc=loc, k_cache=kc, v_cache=vc)  # fmt: skip
        bound.launch(stream)
        torch.cuda.synchronize()
        want, want_k, want_v = bound.out.clone(), kc.clone(), vc.clone()
        assert want.float().abs().sum() > 0

        out = torch.zeros_like(want)
        kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
        bind = host.make("MkQkvBind", w=w, x=x, out=out, cos_sin=cos_sin, cache_loc=loc, k_cache=kc2, v_cache=vc2,
                         q_scale=5.473, eps=1e-5, hidden=hidden, rows=rows, q_heads=qh, kv_heads=kvh, ws=None, ws_bytes=0)  # fmt: skip
        for call in range(2):
            out.zero_()
            lib.check(lib.dll.mk_qkv_launch_static(ctypes.byref(bind), stream), "mk_qkv_launch_static")
            torch.cuda.synchronize()
            assert torch.equal(out, want), f"shape {rows}x{hidden}, call {call}"
            assert torch.equal(kc2, want_k) and torch.equal(vc2, want_v)


def test_static_head_refuses_oversized_rows():
    dev = torch.device("cuda:0")
    lib = host.library()
    w, x, cos_sin, loc = _case(2, 256, 40, 2, 1, dev)  # qkv_row = 2 * 42 * 64 = 5376 > 4096
    out = torch.zeros(2, 5376, dtype=torch.bfloat16, device=dev)
    bind = host.make("MkQkvBind", w=w, x=x, out=out, cos_sin=cos_sin, cache_loc=loc, k_cache=None, v_cache=None,
                     q_scale=1.0, eps=1e-5, hidden=256, rows=2, q_heads=40, kv_heads=2, ws=None, ws_bytes=0)  # fmt: skip
    assert lib.dll.mk_qkv_launch_static(ctypes.byref(bind), torch.cuda.current_stream().cuda_stream) == -1
    assert "exceeds" in lib.dll.mk_last_error().decode()
