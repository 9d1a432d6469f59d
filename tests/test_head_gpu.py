"""Layer 0's head (mk_qkv_bind) against the oracle: GEMM + qk norm + RoPE, and the appended K/V rows."""

import pytest
import torch

from oracle import muse_layer as O
from sgl_muse_mega_b200.common import host
from sgl_muse_mega_b200.muse_spark.b200.head import QkvHead

pytestmark = pytest.mark.gpu


def make_inputs(rows, hidden, qh, kvh, seed, device):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(2 * (qh + kvh) * 64, hidden, generator=g) / hidden**0.5).bfloat16()
    x = torch.randn(rows, hidden, generator=g).bfloat16()
    cos_sin = O.rope_rows(torch.arange(100, 100 + rows), 500000.0)
    loc = torch.arange(5, 5 + rows, dtype=torch.int32)
    return w, x, cos_sin, loc


@pytest.mark.parametrize("rows,hidden,qh,kvh,rope", [(16, 8192, 16, 2, True), (16, 8192, 16, 2, False), (5, 1024, 8, 1, True), (1, 2048, 16, 4, True)])
def test_qkv_head(rows, hidden, qh, kvh, rope):
    dev = torch.device("cuda:0")
    lib = host.library()
    module = lib.load()
    w, x, cos_sin, loc = make_inputs(rows, hidden, qh, kvh, 3, dev)
    kc = torch.zeros(64, kvh * 64, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    head = QkvHead(lib, module, w=w.to(dev), x=x.to(dev), q_heads=qh, kv_heads=kvh, q_scale=43.7840518911 / 8, eps=1e-5,
                   cos_sin=cos_sin.to(dev) if rope else None, cache_loc=loc.to(dev), k_cache=kc, v_cache=vc)  # fmt: skip
    head.launch(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    ref = O.qkv_rowops(x, w, qh, kvh, 43.7840518911 / 8, 1e-5, cos_sin if rope else None)
    got = head.out.cpu()
    _, rel, ok = O.compare(got, ref, "qkv_next")
    assert ok, rel
    # the appended rows are the row's k and v heads, bit for bit
    k0, v0 = qh * 64, (qh + kvh) * 64
    assert torch.equal(kc[5 : 5 + rows].cpu(), got[:, k0:v0])
    assert torch.equal(vc[5 : 5 + rows].cpu(), got[:, v0 : v0 + kvh * 64])
    assert not kc[:5].any() and not kc[5 + rows :].any()
