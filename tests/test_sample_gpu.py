"""The sampled accept through the C ABI against the oracle (``oracle/dflash_sample.py``, pinned to the reference's outputs):
the oracle is fed the kernel's own soft-capped, temperature-scaled rows (the per-stage method), so the kept sets and the
distributions are compared exactly / to 1e-12 and the accept length, the bonus token and the step words exactly."""

import pytest
import torch

from oracle import dflash_accept as A
from oracle import dflash_draft as D
from oracle import dflash_sample as S
from sgl_muse_mega_b200.common import host
from sgl_muse_mega_b200.muse_spark.b200 import headtail as HT
from sgl_muse_mega_b200.muse_spark.b200.dflash.draft import sampling_words

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
MULT, CAP = 32**-0.5, 20.0
SEED, STREAM = 0xFEDCBA9876543210, 5


def stream():
    return torch.cuda.current_stream().cuda_stream


def draw(vocab, rows, boost, grid, seed):
    """Pre-cap logits, the slots' candidates, the walk's probabilities and the window's ids (anchor, then one candidate a
    slot); ``boost`` lifts the drafted ids' target logits, ``grid`` puts the logits on a lattice (ties)."""
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(rows, vocab, generator=g) * 12.0
    if grid:
        logits = (logits / grid).round() * grid
    cand = torch.stack([torch.randperm(vocab, generator=g)[:16] for _ in range(rows - 1)])
    q = torch.softmax(torch.randn(rows - 1, 16, generator=g) / 0.7, -1)
    pick = torch.randint(0, 16, (rows - 1,), generator=g)
    drafts = cand.gather(1, pick[:, None])[:, 0]
    tokens = torch.cat([torch.randint(0, vocab, (1,), generator=g), drafts])
    logits[torch.arange(rows - 1), drafts] += boost
    return logits, cand, q, tokens


CASES = [
    # vocab, rows, temperature, top_k, top_p, block, boost, grid, seed
    (512, 16, 0.7, 1 << 30, 1.0, True, 40.0, 0.0, 1),
    (512, 16, 1.0, 40, 0.9, True, 30.0, 0.0, 2),
    (512, 16, 1.3, 8, 1.0, False, 20.0, 4.0, 3),
    (512, 8, 0.8, 1 << 30, 0.95, False, 35.0, 0.0, 4),
    (25256, 16, 0.8, 1 << 30, 1.0, True, 45.0, 0.0, 5),
    (25256, 16, 1.0, 64, 0.95, True, 40.0, 2.0, 6),
    (202048, 16, 0.7, 1 << 30, 1.0, True, 55.0, 0.0, 7),
    (202048, 16, 1.0, 50, 0.9, True, 50.0, 0.0, 8),
    (202048, 16, 0.9, 1 << 30, 0.8, False, 50.0, 3.0, 9),
    (202048, 16, 0.5, 1 << 30, 1.0, True, 200.0, 0.0, 10),
    # prefixes accepted with a scaled residual (0 < r < 1)
    (512, 16, 0.8, 1 << 30, 1.0, True, 25.0, 0.0, 21),
    (512, 16, 0.8, 1 << 30, 1.0, True, 25.0, 0.0, 22),
    (25256, 16, 1.0, 64, 0.95, True, 32.0, 0.0, 24),
    (202048, 16, 0.8, 1 << 30, 1.0, True, 40.0, 0.0, 30),
    # a vocabulary whose quarter does not fit a CTA's shared memory: one CTA per row, plain bisections
    (262144, 8, 1.0, 64, 0.9, True, 40.0, 0.0, 11),
    (262144, 8, 0.8, 1 << 30, 1.0, False, 40.0, 0.0, 12),
]


@pytest.mark.parametrize("vocab,rows,temp,top_k,top_p,block,boost,grid,seed", CASES)
def test_sampled_accept(vocab, rows, temp, top_k, top_p, block, boost, grid, seed):
    lib = host.library()
    module = lib.load()
    lg, cand, q, tokens = draw(vocab, rows, boost, grid, seed)
    samp = sampling_words(SEED, STREAM, temp, top_k, top_p).to(DEV)
    logits, toks, cand_d, q_d = lg.to(DEV), tokens.to(DEV), cand.to(DEV), q.to(DEV)
    acc = HT.Accept(lib, module, logits=logits, tokens=toks, b_live=rows, scale=MULT, cap=CAP, ring=40, samp=samp,
                    cand=cand_d, walk_q=q_d, block_verify=block)  # fmt: skip
    acc.words[A.WORDS["P"]] = 100
    acc.words[A.WORDS["ITER"]] = 7 + seed
    words, ring = acc.words.cpu(), acc.out_ring.cpu()
    acc.launch(stream())
    torch.cuda.synchronize()
    assert acc.launch.status(stream()).code == 0
    # the kernel's own rows: capped logit / T, and the kept entries' exp(y - max)
    cells = rows * vocab
    ys = acc.sample_ws[: cells * 4].view(torch.float32).view(rows, vocab).cpu()
    off = (cells * 4 + 255) // 256 * 256
    es = acc.sample_ws[off : off + cells * 8].view(torch.float64).view(rows, vocab).cpu()
    zs = acc.sample_ws[off + cells * 8 : off + cells * 8 + rows * 8].view(torch.float64).cpu()
    want_y = (torch.tanh((lg * MULT) / CAP) * CAP) / torch.tensor(temp, dtype=torch.float32)
    assert torch.allclose(ys, want_y, rtol=2e-6, atol=1e-6)
    top_p32 = float(torch.tensor(top_p, dtype=torch.float32))  # the words hold top_p as f32
    probs = S.target_probs(ys, 1.0, min(top_k, vocab), top_p32)
    assert torch.equal(es > 0, probs > 0), "the kept sets differ"
    got = es / zs[:, None]
    assert torch.allclose(got, probs, rtol=1e-12, atol=1e-300)
    u = D.uniforms(SEED, STREAM, 7 + seed, S.PURPOSE_ACCEPT)
    ref = S.sampled_accept(tokens, probs, cand, q, u, block)
    w = acc.words.cpu()
    assert (int(w[A.WORDS["ACCEPT"]]), int(w[A.WORDS["ANCHOR"]])) == (ref.accept_len, ref.bonus)
    scale, mass = acc.sample_out.cpu()[:2].tolist()
    assert scale == pytest.approx(ref.scale, rel=1e-9) and mass == pytest.approx(ref.norm, rel=1e-9)
    step = A.Accept(ref.accept_len, ref.accept_len + 1, ref.bonus, None, 100 + ref.accept_len + 1)
    words, ring = A.step_words(words, ring, step, tokens)
    assert torch.equal(w, words) and torch.equal(acc.out_ring.cpu(), ring)


def test_the_cases_reach_every_branch():
    """Host-only bookkeeping of the table above: the oracle's outcomes over the cases include a rejection at slot 0, a
    partial prefix with a scaled residual, and a full accept (so the GPU test exercises them)."""
    seen = set()
    for vocab, rows, temp, top_k, top_p, block, boost, grid, seed in CASES:
        if vocab > 30000:
            continue
        lg, cand, q, tokens = draw(vocab, rows, boost, grid, seed)
        y = (torch.tanh((lg * MULT) / CAP) * CAP) / torch.tensor(temp, dtype=torch.float32)
        probs = S.target_probs(y, 1.0, min(top_k, vocab), top_p)
        r = S.sampled_accept(tokens, probs, cand, q, D.uniforms(SEED, STREAM, 7 + seed, 1), block)
        seen.add("none" if r.accept_len == 0 else "full" if r.accept_len == rows - 1 else "scaled" if r.scale < 1 else "part")
    assert {"none", "scaled", "part"} <= seen, seen
