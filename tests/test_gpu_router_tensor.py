"""The router that prefill-sized batches take by default: logits on the tensor cores (two fp16 terms per hidden value, fp32
accumulation), top-8 taken from them where the nine largest are further apart than an error bound, and recomputed in the
reference's exact order of operations where they are not.  Contract (maple.c:870-889, 910-923):
  * top-8 indices equal the reference's for every token, ties and near-ties included;
  * weights within 1e-5 relative, logits within 2e-5 absolute of the reference's fp32 values."""
import numpy as np
import pytest

from conftest import SEED

pytestmark = pytest.mark.gpu
TOL_W, TOL_L = 1e-5, 2e-5


@pytest.fixture(scope="module")
def g(gpu):
    gpu.synth_layer(SEED, 2)
    return gpu


def oracle_topk_all(oracle, logits):
    top = np.zeros((logits.shape[0], 8), np.int32); w = np.zeros((logits.shape[0], 8), np.float32)
    for b in range(logits.shape[0]):
        top[b], w[b], _ = oracle.topk(logits[b])
    return top, w


@pytest.mark.parametrize("nb,stream,with_bias", [(512, 601, False), (700, 602, True), (2048, 603, False), (2047, 604, True), (129, 605, False), (1, 606, False)])
def test_indices_equal_and_values_close_to_the_oracle(nb, stream, with_bias, g, clib, oracle, weights):
    from maple_runtime_b200 import lib as ml
    router, _, _ = weights.layer(2)
    hn = weights.hidden(stream, nb)
    bias = ml.synth_zipf_bias(clib, SEED) if with_bias else None
    want_l = oracle.router_logits(router, hn)
    if with_bias:
        want_l = want_l + bias[None, :]
        g.poke("bias", bias)
    want_top, want_w = oracle_topk_all(oracle, want_l)
    g.poke("hn", hn)
    g.stage("router_tensor_bias" if with_bias else "router_tensor", 2, nb)
    got_l, got_top, got_w = g.peek("logits", nb).reshape(nb, 256), g.peek("top", nb).reshape(nb, 8), g.peek("topw", nb).reshape(nb, 8)
    assert np.array_equal(got_top, want_top), f"{int((got_top != want_top).any(1).sum())} tokens with other indices"
    assert float(np.abs(got_l - want_l).max()) <= TOL_L
    assert float((np.abs(got_w - want_w) / want_w).max()) <= TOL_W
    flagged = clib.gmoe_router_flagged()
    assert 0 <= flagged <= max(8, nb // 4), f"{flagged} of {nb} tokens took the exact path"


def test_ties_and_degenerate_rows_take_the_exact_path(g, clib, oracle, weights):
    """All-zero rows (every logit equal), identical tokens, a token that is the negative of another: the selection must be the
    reference's first-maximum rule, bit for bit in the weights too (these rows are recomputed exactly)."""
    router, _, _ = weights.layer(2)
    nb = 600
    hn = weights.hidden(611, nb)
    hn[5] = 0.0; hn[77] = hn[76]; hn[300] = -hn[301]; hn[599] = 0.0
    # a token built to have two equal logits: make two router rows see the same input by zeroing everything (covered by the zero rows)
    want_l = oracle.router_logits(router, hn)
    want_top, want_w = oracle_topk_all(oracle, want_l)
    g.poke("hn", hn)
    g.stage("router_tensor", 2, nb)
    got_top, got_w = g.peek("top", nb).reshape(nb, 8), g.peek("topw", nb).reshape(nb, 8)
    assert np.array_equal(got_top, want_top)
    for b in (5, 599):
        assert list(got_top[b]) == list(range(8)) and np.array_equal(got_w[b].view(np.uint32), want_w[b].view(np.uint32))
    assert clib.gmoe_router_flagged() >= 2


def test_a_million_tokens_select_the_same_experts_as_the_exact_router(g, clib, weights):
    """512 chunks of 2048 synthetic tokens (every fourth with the skewing bias): indices from the tensor-core path against the
    exact-order kernels (which other tests pin to the oracle bit for bit); also the observed error against the bound the
    selection uses (2^-18 |hn| max|W_e|): it must stay below a quarter of it."""
    from maple_runtime_b200 import lib as ml
    nb, chunks = 2048, 512
    router, _, _ = weights.layer(2)
    wn = float(np.sqrt((router.astype(np.uint32) << 16).view(np.float32).astype(np.float64) ** 2).sum(1).max()) if False else None
    wf = (router.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    wnorm = float(np.sqrt((wf ** 2).sum(1)).max())
    bias = ml.synth_zipf_bias(clib, SEED)
    g.poke("bias", bias)
    worst, flagged_max, mism = 0.0, 0, 0
    for c in range(chunks):
        hn = weights.hidden(10000 + c, nb)
        b = (c % 4) == 3
        g.poke("hn", hn)
        g.stage("router_tensor_bias" if b else "router_tensor", 2, nb)
        top_t, l_t = g.peek("top", nb).copy(), g.peek("logits", nb).reshape(nb, 256).copy()
        flagged_max = max(flagged_max, clib.gmoe_router_flagged())
        g.stage("router_bias" if b else "router", 2, nb)
        g.stage("topk", 2, nb)
        top_e, l_e = g.peek("top", nb), g.peek("logits", nb).reshape(nb, 256)
        mism += int((top_t.reshape(nb, 8) != top_e.reshape(nb, 8)).any(1).sum())
        hnorm = np.sqrt((hn.astype(np.float64) ** 2).sum(1))
        worst = max(worst, float((np.abs(l_t.astype(np.float64) - l_e).max(1) / (hnorm * wnorm)).max()))
    print(f"tensor-core router over {chunks * nb} tokens: {mism} tokens with other indices, worst |dlogit| / (|hn| max|W|) = {worst:.3e} "
          f"(bound used 2^-18 = {2.0 ** -18:.3e}), at most {flagged_max} of {nb} tokens per chunk recomputed exactly")
    assert mism == 0
    assert worst < 2.0 ** -20
    assert flagged_max < nb // 4
