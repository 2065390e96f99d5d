"""gmoe_group_noalloc: the grouping for callers that cannot allocate device memory (a fixed memory budget, another
runtime's pool, a latency path).  Its scratch is a fixed array inside the library, so this test checks what that
changes: the result must equal the CPU oracle's grouping and the ordinary grouping stage's, also on later calls
that find an earlier call's leftovers in the shared scratch (a different number of bit-mask words per expert
between calls), and sizes beyond the built-in limit must be refused.

Collected last on purpose: a failure here leaves every other test already run."""
import ctypes as C
import numpy as np
import pytest

from conftest import SEED

pytestmark = pytest.mark.gpu


def routing(rng, nb, skew=False):
    """Random top-8 tables: distinct experts per token, positive weights."""
    p = None
    if skew:
        p = 1.0 / np.arange(1, 257) ** 1.2; p /= p.sum()
    top = np.stack([rng.choice(256, 8, replace=False, p=p) for _ in range(nb)]).astype(np.int32)
    w = rng.random((nb, 8)).astype(np.float32) + 0.01
    return top, (w / w.sum(1, keepdims=True)).astype(np.float32)


def test_noalloc_grouping_equals_oracle_and_grouping_stage(gpu, clib, oracle):
    torch = pytest.importorskip("torch")   # only to own device buffers for the caller's side of the call
    g = gpu
    g.synth_layer(SEED, 23, 0, 256)        # gmoe_stage wants a layer; layer 23 is used by no other test
    rng = np.random.default_rng(11)
    dev = torch.device("cuda:0")
    outs = dict(nu=torch.zeros(1, dtype=torch.int32, device=dev), ue=torch.zeros(256, dtype=torch.int32, device=dev),
                ustart=torch.zeros(257, dtype=torch.int32, device=dev), utok=torch.zeros(2048 * 8, dtype=torch.int32, device=dev),
                uw=torch.zeros(2048 * 8, dtype=torch.float32, device=dev), tp=torch.zeros(2048 * 8, dtype=torch.int32, device=dev))
    # 2048 skewed tokens fill the bit masks in the library's array (64 words per expert); 300 tokens then use 10 words per
    # expert of the same array: bits or counters left by the first call would show up as phantom pairs.  Both sizes take the
    # kernels that keep their masks in that array; 37 tokens take the one-CTA kernel, whose masks live in shared memory.
    for nb, skew in ((2048, True), (300, False), (37, False), (1024, True)):
        top, tw = routing(rng, nb, skew)
        o_nu, o_ue, o_ustart, o_utok, o_uw, o_tp = oracle.group(top, tw)
        g.poke("top", top); g.poke("topw", tw)
        g.stage("group", 23, nb)
        want = {k: g.peek(k, nb) for k in ("nu", "ue", "ustart", "utok", "uw", "tp")}
        nu = int(want["nu"][0])
        t_top, t_tw = torch.from_numpy(top).to(dev), torch.from_numpy(tw).to(dev)
        torch.cuda.synchronize()
        rc = clib.gmoe_group_noalloc(t_top.data_ptr(), t_tw.data_ptr(), nb, outs["nu"].data_ptr(), outs["ue"].data_ptr(),
                                     outs["ustart"].data_ptr(), outs["utok"].data_ptr(), outs["uw"].data_ptr(), outs["tp"].data_ptr(), None)
        assert rc == 0
        torch.cuda.synchronize()
        got = {k: v.cpu().numpy() for k, v in outs.items()}
        # against the CPU oracle (group_pairs and the tp loop of the reference, restated)
        assert int(got["nu"][0]) == o_nu
        assert np.array_equal(got["ue"][:o_nu], o_ue[:o_nu])
        assert np.array_equal(got["ustart"][:o_nu + 1], o_ustart[:o_nu + 1])
        assert np.array_equal(got["utok"][:nb * 8], o_utok) and np.array_equal(got["tp"][:nb * 8], o_tp)
        assert np.array_equal(got["uw"][:nb * 8].view(np.uint32), o_uw.view(np.uint32))
        # and against the allocating entry point
        assert int(got["nu"][0]) == nu
        assert np.array_equal(got["ue"][:nu], want["ue"][:nu])
        assert np.array_equal(got["ustart"][:nu + 1], want["ustart"][:nu + 1])
        for k in ("utok", "tp"):
            assert np.array_equal(got[k][:nb * 8], want[k][:nb * 8]), k
        assert np.array_equal(got["uw"][:nb * 8].view(np.uint32), want["uw"][:nb * 8].view(np.uint32))   # copied weights: same bits
        assert got["ustart"][nu] == nb * 8
    # the limit is enforced before anything is queued
    assert clib.gmoe_group_noalloc(t_top.data_ptr(), t_tw.data_ptr(), 2049, outs["nu"].data_ptr(), outs["ue"].data_ptr(),
                                   outs["ustart"].data_ptr(), outs["utok"].data_ptr(), outs["uw"].data_ptr(), outs["tp"].data_ptr(), None) == -2
    assert clib.gmoe_group_noalloc(None, t_tw.data_ptr(), 8, outs["nu"].data_ptr(), outs["ue"].data_ptr(),
                                   outs["ustart"].data_ptr(), outs["utok"].data_ptr(), outs["uw"].data_ptr(), outs["tp"].data_ptr(), None) == -1
