"""GPU parity tests: the CUDA path, called through the C ABI, against the oracle on the same seeded inputs.
Integer stages (int8 activations, top-8 indices, grouping, int32 dot products) must be equal; fp32 stages are
compared bit for bit first and, where that is not asserted, within 1e-5 relative in the reference's own sense
(max |a-b| / max |ref| per tensor, maple.c:942-946)."""
import hashlib
import os
import sys
import numpy as np
import pytest

from conftest import SEED, same_bits

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden as mg  # noqa: E402

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "moe_cases.npz"))
TOL = 1e-5


def rel(a, b):
    return float(np.abs(a.astype(np.float64) - b).max() / max(float(np.abs(b).max()), 1e-30))


def digest(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), np.uint8)


@pytest.fixture(scope="module")
def layers(gpu):
    """Layers 0..2 generated on the device by the synthetic generator."""
    for L in range(3):
        gpu.synth_layer(SEED, L)
    return gpu


def test_device_generator_equals_host_generator(layers, clib, weights):
    import ctypes as C
    from maple_runtime_b200 import lib as ml
    _, _, experts = weights.layer(1)
    got = np.empty(experts.nbytes, np.uint8)
    rid = layers.layer_region[1]
    assert clib.gmoe_region_read(rid, 0, got.ctypes.data_as(C.c_void_p), got.nbytes) == 0
    assert np.array_equal(got, experts)


def check_stages(g, nb, d, exact_fp=True):
    """Compare every stage buffer of the last call with an oracle dump."""
    nu = int(d["nu"][0])
    assert int(g.peek("nu", nb)[0]) == nu
    for k in ("hq", "hqsum", "top", "utok", "tp", "aq", "aqsum"):
        assert np.array_equal(g.peek(k, nb), d[k].reshape(g.peek(k, nb).shape)), k
    assert np.array_equal(g.peek("ue", nb)[:nu], d["ue"][:nu])
    assert np.array_equal(g.peek("ustart", nb)[:nu + 1], d["ustart"][:nu + 1])
    if "gu_dots" in d:
        assert np.array_equal(g.peek("gu_dots", nb), d["gu_dots"])
        assert np.array_equal(g.peek("dn_dots", nb), d["dn_dots"])
    for k in ("hqs", "logits", "topw", "uw", "gate", "up", "act", "aqs", "down"):
        got, want = g.peek(k, nb), d[k]
        got = got.reshape(want.shape)
        if exact_fp:
            assert same_bits(got, want), f"{k}: rel {rel(got, want):.3e}"
        else:
            assert rel(got, want) <= TOL, k


@pytest.mark.parametrize("nb,stream,norm", [(1, 201, 0), (5, 202, 0), (32, 203, 1), (33, 204, 1), (64, 205, 0), (128, 206, 1), (200, 207, 1), (256, 208, 0), (257, 209, 1)])
def test_layer_all_stages_equal_oracle(nb, stream, norm, layers, oracle, weights):
    """Configs 1 (128-token chunk) and 2 (64 conversations) and the route_small/route_multi boundary."""
    g = layers
    router, post_ln, experts = weights.layer(0)
    x = weights.hidden(stream, nb)
    want, d = oracle.moe(router, post_ln, experts, x, norm, dots=True)
    if norm:
        xx = x.copy(); g.forward(xx, 0, 1); got = xx
        assert same_bits(g.peek("hn", nb), np.stack([oracle.rmsnorm(r, post_ln) for r in x]))
    else:
        got, _ = g.moe(0, x)
    check_stages(g, nb, d)
    assert same_bits(got, want), f"rel {rel(got, want):.3e}"


@pytest.mark.parametrize("nb,tt", [(257, 0), (300, 5), (999, 0), (1300, 0), (1301, 6), (1600, 0), (2048, 0), (2047, 8), (1111, 7), (640, 4)])
def test_tiled_router_equals_oracle_for_every_tile_size(nb, tt, layers, clib, oracle, weights):
    """Batches past the decode sizes take the tiled router kernel; a thread's tile holds 4..8 tokens (tt, 0 = chosen by
    batch size).  Ragged last tiles, every tile size, with and without the selection bias: logits bit for bit."""
    g = layers
    router, _, _ = weights.layer(2)
    hn = weights.hidden(400 + tt, nb)
    bias = np.linspace(-1.0, 1.0, 256).astype(np.float32)
    want = oracle.router_logits(router, hn)
    clib.gmoe_router_tile_tokens(tt)
    try:
        g.poke("hn", hn)
        g.stage("router", 2, nb)
        assert same_bits(g.peek("logits", nb).reshape(nb, 256), want)
        g.poke("bias", bias)
        g.stage("router_bias", 2, nb)
        assert same_bits(g.peek("logits", nb).reshape(nb, 256), want + bias[None, :])
    finally:
        clib.gmoe_router_tile_tokens(0)


def test_compact_down_rows_escape_plane(layers, clib, oracle, weights):
    """The tcgen05 down kernel stores dot + 32768 in 16 bits and the rare |dot| >= 32768 through a 2-bit escape plane.  Down rows
    of all +1 / all -1 against int8 rows of all +-127 give dots of +-65024: both signs of the escape, next to ordinary values;
    the result must equal the register-decode path's and the expected integers, and the plane must be clean afterwards."""
    from maple_runtime_b200 import lib as ml
    g = layers
    router, post_ln, experts = weights.layer(2)
    ex = experts.copy().reshape(256, ml.CONST.EXPERT_BYTES)
    dn = ex[:, 2 * ml.CONST.GU_BYTES:2 * ml.CONST.GU_BYTES + ml.CONST.GU_CODES].reshape(256, 2048, 128)
    dn[:, 0:300, :] = 0xAA        # code 2 everywhere: t = +1
    dn[:, 300:640, :] = 0x00      # code 0 everywhere: t = -1
    dn[:, 1500:1503, :] = 0xAA
    span = ml.page_aligned(ex.nbytes)
    span[:ex.nbytes] = ex.reshape(-1)
    rid = g.region(span)
    g.set_layer(3, router, post_ln, ml.gloc_for_contiguous(0, slot=0), np.array([rid, -1, -1, -1], np.int32))
    nb = 600
    x = weights.hidden(311, nb)
    g.poke("x", x)
    g.set_path(2)
    try:
        for st in ("norm", "router", "topk", "group", "gateup", "actq"):
            g.stage(st, 3, nb)
        aq = g.peek("aq", nb).copy()
        aq[0::3] = 127; aq[1::3] = -127                                   # every third pair keeps its ordinary row
        g.poke("aq", aq); g.poke("aqsum", aq.astype(np.int32).sum(1).astype(np.int32))
        g.stage("down", 3, nb); g.stage("combine_y", 3, nb)
        dots2, down2, y2 = g.peek("dn_dots", nb).copy(), g.peek("down", nb).copy(), g.peek("y", nb).copy()
        g.set_path(1)
        g.stage("down", 3, nb); g.stage("combine_y", 3, nb)
        dots1, down1, y1 = g.peek("dn_dots", nb), g.peek("down", nb), g.peek("y", nb)
        assert dots2.max() == 65024 and dots2.min() == -65024
        assert np.array_equal(dots2, dots1)
        assert same_bits(down2, down1) and same_bits(y2, y1)
        ustart = g.peek("ustart", nb)
        rows = aq[ustart[0]:ustart[1]].astype(np.int64)                    # first used expert: the expected integers of uniform rows
        assert np.array_equal(dots2[ustart[0]:ustart[1]][:, [0, 299, 300, 639, 1501]], np.stack([rows.sum(1), rows.sum(1), -rows.sum(1), -rows.sum(1), rows.sum(1)], 1))
        # the escapes were consumed: an ordinary pass through the same layer equals the oracle again
        g.set_path(2)
        want, _ = oracle.moe(router, post_ln, ex.reshape(-1), x, 1)
        got = x.copy(); g.forward(got, 3, 1)
        assert same_bits(got, want)
    finally:
        g.set_path(0)


@pytest.mark.parametrize("case", list(mg.CASES))
def test_fixtures_from_the_reference(case, layers, clib):
    """The reference's own outputs (tests/golden) without the oracle in between."""
    g = layers
    L, x, norm, bias = mg.make_input(clib, case)
    nb = x.shape[0]
    if norm:
        y = x.copy(); g.forward(y, L, 1, bias)
    else:
        y, _ = g.moe(L, x, bias)
    nu = int(GOLD[f"{case}/nu"][0])
    for k in ("top", "utok", "tp", "hqsum", "aqsum"):
        assert np.array_equal(g.peek(k, nb).ravel(), GOLD[f"{case}/{k}"].ravel()), k
    assert np.array_equal(g.peek("ustart", nb)[:nu + 1], GOLD[f"{case}/ustart"])
    for k in ("hq", "aq", "gate", "up", "act", "down"):
        assert np.array_equal(digest(g.peek(k, nb)), GOLD[f"{case}/{k}_sha"]), k
    assert rel(y[:2], GOLD[f"{case}/y_head"]) <= TOL
    assert np.array_equal(digest(y), GOLD[f"{case}/y_sha"])


@pytest.mark.parametrize("nb,stream,norm,zipf", [(1, 401, 0, False), (5, 402, 1, False), (33, 403, 0, False), (128, 404, 1, False),
                                                  (300, 405, 1, True), (600, 406, 1, False)])
def test_tcgen05_path_all_stages_equal_oracle(nb, stream, norm, zipf, layers, clib, oracle, weights):
    """The tensor-core (tcgen05 kind::i8) grouped kernels forced for every size, including one-token tiles, tiles
    padded to 16 columns, experts split over several 128-token tiles (Zipf bias) and the size where it is the default."""
    from maple_runtime_b200 import lib as ml
    g = layers
    bias = ml.synth_zipf_bias(clib, SEED) if zipf else None
    x = weights.hidden(stream, nb)
    want, d = oracle.moe(*weights.layer(1), x, norm, bias, dots=True)
    g.set_path(2)
    try:
        if norm:
            got = x.copy(); g.forward(got, 1, 1, bias)
        else:
            got, _ = g.moe(1, x, bias)
        check_stages(g, nb, d)
    finally:
        g.set_path(0)
    if zipf:
        assert np.diff(d["ustart"][:int(d["nu"][0]) + 1]).max() > 128
    assert same_bits(got, want), f"rel {rel(got, want):.3e}"


def test_gpre_moe_reference_signature(layers, clib, oracle, weights):
    """The drop-in call of maple.c:763: weights registered as page-aligned host regions, grouping from the host."""
    from maple_runtime_b200 import lib as ml
    g = layers
    router, post_ln, experts = weights.layer(2)
    span = ml.page_aligned(experts.nbytes + 4096)
    span[4096:4096 + experts.nbytes] = experts                           # experts start one page into the region
    rid = g.region(span)
    gloc = ml.gloc_for_contiguous(4096, slot=1)
    regs = np.array([-1, rid, -1, -1], np.int32)
    nb = 48
    x = weights.hidden(301, nb)
    want, d = oracle.moe(router, post_ln, experts, x, 0, dots=True)
    nu = int(d["nu"][0])
    loc = np.ascontiguousarray(gloc[d["ue"][:nu]])
    y, secs = g.gpre_moe(x, nu, loc, regs, d["ustart"], d["utok"], d["uw"], d["tp"])
    assert secs > 0
    assert np.array_equal(g.peek("gu_dots", nb), d["gu_dots"]) and np.array_equal(g.peek("dn_dots", nb), d["dn_dots"])
    assert np.array_equal(g.peek("aq", nb), d["aq"])
    assert same_bits(y, want), f"rel {rel(y, want):.3e}"
    # rejected arguments: -1 and a message, nothing launched
    bad = loc.copy(); bad[0, 1] = span.nbytes
    with pytest.raises(RuntimeError, match="beyond region"):
        g.gpre_moe(x, nu, bad, regs, d["ustart"], d["utok"], d["uw"], d["tp"])
    with pytest.raises(RuntimeError, match="not registered"):
        g.gpre_moe(x, nu, loc, np.array([-1, 63, -1, -1], np.int32), d["ustart"], d["utok"], d["uw"], d["tp"])
    with pytest.raises(RuntimeError, match="page-aligned"):
        g.region(span[1:4097])


def test_gfull_moe_async_form(layers, clib, oracle, weights):
    """gfull_begin -> (norm + router on the card) -> host top-8/grouping -> gfull_moe -> gfull_read (maple.c:1005-1027)."""
    import ctypes as C
    from maple_runtime_b200 import lib as ml
    g = layers
    router, post_ln, experts = weights.layer(1)
    nb = 40
    x = weights.hidden(302, nb)
    want, d = oracle.moe(router, post_ln, experts, x, 1)
    vp = C.c_void_p
    clib.gfull_begin(x.ctypes.data_as(vp), nb, 0)
    logits = np.empty((nb, 256), np.float32)
    assert clib.gmoe_post_norm(1, nb, logits.ctypes.data_as(vp)) == 0
    assert same_bits(logits, d["logits"])
    # host side as maple.c:1015-1019, here through the oracle's statements of job_topk and group_pairs
    top = np.zeros((nb, 8), np.int32); tw = np.zeros((nb, 8), np.float32)
    for b in range(nb):
        top[b], tw[b], _ = oracle.topk(logits[b])
    nu, ue, ustart, utok, uw, tp = oracle.group(top, tw)
    span = ml.page_aligned(experts.nbytes); span[:experts.nbytes] = experts
    rid = g.region(span)
    loc = np.ascontiguousarray(ml.gloc_for_contiguous(0, 0)[ue[:nu]])
    regs = np.array([rid, -1, -1, -1], np.int32)
    clib.gfull_moe(nu, loc.ctypes.data_as(vp), regs.ctypes.data_as(vp), ustart.ctypes.data_as(vp), utok.ctypes.data_as(vp),
                   uw.ctypes.data_as(vp), tp.ctypes.data_as(vp))
    out = np.empty_like(x); ko = vp()
    clib.gfull_read(out.ctypes.data_as(vp), C.byref(ko))
    assert ko.value is None and clib.gfull_maxtok() == 2048
    assert same_bits(out, want), f"rel {rel(out, want):.3e}"


def test_stack_of_layers_and_determinism(layers, oracle, weights):
    """Three layers of residual stream (config 3 in small): equal to the oracle layer after layer, and the same
    bits on a second run."""
    g = layers
    nb = 96
    x0 = weights.hidden(303, nb)
    want = x0.copy()
    for L in range(3):
        want, _ = oracle.moe(*weights.layer(L), want, 1)
    a = x0.copy(); g.forward(a, 0, 3)
    b = x0.copy(); g.forward(b, 0, 3)
    assert same_bits(a, b)
    assert same_bits(a, want), f"rel {rel(a, want):.3e}"


def test_zipf_bias_skewed_load(layers, clib, oracle, weights):
    from maple_runtime_b200 import lib as ml
    g = layers
    nb = 200
    bias = ml.synth_zipf_bias(clib, SEED)
    x = weights.hidden(304, nb)
    want, d = oracle.moe(*weights.layer(0), x, 1, bias, dots=True)
    y = x.copy(); g.forward(y, 0, 1, bias)
    check_stages(g, nb, d)
    cnt = np.diff(d["ustart"][:int(d["nu"][0]) + 1])
    assert cnt.max() > 100                                               # one expert holds most tokens: multi-tile path
    assert same_bits(y, want)


def test_full_chunk_2048_properties(layers, oracle, weights):
    """BASELINE config 3's chunk size on one layer: oracle comparison of the integer stages plus size-independent
    properties (each token in exactly 8 groups, permutation is a bijection, the layer is a function of each token
    alone)."""
    g = layers
    nb = 2048
    x = weights.hidden(305, nb)
    want, d = oracle.moe(*weights.layer(0), x, 1, dots=False)
    y = x.copy(); g.forward(y, 0, 1)
    for k in ("hq", "top", "utok", "tp", "aq"):
        assert np.array_equal(g.peek(k, nb), d[k].reshape(g.peek(k, nb).shape)), k
    assert same_bits(y, want), f"rel {rel(y, want):.3e}"
    tp = g.peek("tp", nb).reshape(nb, 8)
    assert np.array_equal(np.sort(tp.ravel()), np.arange(nb * 8))
    sub = x[1000:1010].copy(); g.forward(sub, 0, 1)
    assert same_bits(sub, y[1000:1010])                                  # tokens do not interact


def test_dense_projections_equal_reference_statement(layers, clib):
    """gpre_dense_add / _done / gpre_dense (gpu_pre.m:200-256): q, k, v in one group, o in another; results bit for bit equal to
    the numpy statement that the CPU suite pins to the reference's tdot.  Ragged token counts, an all-zero token, bad calls."""
    import dense_ref
    g = layers
    rng = np.random.default_rng(23)

    def matrix(rows):
        codes = rng.choice(np.array([0, 1, 2], np.uint8), size=(rows, 2048), p=[0.3, 0.4, 0.3]).reshape(rows, 16, 4, 32)
        packed = np.zeros((rows, 16, 32), np.uint8)
        for k in range(4):
            packed |= (codes[:, :, k, :] << (2 * k)).astype(np.uint8)
        return np.ascontiguousarray(packed.reshape(rows, 512)), rng.uniform(0.01, 0.05, rows).astype(np.float32)
    q, k, v, o = matrix(2048), matrix(512), matrix(512), matrix(2048)
    for m in (q, k, v):
        g.dense_add(0, m[0], m[1], m[0].shape[0], 2048)
    g.dense_add(1, o[0], o[1], 2048, 2048)
    g.dense_done(2048)
    for nb in (1, 33, 300, 512, 700):                                     # from 512 tokens on the tcgen05 kernel takes the group
        x = rng.standard_normal((nb, 2048)).astype(np.float32) * np.float32(3.0)
        if nb > 2:
            x[2] = 0.0
        y, secs = g.dense(0, x, 3072)
        want = np.concatenate([dense_ref.dense(m[0], m[1], m[0].shape[0], 2048, x) for m in (q, k, v)], axis=1)
        assert secs > 0 and same_bits(y, want), f"nb {nb}: rel {rel(y, want):.3e}"
        y1, _ = g.dense(1, x, 2048)
        assert same_bits(y1, dense_ref.dense(o[0], o[1], 2048, 2048, x))
    with pytest.raises(RuntimeError, match="no matrices"):
        g.dense(5, np.zeros((4, 2048), np.float32), 2048)
    # the MoE path still works after the projections used its staging buffers
    xx = np.ascontiguousarray(rng.standard_normal((40, 2048)).astype(np.float32))
    a = xx.copy(); g.forward(a, 0, 1)
    b = xx.copy(); g.forward(b, 0, 1)
    assert same_bits(a, b)


def test_loader_reads_a_converted_directory(layers, clib, weights, tmp_path):
    """gmoe_load_layers walks layout.bin as maple.c:61-81 does and registers per layer and shard one region (maple.c:1106-1131).
    A directory written in the converter's format from the synthetic generator must behave exactly like the same layer
    generated on the device; its q,k,v,o matrices arrive as dense groups."""
    import dense_ref
    from maple_runtime_b200 import synth_dir
    g = layers
    info = synth_dir.write(str(tmp_path), clib, SEED, [1])                  # directory layer 0 = synthetic layer 1 of the fixture
    assert g.lib.gmoe_load_layers(str(tmp_path).encode(), 0, 1, 7, 1) == 0, g.lib.gmoe_load_error()
    for nb in (64, 600):
        x = weights.hidden(320 + nb, nb)
        a = x.copy(); g.forward(a, 1, 1)
        b = x.copy(); g.forward(b, 7, 1)
        assert same_bits(a, b)
    g.dense_done(2048)
    x = weights.hidden(333, 40)
    y, _ = g.dense(14, x, 3072)
    want = np.concatenate([dense_ref.dense(c, s, c.shape[0], 2048, x) for c, s in info["dense"][0][:3]], axis=1)
    assert same_bits(y, want)
    assert g.lib.gmoe_load_layers(str(tmp_path).encode(), 1, 1, 8, 0) == -1 and b"no layer 1" in g.lib.gmoe_load_error()
    assert g.lib.gmoe_load_layers(str(tmp_path / "nowhere").encode(), 0, 1, 8, 0) == -1


def test_single_token_step_order_router(layers, clib, oracle, weights):
    """One token in the order of the reference's `step` (bf_row, maple.c:146-157, 609): logits bit for bit against the oracle's
    statement of that order, which differs from the step_batch order in the last bits; top-8 and weights follow from those logits."""
    g = layers
    router, _, _ = weights.layer(2)
    differ = 0
    try:
        for stream in range(700, 708):
            hn = weights.hidden(stream, 1)
            want_step, want_batch = oracle.router_logits_step(router, hn[0]), oracle.router_logits(router, hn)[0]
            differ += int((want_step.view(np.uint32) != want_batch.view(np.uint32)).sum())
            g.poke("hn", hn)
            clib.gmoe_set_step_order(1)
            g.stage("router", 2, 1)
            assert same_bits(g.peek("logits", 1).reshape(256), want_step)
            g.stage("topk", 2, 1)
            top, w, _ = oracle.topk(want_step)
            assert np.array_equal(g.peek("top", 1).reshape(8), top) and same_bits(g.peek("topw", 1).reshape(8), w)
            clib.gmoe_set_step_order(0)
            g.stage("router", 2, 1)
            assert same_bits(g.peek("logits", 1).reshape(256), want_batch)
    finally:
        clib.gmoe_set_step_order(0)
    assert differ > 0          # the two orders are not the same arithmetic


def test_fast_silu_int8_equals_exact_variant(layers, oracle):
    """The SiLU*up + int8 kernel the timed path runs (hardware exp/reciprocal, exact re-evaluation near the row maximum and near rounding
    boundaries) against the variant that evaluates every element with the libm-equal expf: int8 rows, scales and sums must be the same
    bits, on ordinary values and on rows built to stress the fall-backs; a sample of rows also against the oracle's prep (maple.c:184-194,
    825-832)."""
    g = layers
    nb = 2048; P = nb * 8
    rng = np.random.default_rng(77)
    gate = (rng.standard_normal((P, 512)) * 3.0).astype(np.float32)
    up = (rng.standard_normal((P, 512)) * 2.0).astype(np.float32)
    gate[100:200] *= 10.0                                    # clamped at 7 above, deep negative tails below
    gate[200:260] = -np.abs(gate[200:260]) * 25.0            # exp(-g) up to overflow: act = -0 or denormal
    up[260:300] = 0.0                                        # all-zero rows: scale 1
    gate[300:340] *= 1e-20; up[300:340] *= 1e-18             # tiny rows: the absolute slack takes over
    gate[340:400, :] = gate[340:400, :1]; up[340:400, :] = up[340:400, :1]   # 512 equal values: every element is a maximum candidate
    up[400:500] = np.where(rng.random((100, 512)) < 0.5, 7.5, -7.5)          # clamped |u| = 7, many near-equal maxima
    gate[500:600] = np.float32(7.0) + rng.integers(-3, 4, (100, 512)).astype(np.float32) * np.float32(2.0 ** -20)   # around the clamp
    g.set_path(2)
    try:
        g.poke("gate", gate); g.poke("up", up)
        g.keep_stages(True)
        g.stage("actq", 0, nb)
        want = {k: g.peek(k, nb).copy() for k in ("aq", "aqs", "aqsum", "act")}
        g.poke("aq", np.zeros((P, 512), np.int8))
        g.keep_stages(False)
        g.stage("actq", 0, nb)
        got = {k: g.peek(k, nb) for k in ("aq", "aqs", "aqsum")}
    finally:
        g.keep_stages(True); g.set_path(0)
    bad = np.argwhere(got["aq"] != want["aq"])
    assert bad.size == 0, f"{len(bad)} int8 values differ, first at {bad[:3].tolist()}"
    assert same_bits(got["aqs"], want["aqs"]) and np.array_equal(got["aqsum"], want["aqsum"])
    for a in list(range(601, P, 997)) + [150, 270, 350, 450, 550]:     # the exact variant itself against the oracle's prep of its act row (rows of ordinary magnitude)
        q, qs, qsum = oracle.prep(want["act"][a])
        assert np.array_equal(q, want["aq"][a]) and np.float32(qs).tobytes() == want["aqs"][a].tobytes() and qsum == want["aqsum"][a]


@pytest.mark.parametrize("nb,stream", [(2048, 801), (700, 802)])
def test_timed_path_int8_rows_equal_the_kept_stages_path(nb, stream, layers, oracle, weights):
    """Without kept stages the tcgen05 gate+up kernel stores SiLU(gate) * up evaluated with the hardware's approximate exponential and
    the int8 step computes again, exactly, the elements where that could show (row maximum candidates, values next to a rounding
    boundary).  Its int8 rows, scales and sums must be the bits of the kept-stages path (every element with the libm-equal expf,
    which other tests pin to the oracle), on ordinary tokens and on tokens built to stress the fall-backs: zero rows (512 equal
    products), tiny and huge magnitudes (underflowing products; gate clamped at 7 and up at +-7, exp(-g) up to overflow), repeated
    and negated tokens; a sample of rows also against the oracle's prep (maple.c:184-194, 825-832)."""
    g = layers
    P = nb * 8
    hn = weights.hidden(stream, nb)
    hn[3] = 0.0; hn[40] = 0.0
    hn[50:80] *= np.float32(1e-20); hn[80:100] *= np.float32(1e-30); hn[100:110] *= np.float32(1e-37)
    hn[110:160] *= np.float32(30.0); hn[160:200] *= np.float32(300.0); hn[200:220] *= np.float32(1e6)
    hn[220] = hn[221]; hn[222] = -hn[223]
    hn[230:260, 1:] = 0.0                                   # one non-zero hidden value: dots are +-q or 0, many equal products
    out = {}
    g.set_path(2)
    try:
        g.poke("hn", hn)
        for name in ("prep", "router", "topk", "group"):
            g.stage(name, 0, nb)
        for keep in (True, False):
            g.keep_stages(keep)
            if not keep:
                g.poke("aq", np.zeros((P, 512), np.int8))
            g.stage("gateup", 0, nb); g.stage("actq", 0, nb)
            out[keep] = {k: g.peek(k, nb).copy() for k in (("aq", "aqs", "aqsum", "act") if keep else ("aq", "aqs", "aqsum"))}
    finally:
        g.keep_stages(True); g.set_path(0)
    want, got = out[True], out[False]
    bad = np.argwhere(got["aq"].reshape(P, 512) != want["aq"].reshape(P, 512))
    assert bad.size == 0, f"{len(bad)} int8 values differ, first at {bad[:3].tolist()}"
    assert same_bits(got["aqs"], want["aqs"]) and np.array_equal(got["aqsum"], want["aqsum"])
    act = want["act"].reshape(P, 512)
    for a in range(5, P, 1499):                              # the kept-stages path itself against the oracle's prep of its act row
        if float(np.abs(act[a]).max()) < 1e-30:
            continue
        q, qs, qsum = oracle.prep(act[a])
        assert np.array_equal(q, want["aq"].reshape(P, 512)[a]) and np.float32(qs).tobytes() == want["aqs"].reshape(P)[a].tobytes() and qsum == want["aqsum"].reshape(P)[a]


def test_gpre_moe_page_locks_buffers_it_sees_again(layers, clib, oracle, weights):
    """gpre_moe with the same host arrays call after call (maple.c's HNB and YB) and the page-locking policy on: from the second call on
    they are page-locked in place; the results stay the bits of a call on fresh arrays, with the policy on, off (registrations released)
    and on again."""
    from maple_runtime_b200 import lib as ml
    g = layers
    nb = 640
    x = weights.hidden(831, nb)
    g.forward(x.copy(), 0, 1)
    nu = int(g.peek("nu", nb)[0]); ue = g.peek("ue", nb)[:nu]
    args = (nu, np.ascontiguousarray(ml.gloc_for_contiguous()[ue]), np.array([g.layer_region[0], -1, -1, -1], np.int32), g.peek("ustart", nb)[:nu + 1].copy(),
            g.peek("utok", nb).copy(), g.peek("uw", nb).copy(), g.peek("tp", nb).copy())
    hn = g.peek("hn", nb).copy()
    want, _ = g.gpre_moe(hn.copy(), *args)
    hnb, yb = np.empty_like(hn), np.empty_like(hn)
    try:
        for policy in (1, 0, 1):
            assert clib.gpre_pin_policy(policy) == 0
            for call in range(3):
                hnb[:] = hn; yb[:] = 0
                g.gpre_moe(hnb, *args, out=yb)
                assert same_bits(yb, want), f"policy {policy}, call {call}"
    finally:
        clib.gpre_pin_policy(0)             # releases the registrations before the arrays are freed
