"""CPU tests of the oracle: against the fixtures the reference itself produced (tests/golden/), against the
reference compiled here when present (oracle/_ref), and against independent numpy statements of the layout."""
import hashlib
import os
import sys
import numpy as np
import pytest

from conftest import SEED, same_bits

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden as mg  # noqa: E402

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "moe_cases.npz"))


def digest(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), np.uint8)


@pytest.mark.parametrize("case", list(mg.CASES))
def test_oracle_matches_reference_fixtures(case, clib, oracle, weights):
    """Every stage of the restatement equals what maple.c produced for the same seeded input: bit for bit."""
    L, x, norm, bias = mg.make_input(clib, case)
    assert np.array_equal(digest(x), GOLD[f"{case}/x_sha"]), "the synthetic input generator changed"
    router, post_ln, experts = weights.layer(L)
    y, d = oracle.moe(router, post_ln, experts, x, norm, bias)
    nu = int(d["nu"][0])
    d["ue"], d["ustart"] = d["ue"][:nu], d["ustart"][:nu + 1]
    for k in mg.FULL:
        want = GOLD[f"{case}/{k}"]
        got = d[k][:2] if k == "logits" else d[k]
        assert same_bits(got, want), k
    assert np.array_equal(digest(d["logits"]), GOLD[f"{case}/logits_sha"])
    for k in mg.HASHED:
        assert np.array_equal(digest(d[k]), GOLD[f"{case}/{k}_sha"]), k
    assert same_bits(y[:2], GOLD[f"{case}/y_head"])
    assert np.array_equal(digest(y), GOLD[f"{case}/y_sha"])


@pytest.mark.parametrize("nb,norm,stream", [(1, 0, 101), (7, 1, 102), (32, 0, 103), (33, 1, 104), (128, 1, 105)])
def test_oracle_matches_reference_live(nb, norm, stream, clib, oracle, reference, weights):
    """Same comparison on fresh inputs against the reference compiled on this machine (config 1 is nb = 128)."""
    router, post_ln, experts = weights.layer(2)
    reference.set_layer(2, router, post_ln, experts)
    x = weights.hidden(stream, nb)
    yo, do = oracle.moe(router, post_ln, experts, x, norm)
    yr, dr = reference.moe(2, x, norm)
    nu = int(dr["nu"][0])
    assert int(do["nu"][0]) == nu
    for k in dr:
        a, b = do[k], dr[k]
        if k == "ue":
            a, b = a[:nu], b[:nu]
        if k == "ustart":
            a, b = a[:nu + 1], b[:nu + 1]
        assert same_bits(a, b), k
    assert same_bits(yo, yr)


def test_expf_model_equals_libm(oracle):
    """The exponential the kernels evaluate is libm's, bit for bit: every float in [2^-20, 16] and its negative
    (the softmax and SiLU arguments live here), and a stride through the rest of [-104, 89]."""
    import ctypes as C
    f = oracle.lib.orc_expf_check
    f.restype = C.c_long; f.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32]
    lo = np.array([2.0 ** -20, 16.0, 89.5], np.float32).view(np.uint32)
    assert f(int(lo[0]), int(lo[1]), 1) == 0
    assert f(0, int(lo[2]), 997) == 0
    assert f(int(lo[2]), 0x7F800000, 65521) == 0          # overflow to inf / underflow to 0 beyond the range


def test_packed_layout_matches_converter_statement(clib, oracle, weights):
    """orc_dot against a numpy statement of the converter's layout (convert.py:29-33, 36-40): byte j of a
    128-column group holds columns j, j+32, j+64, j+96."""
    import ctypes as C
    _, _, experts = weights.layer(0)
    rng = np.random.default_rng(5)
    for cols, off in ((2048, 0), (512, 2 * 264192)):
        row = experts[off + 3 * (cols // 4): off + 4 * (cols // 4)]
        p = row.reshape(cols // 128, 32)
        codes = np.stack([(p >> sh) & 3 for sh in (0, 2, 4, 6)], axis=1).reshape(cols).astype(np.int64)
        q = rng.integers(-127, 128, cols).astype(np.int8)
        want = int((codes * q.astype(np.int64)).sum())
        got = oracle.lib.orc_dot(row.ctypes.data_as(C.c_void_p), cols, q.ctypes.data_as(C.c_void_p))
        assert got == want
        # pack(unpack) round trip restates pack_ternary
        g = codes.reshape(cols // 128, 4, 32)
        packed = (g[:, 0] | (g[:, 1] << 2) | (g[:, 2] << 4) | (g[:, 3] << 6)).astype(np.uint8).reshape(-1)
        assert np.array_equal(packed, row)


def test_prep_edge_cases(oracle):
    z = np.zeros(2048, np.float32)
    q, qs, qsum = oracle.prep(z)
    assert qs == 1.0 and qsum == 0 and not q.any()                      # maple.c:187: all-zero vector -> scale 1
    x = np.zeros(512, np.float32); x[3] = -5.0; x[7] = 2.5; x[9] = 5.0 * 0.5 / 127
    q, qs, qsum = oracle.prep(x)
    assert q[3] == -127 and q[7] == 64 and q[9] in (0, 1) and qs == np.float32(5.0) / np.float32(127.0)
    assert q[7] == 64                                                    # 63.5 rounds to even (lrintf)


def test_topk_ties_take_lowest_index(oracle):
    lg = np.full(256, -3.0, np.float32)
    lg[[200, 17, 90]] = 1.0
    top, w, _ = oracle.topk(lg)
    assert list(top[:3]) == [17, 90, 200]                                # equal probabilities: first maximum wins
    assert list(top[3:]) == [0, 1, 2, 3, 4]
    assert abs(float(w.sum()) - 1.0) < 1e-6


def test_group_properties(oracle):
    rng = np.random.default_rng(3)
    nb = 77
    top = np.stack([rng.choice(256, 8, replace=False) for _ in range(nb)]).astype(np.int32)
    tw = rng.random((nb, 8)).astype(np.float32)
    nu, ue, ustart, utok, uw, tp = oracle.group(top, tw)
    assert ustart[nu] == nb * 8 and np.all(np.diff(ue[:nu]) > 0)
    for u in range(nu):
        seg = utok[ustart[u]:ustart[u + 1]]
        assert np.all(np.diff(seg) > 0)                                   # token order inside an expert
        for a in range(ustart[u], ustart[u + 1]):
            s = list(top[utok[a]]).index(ue[u]); assert uw[a] == tw[utok[a], s]
    t = tp.reshape(nb, 8)
    assert np.all(np.diff(t, axis=1) > 0) and np.array_equal(np.sort(t.ravel()), np.arange(nb * 8))
    assert all(utok[a] == b for b in range(nb) for a in t[b])


def test_dense_projection_statement_equals_reference_tdot(reference):
    """The numpy statement the GPU dense projections are tested against equals the compiled reference's prep + tdot."""
    import ctypes as C
    import dense_ref
    rng = np.random.default_rng(11)
    rows, cols, nb = 256, 2048, 5
    codes = rng.choice(np.array([0, 1, 2], np.uint8), size=(rows, cols), p=[0.3, 0.4, 0.3])
    packed = np.zeros((rows, cols // 128, 32), np.uint8)
    g = codes.reshape(rows, cols // 128, 4, 32)
    for k in range(4):
        packed |= (g[:, :, k, :] << (2 * k)).astype(np.uint8)
    packed = np.ascontiguousarray(packed.reshape(rows, cols // 4))
    scales = rng.uniform(0.01, 0.05, rows).astype(np.float32)
    x = rng.standard_normal((nb, cols)).astype(np.float32)
    x[3] = 0.0                                                            # the all-zero vector: qs = 1
    want = dense_ref.dense(packed, scales, rows, cols, x)
    lib = reference.lib
    lib.rh_tdot.restype = C.c_float
    lib.rh_tdot.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    for b in range(nb):
        xb = np.ascontiguousarray(x[b])
        for r in (0, 1, 17, 128, 255):
            got = np.float32(lib.rh_tdot(packed.ctypes.data, scales.ctypes.data, rows, cols, r, xb.ctypes.data))
            assert got.tobytes() == want[b, r].tobytes(), (b, r, got, want[b, r])


def attention_head_case(seed, nb):
    """q, k, v rows of ordinary magnitude plus rows that stress the fp16 conversion (overflow, subnormals, ties), norm weights near 1
    (bf16), positions over the whole table including 0."""
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((nb, 2048)).astype(np.float32); k = rng.standard_normal((nb, 512)).astype(np.float32)
    v = rng.standard_normal((nb, 512)).astype(np.float32)
    if nb > 4:
        v[1] *= np.float32(1e5); v[2] *= np.float32(1e-6); v[3, ::2] = np.float32(2049.0); v[3, 1::2] = np.float32(6.0e-8)    # inf, subnormal halves, ties
        k[2] *= np.float32(300.0); q[3] = 0.0
    qn = ((rng.standard_normal(128) * 0.1 + 1).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    kn = ((rng.standard_normal(128) * 0.1 + 1).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    pos = rng.integers(0, 4096, nb).astype(np.int32); pos[0] = 0
    return q, k, v, qn, kn, pos


@pytest.mark.parametrize("nb,glob,seed", [(1, 0, 41), (33, 0, 42), (33, 1, 43), (257, 0, 44)])
def test_attention_head_restatement_equals_the_reference(nb, glob, seed, oracle, reference):
    """q/k RMS norm, half-rotary embedding and the fp16 cache rows (maple.c:711-717): the restatement against the compiled reference, bit
    for bit, fp32 and fp16 outputs; the rotation's fused multiply-add forms are the ones the reference's compiler chose."""
    q, k, v, qn, kn, pos = attention_head_case(seed, nb)
    cs = reference.rope_table(4096)
    want = reference.qk_rope(q, k, v, qn, kn, pos, glob)
    got = oracle.qk_rope(q, k, v, qn, kn, pos, cs, glob)
    for name, a, b in zip(("q", "k", "kc", "vc"), got, want):
        assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), name
    # the fp16 conversion itself against numpy's round-to-nearest-even
    with np.errstate(over="ignore"):
        assert np.array_equal(got[3], v.astype(np.float16).view(np.uint16))
