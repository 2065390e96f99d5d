"""ctypes loaders for the test oracle: the CPU restatement (liboracle.so) and, when built, the reference itself
(oracle/_ref/libmaple_ref*.so).  TEST INFRASTRUCTURE: only tests/, the smoke check and the CPU-baseline legs of
bench.py may import this module."""
import ctypes as C
import os
import subprocess
import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
vp = C.c_void_p
H, FF, NE, TOPK, EXPERT_BYTES = 2048, 512, 256, 8, 798720


def build():
    r = subprocess.run(["make", "-C", HERE], capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError("building the oracle failed:\n" + r.stdout[-2000:] + r.stderr[-2000:])


def _p(a):
    return None if a is None else a.ctypes.data_as(vp)


class Dump(C.Structure):
    _fields_ = [(n, vp) for n in ("logits", "top", "topw", "nu", "ue", "ustart", "utok", "uw", "tp", "hq", "hqs", "hqsum",
                                  "gate", "up", "act", "aq", "aqs", "aqsum", "down", "gu_dots", "dn_dots")]


def alloc_dump(nb, dots=False):
    np_ = nb * TOPK
    d = dict(logits=np.zeros((nb, NE), np.float32), top=np.zeros((nb, TOPK), np.int32), topw=np.zeros((nb, TOPK), np.float32),
             nu=np.zeros(1, np.int32), ue=np.zeros(NE, np.int32), ustart=np.zeros(NE + 1, np.int32),
             utok=np.zeros(np_, np.int32), uw=np.zeros(np_, np.float32), tp=np.zeros(np_, np.int32),
             hq=np.zeros((nb, H), np.int8), hqs=np.zeros(nb, np.float32), hqsum=np.zeros(nb, np.int32),
             gate=np.zeros((np_, FF), np.float32), up=np.zeros((np_, FF), np.float32), act=np.zeros((np_, FF), np.float32),
             aq=np.zeros((np_, FF), np.int8), aqs=np.zeros(np_, np.float32), aqsum=np.zeros(np_, np.int32),
             down=np.zeros((np_, H), np.float32))
    if dots:
        d["gu_dots"] = np.zeros((np_, 2 * FF), np.int32)
        d["dn_dots"] = np.zeros((np_, H), np.int32)
    s = Dump()
    for k, _ in Dump._fields_:
        setattr(s, k, _p(d.get(k)))
    return d, s


class Oracle:
    """The CPU restatement (moe_oracle.c)."""

    def __init__(self):
        path = os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        self.lib = L = C.CDLL(path)
        L.orc_expf_model.restype = C.c_float; L.orc_expf_model.argtypes = [C.c_float]
        L.orc_dot.restype = C.c_int32; L.orc_dot.argtypes = [vp, C.c_int, vp]
        L.orc_moe.restype = C.c_int
        L.orc_moe.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int, vp, vp, C.POINTER(Dump)]
        L.orc_threads.restype = C.c_int; L.orc_threads.argtypes = [C.c_int]

    def moe(self, router, post_ln, experts, x, norm, bias=None, dump=True, dots=False):
        """Returns (y_or_x, dump dict). norm: x is the residual stream (updated copy returned); else normalised input."""
        nb = x.shape[0]
        x = np.array(x, np.float32, copy=True)
        y = np.zeros((nb, H), np.float32)
        d, s = alloc_dump(nb, dots) if dump else ({}, None)
        rc = self.lib.orc_moe(_p(router), _p(post_ln), _p(experts), _p(x), nb, int(norm), _p(y), _p(bias), C.byref(s) if dump else None)
        assert rc == nb * TOPK
        return (x if norm else y), d

    def prep(self, x):
        n = x.shape[-1]; q = np.zeros(n, np.int8); qs = C.c_float(); qsum = C.c_int32()
        self.lib.orc_prep(_p(x), n, _p(q), C.byref(qs), C.byref(qsum))
        return q, qs.value, qsum.value

    def rmsnorm(self, x, w):
        out = np.zeros_like(x); self.lib.orc_rmsnorm(_p(out), _p(x), _p(w), x.shape[-1]); return out

    def qk_rope(self, q, k, v, qn, kn, pos, cs, glob):
        """maple.c:711-717 on copies: returns q (fp32), k (fp32), kc, vc (fp16 bit patterns)."""
        nb = q.shape[0]
        q = np.array(q, np.float32, copy=True); k = np.array(k, np.float32, copy=True)
        kc = np.zeros((nb, 512), np.uint16); vc = np.zeros((nb, 512), np.uint16)
        self.lib.orc_qk_rope(_p(q), _p(k), _p(np.ascontiguousarray(v, np.float32)), _p(qn), _p(kn), _p(np.ascontiguousarray(pos, np.int32)), _p(cs), nb, int(glob), _p(kc), _p(vc))
        return q, k, kc, vc

    def router_logits(self, router, hn):
        nb = hn.shape[0]; out = np.zeros((nb, NE), np.float32)
        self.lib.orc_router_logits(_p(router), _p(hn), nb, _p(out)); return out

    def router_logits_step(self, router, hn_row):
        """bf_row order (maple.c:146-157), one token."""
        out = np.zeros(NE, np.float32)
        self.lib.orc_router_logits_step(_p(router), _p(np.ascontiguousarray(hn_row, np.float32)), _p(out)); return out

    def topk(self, logits_row):
        lg = np.array(logits_row, np.float32, copy=True); top = np.zeros(TOPK, np.int32); w = np.zeros(TOPK, np.float32)
        self.lib.orc_topk(_p(lg), _p(top), _p(w)); return top, w, lg

    def group(self, top, tw):
        nb = top.shape[0]; np_ = nb * TOPK
        nu = C.c_int(); ue = np.zeros(NE, np.int32); ustart = np.zeros(NE + 1, np.int32)
        utok = np.zeros(np_, np.int32); uw = np.zeros(np_, np.float32); tp = np.zeros(np_, np.int32)
        self.lib.orc_group(_p(np.ascontiguousarray(top, np.int32)), _p(np.ascontiguousarray(tw, np.float32)), nb, C.byref(nu), _p(ue), _p(ustart), _p(utok), _p(uw), _p(tp))
        return nu.value, ue, ustart, utok, uw, tp


class Reference:
    """The reference's own maple.c, compiled from its sources by oracle/Makefile (absent where those are absent)."""

    def __init__(self, fast=False):
        path = os.path.join(HERE, "_ref", "libmaple_ref_fast.so" if fast else "libmaple_ref.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = L = C.CDLL(path)
        L.rh_threads.restype = C.c_int; L.rh_threads.argtypes = [C.c_int]
        L.rh_set_layer.argtypes = [C.c_int, vp, vp, vp]
        L.rh_moe.restype = C.c_int; L.rh_moe.argtypes = [C.c_int, vp, C.c_int, C.c_int, vp, vp, C.POINTER(Dump)]
        L.rh_stack.restype = C.c_double; L.rh_stack.argtypes = [vp, C.c_int, C.c_int, C.c_int, vp]
        L.rh_expf.restype = C.c_float; L.rh_expf.argtypes = [C.c_float]
        L.rh_tdot.restype = C.c_float; L.rh_tdot.argtypes = [vp, vp, C.c_int, C.c_int, C.c_int, vp]
        self._keep = {}
        L.rh_threads(1)   # maple.c starts with NT = 4 and no workers running: without this its run() would wait for threads that do not exist

    @staticmethod
    def available(fast=False):
        return os.path.exists(os.path.join(HERE, "_ref", "libmaple_ref_fast.so" if fast else "libmaple_ref.so"))

    def threads(self, n):
        return self.lib.rh_threads(n)

    def set_layer(self, L, router, post_ln, experts):
        self._keep[L] = (router, post_ln, experts)  # the reference keeps raw pointers
        self.lib.rh_set_layer(L, _p(router), _p(post_ln), _p(experts))

    def moe(self, L, x, norm, bias=None):
        nb = x.shape[0]
        x = np.array(x, np.float32, copy=True); y = np.zeros((nb, H), np.float32)
        d, s = alloc_dump(nb)
        rc = self.lib.rh_moe(L, _p(x), nb, int(norm), _p(y), _p(bias), C.byref(s))
        assert rc == nb * TOPK, rc
        return (x if norm else y), d

    def qk_rope(self, q, k, v, qn, kn, pos, glob):
        """rmsnorm + rope + to_f16 as step_batch calls them (maple.c:711-717), on copies."""
        nb = q.shape[0]
        q = np.array(q, np.float32, copy=True); k = np.array(k, np.float32, copy=True)
        kc = np.zeros((nb, 512), np.uint16); vc = np.zeros((nb, 512), np.uint16)
        self.lib.rh_qk_rope(_p(q), _p(k), _p(np.ascontiguousarray(v, np.float32)), _p(qn), _p(kn), _p(np.ascontiguousarray(pos, np.int32)), nb, int(glob), _p(kc), _p(vc))
        return q, k, kc, vc

    def rope_table(self, positions):
        """The (cos, sin) table maple.c builds for gfull_init (maple.c:1151-1153)."""
        cs = np.zeros((positions, 32, 2), np.float32); self.lib.rh_rope_table(_p(cs), positions); return cs

    def stack(self, x, l0, nl, bias=None):
        """x updated in place; seconds on the reference's own clock."""
        return self.lib.rh_stack(_p(x), x.shape[0], l0, nl, _p(bias))
