"""ctypes binding of libgpre_cuda.so: every symbol of include/gpre.h and include/gmoe.h, with numpy helpers.

The argument meaning and error behaviour are the C library's (see the headers); nothing is computed here.
"""
import ctypes as C
import os
import subprocess
import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libgpre_cuda.so")


class CONST:
    H = 2048; FF = 512; NE = 256; TOPK = 8; LAYERS = 24
    GU_CODES = 262144; GU_BYTES = 264192; DN_BYTES = 270336; EXPERT_BYTES = 798720; LAYER_BYTES = 204472320


vp, i32, f64, u64, sz = C.c_void_p, C.c_int, C.c_double, C.c_uint64, C.c_size_t
# name -> (restype, argtypes); the complete export list of the two public headers
DECLS = {
    # include/gpre.h (maple.c:247-272)
    "gpre_init": (i32, [i32, i32]), "gpre_region": (i32, [vp, sz]),
    "gpre_moe": (f64, [vp, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp]),
    "gpre_stage": (i32, [sz]), "gpre_blit_seconds": (f64, []),
    "gfull_moe": (None, [i32, vp, vp, vp, vp, vp, vp]), "gfull_begin": (None, [vp, i32, i32]),
    "gfull_read": (None, [vp, vp]), "gfull_write_x": (None, [vp]), "gfull_maxtok": (i32, []), "gfull_report": (None, []),
    "gfull_init": (i32, [i32, i32, i32, vp, vp, vp]), "gfull_attn": (f64, [i32, i32, vp]),
    "gpre_dense_add": (None, [i32, vp, vp, i32, i32]), "gpre_dense_done": (i32, [i32]), "gpre_dense": (f64, [i32, vp, i32, vp]),
    "gpu_head_init": (i32, [vp, i32, i32]), "gpu_head_init_i8": (i32, [vp, vp, i32, i32]),
    "gpu_head_run": (None, [vp, vp]), "gpu_head_run_multi": (None, [vp, i32, vp]),
    "gpux_init": (i32, [i32, i32]), "gpux_upload": (None, [i32, i32, vp, vp, vp, vp, vp, vp]),
    "gpux_begin": (vp, [i32, vp, i32, vp]), "gpux_end": (None, [vp, vp, i32]),
    "gpux_begin_multi": (vp, [i32, vp, i32, i32, vp, vp, vp]), "gpux_end_multi": (None, [vp, vp, i32]),
    # include/gmoe.h
    "gmoe_init": (i32, [i32]), "gmoe_set_device": (i32, [i32]),
    "gmoe_set_layer": (i32, [i32, vp, vp, vp, vp]), "gmoe_synth_layer": (i32, [u64, i32, i32, i32]),
    "gmoe_moe": (f64, [i32, vp, i32, vp, vp]), "gmoe_forward": (f64, [vp, i32, i32, i32, vp]), "gmoe_forward_submit": (i32, [vp, vp, i32, i32, i32, vp]), "gmoe_forward_wait": (f64, []), "gmoe_forward_mark": (i32, []), "gpre_pin_policy": (i32, [i32]), "gmoe_rope_table": (i32, [vp, i32]), "gmoe_qk_rope": (f64, [vp, vp, i32, i32, vp, vp, vp, vp, vp]),
    "gmoe_x_upload": (i32, [vp, i32]), "gmoe_x_download": (i32, [vp, i32]),
    "gmoe_forward_dev": (i32, [i32, i32, i32, vp]),
    "gmoe_chunks_upload": (i32, [vp, i32, i32]), "gmoe_forward_chunk": (i32, [i32, i32, i32, i32, vp]),
    "gmoe_set_graph": (i32, [i32]), "gmoe_graph_launches": (C.c_long, []), "gmoe_router_tile_tokens": (None, [i32]), "gmoe_profile": (i32, [C.c_uint]), "gmoe_profile_read": (i32, [vp, vp]), "gmoe_sync": (f64, []), "gmoe_post_norm": (i32, [i32, i32, vp]),
    "gmoe_peek": (i32, [C.c_char_p, vp, sz]), "gmoe_poke": (i32, [C.c_char_p, vp, sz]),
    "gmoe_keep_stages": (i32, [i32]), "gmoe_stage": (i32, [C.c_char_p, i32, i32]), "gmoe_set_path": (i32, [i32]), "gmoe_set_router": (i32, [i32]), "gmoe_router_flagged": (i32, []), "gmoe_set_step_order": (i32, [i32]),
    "gmoe_ep_unique_id": (i32, [vp]), "gmoe_ep_init": (i32, [i32, i32, vp]), "gmoe_ep_handles": (i32, [vp]), "gmoe_ep_connect": (i32, [vp]),
    "gmoe_ep_forward_dev": (i32, [i32, i32, i32, i32, vp]), "gmoe_ep_forward": (f64, [vp, i32, i32, i32, vp]),
    "gmoe_ep_allmax": (i32, [vp]), "gmoe_load_layers": (i32, [C.c_char_p, i32, i32, i32, i32]), "gmoe_load_error": (C.c_char_p, []),
    "gmoe_ep_received": (i32, []), "gmoe_ep_timeout_selftest": (i32, [i32]),
    "gmoe_group_noalloc": (i32, [vp, vp, i32, vp, vp, vp, vp, vp, vp, vp]),
    "gmoe_umma_selftest": (i32, [vp, vp, i32, i32, i32, vp]), "gmoe_i8_peak": (f64, [i32, i32]),
    "gmoe_region_read": (i32, [i32, sz, vp, sz]), "gmoe_region_count": (i32, []),
    "gmoe_last_error": (C.c_char_p, []), "gmoe_launch_count": (C.c_long, []),
    "gmoe_pinned_alloc": (vp, [sz]), "gmoe_pinned_free": (None, [vp]), "gmoe_device_info": (i32, [vp, i32, vp, vp]),
    "msynth_expert": (None, [u64, i32, i32, vp]), "msynth_experts": (None, [u64, i32, i32, i32, vp]),
    "msynth_router": (None, [u64, i32, vp]), "msynth_norm": (None, [u64, i32, vp]),
    "msynth_hidden": (None, [u64, u64, i32, vp]), "msynth_zipf_bias": (None, [u64, f64, vp]),
}


def build(verbose=False):
    """Compile csrc/ for sm_100a into libgpre_cuda.so (nvcc cross-compiles without a GPU)."""
    r = subprocess.run(["make", "-C", os.path.join(HERE, "csrc"), "-j8"], capture_output=True, text=True)
    if verbose or r.returncode:
        print(r.stdout[-4000:], r.stderr[-4000:])
    if r.returncode:
        raise RuntimeError("building libgpre_cuda.so failed")
    return LIB_PATH


def load(path=LIB_PATH):
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: build it with maple_runtime_b200.build() (there is no CPU fallback)")
    lib = C.CDLL(path)
    for name, (res, args) in DECLS.items():
        fn = getattr(lib, name)  # AttributeError = a declared symbol is not exported
        fn.restype, fn.argtypes = res, args
    return lib


def _p(a):
    return None if a is None else a.ctypes.data_as(vp)


class Gpre:
    """Convenience wrapper: numpy in, numpy out, exceptions instead of return codes."""
    PEEK = {  # name -> (dtype, elements per token, elements per pair, fixed)
        "x": (np.float32, 2048, 0, 0), "hn": (np.float32, 2048, 0, 0), "y": (np.float32, 2048, 0, 0),
        "hq": (np.int8, 2048, 0, 0), "hqs": (np.float32, 1, 0, 0), "hqsum": (np.int32, 1, 0, 0),
        "logits": (np.float32, 256, 0, 0), "top": (np.int32, 8, 0, 0), "topw": (np.float32, 8, 0, 0),
        "nu": (np.int32, 0, 0, 1), "ue": (np.int32, 0, 0, 256), "ustart": (np.int32, 0, 0, 257),
        "utok": (np.int32, 0, 1, 0), "uw": (np.float32, 0, 1, 0), "tp": (np.int32, 0, 1, 0),
        "gate": (np.float32, 0, 512, 0), "up": (np.float32, 0, 512, 0), "act": (np.float32, 0, 512, 0),
        "aq": (np.int8, 0, 512, 0), "aqs": (np.float32, 0, 1, 0), "aqsum": (np.int32, 0, 1, 0),
        "down": (np.float32, 0, 2048, 0), "gu_dots": (np.int32, 0, 1024, 0), "dn_dots": (np.int32, 0, 2048, 0),
        "bias": (np.float32, 0, 0, 256),
    }

    def __init__(self, maxtok, device=None):
        self.lib = load()
        if device is not None:
            self._chk(self.lib.gmoe_set_device(device))
        self._chk(self.lib.gmoe_init(maxtok))
        self.maxtok = maxtok
        self.layer_region = {}

    def err(self):
        return (self.lib.gmoe_last_error() or b"").decode()

    def _chk(self, rc):
        if rc is None or rc < 0:
            raise RuntimeError(self.err())
        return rc

    # --- weights
    def synth_layer(self, seed, L, e0=0, ne=256):
        self._chk(self.lib.gmoe_synth_layer(seed, L, e0, ne))
        self.layer_region[L] = self.lib.gmoe_region_count() - 1

    STAGES = ("norm_int8", "router", "top8", "grouping", "gate_up", "silu_int8", "down", "combine")

    def profile(self, mask):
        self._chk(self.lib.gmoe_profile(mask))

    def profile_read(self):
        secs = np.zeros(8, np.float64); n = np.zeros(8, np.int64)
        self._chk(self.lib.gmoe_profile_read(_p(secs), _p(n)))
        return secs, n

    def region(self, buf):
        """buf: page-aligned uint8 array whose length is a multiple of the page size."""
        return self._chk(self.lib.gpre_region(_p(buf), buf.nbytes))

    def set_layer(self, L, router, post_ln, gloc, regs):
        self._chk(self.lib.gmoe_set_layer(L, _p(router), _p(post_ln), _p(gloc), _p(regs)))

    # --- attention projections (gpre_dense_*)
    def dense_add(self, g, codes, scales, rows, cols):
        codes = np.ascontiguousarray(codes, np.uint8); scales = np.ascontiguousarray(scales, np.float32)
        self.lib.gpre_dense_add(g, _p(codes), _p(scales), rows, cols)

    def dense_done(self, maxtok):
        return self._chk(self.lib.gpre_dense_done(maxtok))

    def dense(self, g, x, rows):
        nb = x.shape[0]
        y = np.empty((nb, rows), np.float32)
        t = self._chk(self.lib.gpre_dense(g, _p(x), nb, _p(y)))
        return y, t

    # --- compute
    def gpre_moe(self, x, nu, loc, regs, ustart, ptok, pw, tp, out=None):
        nb = x.shape[0]
        y = np.empty((nb, 2048), np.float32) if out is None else out
        t = self.lib.gpre_moe(_p(x), nb, nu, _p(loc), _p(regs), None, _p(ustart), _p(ptok), _p(pw), _p(tp), _p(y))
        self._chk(t)
        return y, t

    def moe(self, L, x, bias=None):
        nb = x.shape[0]
        y = np.empty((nb, 2048), np.float32)
        t = self._chk(self.lib.gmoe_moe(L, _p(x), nb, _p(y), _p(bias)))
        return y, t

    def rope_table(self, cs):
        """cs [positions][32][2] fp32 (cos, sin), as maple.c builds it for gfull_init."""
        cs = np.ascontiguousarray(cs, np.float32)
        self._chk(self.lib.gmoe_rope_table(_p(cs), cs.shape[0]))

    def qk_rope(self, qkv, pos, glob, qn, kn):
        """qkv [nb][3072] fp32, pos [nb] int32, qn/kn [128] fp32 -> q [nb][2048] fp32, kc, vc [nb][512] fp16 bit patterns, seconds."""
        nb = qkv.shape[0]
        q = np.empty((nb, 2048), np.float32); kc = np.empty((nb, 512), np.uint16); vc = np.empty((nb, 512), np.uint16)
        t = self._chk(self.lib.gmoe_qk_rope(_p(np.ascontiguousarray(qkv, np.float32)), _p(np.ascontiguousarray(pos, np.int32)), nb, int(glob),
                                            _p(np.ascontiguousarray(qn, np.float32)), _p(np.ascontiguousarray(kn, np.float32)), _p(q), _p(kc), _p(vc)))
        return q, kc, vc, t

    def forward(self, x, l0, nl, bias=None):
        """x is updated in place; returns GPU seconds."""
        return self._chk(self.lib.gmoe_forward(_p(x), x.shape[0], l0, nl, _p(bias)))

    def stage(self, name, L, nb):
        self._chk(self.lib.gmoe_stage(name.encode(), L, nb))

    def peek(self, name, nb):
        dt, per_tok, per_pair, fixed = self.PEEK[name]
        n = per_tok * nb + per_pair * nb * 8 + fixed
        out = np.empty(n, dt)
        self._chk(self.lib.gmoe_peek(name.encode(), _p(out), out.nbytes))
        if per_tok > 1:
            return out.reshape(nb, per_tok)
        if per_pair > 1:
            return out.reshape(nb * 8, per_pair)
        return out

    def poke(self, name, arr):
        arr = np.ascontiguousarray(arr)
        self._chk(self.lib.gmoe_poke(name.encode(), _p(arr), arr.nbytes))

    def set_path(self, path):
        """0 = by size, 1 = register-decode mma.sync kernels, 2 = tcgen05 kernels."""
        self._chk(self.lib.gmoe_set_path(path))

    def set_router(self, mode):
        """0 = by size (tensor cores from 512 tokens on), 1 = exact-order kernels always, 2 = tensor cores always."""
        self._chk(self.lib.gmoe_set_router(mode))

    def keep_stages(self, keep=True):
        self._chk(self.lib.gmoe_keep_stages(int(keep)))


# --- host-side synthetic workload (no GPU needed) ----------------------------------------------------------------
def synth_experts(lib, seed, L, e0, ne):
    buf = np.empty(ne * CONST.EXPERT_BYTES, np.uint8)
    lib.msynth_experts(seed, L, e0, ne, _p(buf))
    return buf


def synth_router(lib, seed, L):
    r = np.empty((256, 2048), np.uint16)
    lib.msynth_router(seed, L, _p(r))
    return r


def synth_norm(lib, seed, L):
    w = np.empty(2048, np.uint16)
    lib.msynth_norm(seed, L, _p(w))
    return w


def synth_hidden(lib, seed, stream, nb):
    x = np.empty((nb, 2048), np.float32)
    lib.msynth_hidden(seed, stream, nb, _p(x))
    return x


def synth_zipf_bias(lib, seed, s=1.2):
    b = np.empty(256, np.float32)
    lib.msynth_zipf_bias(seed, s, _p(b))
    return b


def page_aligned(nbytes):
    """A zeroed uint8 array whose address and length are multiples of the page size (what gpre_region demands)."""
    pg = os.sysconf("SC_PAGE_SIZE")
    n = (nbytes + pg - 1) // pg * pg
    raw = np.zeros(n + pg, np.uint8)
    off = (-raw.ctypes.data) % pg
    return raw[off:off + n]


def gloc_for_contiguous(e0_offset=0, slot=0):
    """GLOC-style table [256][12] for 256 experts stored back to back (converter order) from byte e0_offset."""
    g = np.zeros((256, 12), np.uint32)
    for e in range(256):
        b = e0_offset + e * CONST.EXPERT_BYTES
        offs = [b, b + CONST.GU_CODES, b + CONST.GU_BYTES, b + CONST.GU_BYTES + CONST.GU_CODES,
                b + 2 * CONST.GU_BYTES, b + 2 * CONST.GU_BYTES + CONST.GU_CODES]
        for m in range(6):
            g[e, 2 * m] = slot
            g[e, 2 * m + 1] = offs[m]
    return g
