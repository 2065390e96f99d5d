"""The C-ABI library loads without a GPU, exports every symbol the public headers declare, and refuses to compute
without a device (no CPU fallback)."""
import ctypes as C
import os
import re
import subprocess
import numpy as np
import pytest

from conftest import ROOT, SEED


def header_functions():
    names = []
    for h in ("gpre.h", "gmoe.h"):
        src = open(os.path.join(ROOT, "include", h)).read()
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        names += re.findall(r"\b(g(?:pre|full|moe|pu_head|pux)_\w+|msynth_\w+)\s*\(", src)
    return sorted(set(names))


def test_every_declared_symbol_is_exported_and_bound(clib):
    from maple_runtime_b200 import lib as ml
    names = header_functions()
    assert len(names) >= 45
    for n in names:
        assert hasattr(clib, n), f"{n} declared in include/ but not exported"
        assert n in ml.DECLS, f"{n} has no ctypes prototype"
    assert set(ml.DECLS) == set(names)


def test_reference_abi_names_present(clib):
    # the undefined symbols of maple.c built with -DGPU_HEAD (maple.c:247-272)
    for n in ("gpre_init gpre_region gpre_moe gpre_stage gpre_dense_add gpre_dense_done gpre_dense gpre_blit_seconds "
              "gfull_init gfull_begin gfull_attn gfull_moe gfull_read gfull_write_x gfull_maxtok gfull_report "
              "gpu_head_init gpu_head_init_i8 gpu_head_run gpu_head_run_multi gpux_init gpux_upload gpux_begin gpux_end "
              "gpux_begin_multi gpux_end_multi").split():
        assert hasattr(clib, n)


def test_out_of_scope_plugins_report_unavailable(clib):
    assert clib.gpu_head_init(None, 1, 1) == -1 and clib.gpux_init(24, 32) == -1
    assert clib.gfull_init(4096, 128, 512, None, None, None) == -1
    assert clib.gpre_dense_done(128) == -1          # before gpre_init (and on a machine without a GPU): the projections stay on the CPU


@pytest.mark.skipif(os.path.exists("/dev/nvidiactl"), reason="needs a machine without a GPU")
def test_no_cpu_fallback(clib):
    assert clib.gpre_init(128, 8) == -1
    assert b"no CUDA device" in clib.gmoe_last_error() or b"gpre" in clib.gmoe_last_error()
    x = np.zeros((1, 2048), np.float32)
    assert clib.gmoe_moe(0, x.ctypes.data_as(C.c_void_p), 1, x.ctypes.data_as(C.c_void_p), None) < 0


def test_argument_checks_before_any_device_work(clib):
    assert clib.gpre_init(128, 4) == -1 and b"topk" in clib.gmoe_last_error()
    assert clib.gpre_init(0, 8) == -1 and clib.gpre_init(1 << 20, 8) == -1


MAPLE_C = os.environ.get("MAPLE_C", "/root/reference/maple.c")   # the reference's single source file, where this machine keeps it


@pytest.mark.skipif(not os.path.exists(MAPLE_C), reason="reference sources not on this machine")
def test_reference_links_against_the_library(tmp_path):
    """maple.c built with -DGPU_HEAD resolves every plug-in symbol from libgpre_cuda.so (link check only)."""
    from maple_runtime_b200 import lib as ml
    exe = tmp_path / "maple_gpu"
    r = subprocess.run(["gcc", "-w", "-O1", "-march=x86-64-v3", "-DGPU_HEAD", "-o", str(exe), MAPLE_C,
                        ml.LIB_PATH, "-lpthread", "-lm", "-Wl,-rpath," + os.path.dirname(ml.LIB_PATH)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]


def test_host_generator_layout(clib, weights):
    from maple_runtime_b200 import lib as ml
    router, post_ln, experts = weights.layer(0)
    assert experts.nbytes == ml.CONST.LAYER_BYTES
    e = experts[5 * ml.CONST.EXPERT_BYTES:6 * ml.CONST.EXPERT_BYTES]
    codes = e[:ml.CONST.GU_CODES]
    c4 = np.stack([(codes >> s) & 3 for s in (0, 2, 4, 6)])
    assert c4.max() == 2                                                 # 3 never appears: ternary
    frac = np.bincount(c4.ravel(), minlength=3) / c4.size
    assert np.allclose(frac, [0.3, 0.4, 0.3], atol=0.005)
    for off, n in ((ml.CONST.GU_CODES, 512), (ml.CONST.GU_BYTES + ml.CONST.GU_CODES, 512), (2 * ml.CONST.GU_BYTES + ml.CONST.GU_CODES, 2048)):
        s = np.frombuffer(e[off:off + 4 * n].tobytes(), np.float32)
        assert s.min() >= 0.01 and s.max() <= 0.05 and 0.028 < s.mean() < 0.032
    one = np.empty(ml.CONST.EXPERT_BYTES, np.uint8); clib.msynth_expert(SEED, 0, 5, one.ctypes.data_as(C.c_void_p))
    assert np.array_equal(one, e)                                        # any slice can be regenerated alone
    r = (router.astype(np.uint32) << 16).view(np.float32)
    assert abs(float(r.std()) * np.sqrt(2048) - 1.0) < 0.02 and np.all(post_ln == 0x3F80)
    b = ml.synth_zipf_bias(clib, SEED)
    p = np.exp(np.sort(b.astype(np.float64))[::-1]) / 256
    assert abs(p.sum() - 1) < 1e-5 and abs(np.log(p[0] / p[1]) - 1.2 * np.log(2)) < 1e-4


def test_loader_rejects_what_it_cannot_read(clib, tmp_path):
    import ctypes as C
    clib.gmoe_load_error.restype = C.c_char_p
    assert clib.gmoe_load_layers(str(tmp_path / "nowhere").encode(), 0, 1, 0, 0) == -1
    assert b"layout.bin" in clib.gmoe_load_error()
    (tmp_path / "layout.bin").write_bytes(b"\0" * 100)                      # shorter than one layer's records
    assert clib.gmoe_load_layers(str(tmp_path).encode(), 0, 1, 0, 0) == -1
    assert b"no layer 0" in clib.gmoe_load_error()
    assert clib.gmoe_load_layers(str(tmp_path).encode(), 0, 1, 24, 0) == -1    # layer index outside the library's 24


def test_synthetic_directory_has_the_converters_record_order(clib, tmp_path):
    import struct
    from maple_runtime_b200 import synth_dir, lib as ml
    synth_dir.write(str(tmp_path), clib, 7, [3])
    raw = (tmp_path / "layout.bin").read_bytes()
    recs = [struct.unpack_from("<BBQQII", raw, 26 * i) for i in range(len(raw) // 26)]
    assert len(recs) == 3 + 5 + 4 + 3 * 256
    assert [chr(r[0]) for r in recs[:8]] == list("bbbbbbbb") and all(chr(r[0]) == "t" for r in recs[8:])
    assert recs[7][4:] == (256, 2048)                                       # the router
    assert recs[12][4:] == (512, 2048) and recs[14][4:] == (2048, 512)      # expert 0: gate, down
    k, off = recs[12][1], recs[12][2]
    shard = (tmp_path / f"shard-{k + 1:05d}.bin").read_bytes()
    want = np.asarray(ml.synth_experts(clib, 7, 3, 0, 1), np.uint8)
    assert shard[off:off + 1024] == want[:1024].tobytes() and off % 16 == 0
