#!/usr/bin/env python3
"""Writes tests/golden/moe_cases.npz by running the REFERENCE ITSELF (oracle/_ref/libmaple_ref.so, i.e. maple.c
compiled from its own sources by oracle/Makefile) on seeded synthetic inputs from the product's host generator.

Run where the reference sources are present:   python tests/golden/make_golden.py
The fixtures pin the oracle restatement (and through it the CUDA path) on machines where the reference is absent.
Large stage tensors are stored as SHA-256 digests, small ones in full.
"""
import hashlib
import os
import sys
import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from maple_runtime_b200 import lib as ml  # noqa: E402
from oracle import oracle as orc          # noqa: E402

SEED = 20261125
# name: (layer, tokens, hidden stream, norm, zipf bias, edit)
CASES = {
    "decode1":   (0, 1, 11, 0, False, None),
    "small5":    (0, 5, 12, 0, False, None),
    "route32":   (1, 32, 13, 1, False, None),      # last size on the job_route_small path (maple.c:734)
    "route33":   (1, 33, 14, 1, False, None),      # first size on the job_route_multi path
    "multi64":   (0, 64, 15, 0, False, None),      # the --multi 64 decode shape
    "zipf40":    (1, 40, 16, 1, True, None),       # skewed routing through a router bias
    "zerotok":   (0, 6, 17, 0, False, "zero"),     # an all-zero token: qs = 1 (maple.c:187), equal logits -> ties
    "twins":     (0, 8, 18, 1, False, "twins"),    # identical tokens share experts: tokens per expert > 1
}
FULL = ("logits", "top", "topw", "nu", "ue", "ustart", "utok", "uw", "tp", "hqs", "hqsum", "aqs", "aqsum")
HASHED = ("hq", "gate", "up", "act", "aq", "down")


def digest(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), np.uint8)


def make_input(clib, case):
    L, nb, stream, norm, zipf, edit = CASES[case]
    x = ml.synth_hidden(clib, SEED, stream, nb)
    if edit == "zero":
        x[2] = 0.0
    if edit == "twins":
        x[4:] = x[:4]
    bias = ml.synth_zipf_bias(clib, SEED, 1.2) if zipf else None
    return L, x, norm, bias


def main():
    clib = ml.load()
    ref = orc.Reference(); ref.threads(min(8, os.cpu_count() or 1))
    out, layers = {}, {}
    for name in CASES:
        L, x, norm, bias = make_input(clib, name)
        if L not in layers:
            layers[L] = (ml.synth_router(clib, SEED, L), ml.synth_norm(clib, SEED, L), ml.synth_experts(clib, SEED, L, 0, 256))
            ref.set_layer(L, *layers[L])
        y, d = ref.moe(L, x, norm, bias)
        nu = int(d["nu"][0])
        d["ue"], d["ustart"] = d["ue"][:nu], d["ustart"][:nu + 1]
        out[f"{name}/x_sha"] = digest(x)
        out[f"{name}/y_sha"] = digest(y)
        out[f"{name}/y_head"] = y[:2].copy()          # two full rows for tolerance checks; the digest pins the rest
        out[f"{name}/logits_sha"] = digest(d["logits"])
        for k in FULL:
            out[f"{name}/{k}"] = d[k][:2].copy() if k == "logits" else d[k]
        for k in HASHED:
            out[f"{name}/{k}_sha"] = digest(d[k])
        print(name, "tokens", x.shape[0], "used experts", nu, "max|y|", float(np.abs(y).max()))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "moe_cases.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
