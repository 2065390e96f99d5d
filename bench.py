#!/usr/bin/env python3
"""bench.py -- Maple MoE prefill throughput on B200: a 24-layer stack of mixture-of-experts blocks
(d=2048, 256 ternary experts 512/2048, top-8) over 2048-token chunks of synthetic hidden states.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one 2048-token chunk through all 24 layers on each GPU.  `value` is tokens/s with the chunk already in
HBM (device-timed, max over ranks); `e2e` is the same through the host-buffer entry points (pinned host
input copied in, result copied out, inside the timed region): gmoe_forward_submit / gmoe_forward_wait with two chunks outstanding,
and the waiting call gmoe_forward beside it (`e2e.waiting_call`).  `roofline` describes the dominant kernel (the grouped
gate+up GEMM), timed with CUDA events around its launches in a pass of its own: its algorithmic bytes against the measured copy
bandwidth (the roof that binds at 64 pairs per expert), and its integer operations against the tcgen05 kind::i8 rate measured on
this GPU in the same run (`roofline.tensor`).  `e2e_gpre_moe` is the same chunk through 24 calls of the reference-signature gpre_moe (host
grouping tables, host buffers: the call an unmodified maple.c makes).  `parity_check` compares two layers of the chunk with
the reference (oracle/_ref) before anything is timed.  `cpu_baseline` times the reference's own CPU code on a bounded sample
on this host; `--impl reference` runs that code over the whole 24-layer stack.  `decode` repeats the measurement for the
64-conversation decode shape (HBM-bound).  Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED = 20261125
NB, LAYERS, H = 2048, 24, 2048
EXPERT_BYTES = 798720
OPS_PER_PAIR = 2 * (2 * 512 * 2048 + 2048 * 512)        # int8 multiply-adds x2 of one (token, expert) pair: 6,291,456
GU_OPS_PER_PAIR = 2 * 2 * 512 * 2048                     # the gate+up share: 4,194,304
METRIC, UNIT = "moe_prefill_tokens_per_s_2048tok_chunk_24_layers", "tokens/s"


def profiled_traffic(name):
    """DRAM bytes per launch of a kernel as the ncu summary under profiles/ records it (a line `dram_bytes_per_launch <name>: <bytes>`)."""
    import glob, re
    for f in sorted(glob.glob(os.path.join(ROOT, "profiles", "*.md"))):
        m = re.search(r"dram_bytes_per_launch " + re.escape(name) + r":\s*([0-9.eE+]+)", open(f).read())
        if m:
            return float(m.group(1)), os.path.basename(f)
    return None, None


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "src": "fallback"}


class ClockSampler(threading.Thread):
    """nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.rows, self.stop_flag = index, [], False

    def run(self):
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            time.sleep(0.1)

    def summary(self):
        self.stop_flag = True
        self.join(timeout=6)
        sm = [float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [s for s in sm if s > 0]
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": float(self.rows[0][1]) if self.rows else None,
                "reasons": sorted(reasons), "samples": len(self.rows)}


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def init_dist(world):
    if world == 1:
        return None
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("gloo")   # plumbing only: hands the NCCL id and the CUDA IPC handles to the ranks, host barriers
    return dist


def gather_obj(dist):
    def f(obj):
        out = [None] * dist.get_world_size()
        dist.all_gather_object(out, obj)
        return out
    return f


def allmax(dist, v):
    if dist is None:
        return v
    import torch
    t = torch.tensor([v], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def barrier(dist):
    if dist is not None:
        dist.barrier()


# ---------------------------------------------------------------------------------------------------------------
def cpu_reference_arm(steps, warmup, nlay, budget_s=None):
    """The reference's CPU path (maple.c through oracle/_ref, documented -ffast-math build) on this host's cores: a step = one
    2048-token chunk through nlay distinct layers, router to combine (rh_stack).  nlay = 24 is the whole workload; a smaller nlay is
    a bounded sample whose time is scaled to 24 layers.  budget_s stops the loop early (the baseline leg inside the GPU arm)."""
    from maple_runtime_b200 import lib as ml
    from oracle import oracle as orc
    clib = ml.load()
    cores = os.cpu_count() or 1
    kind = "reference" if orc.Reference.available(fast=True) else "port"
    layers = [(ml.synth_router(clib, SEED, L), ml.synth_norm(clib, SEED, L), ml.synth_experts(clib, SEED, L, 0, 256)) for L in range(nlay)]
    x0 = ml.synth_hidden(clib, SEED, 1000, NB)
    if kind == "reference":
        ref = orc.Reference(fast=True)
        threads = ref.threads(min(cores, 64))
        for L in range(nlay):
            ref.set_layer(L, *layers[L])

        def step():
            x = x0.copy(); return ref.stack(x, 0, nlay)     # seconds on the reference's own clock (maple.c:47)
    else:
        o = orc.Oracle(); threads = o.lib.orc_threads(min(cores, 64))

        def step():
            x = x0; t = time.perf_counter()
            for L in range(nlay):
                x, _ = o.moe(*layers[L], x, 1, dump=False)
            return time.perf_counter() - t
    for _ in range(warmup):
        step()
    t_all, t0 = [], time.perf_counter()
    for _ in range(steps):
        t_all.append(step())
        if budget_s is not None and time.perf_counter() - t0 > budget_s:
            break
    per_step = sum(t_all) / len(t_all) * (LAYERS / nlay)
    value = NB / per_step
    sample = (f"{len(t_all)} steps of one 2048-token chunk through {nlay} distinct layers (router to combine)" +
              ("" if nlay == LAYERS else f", scaled x{LAYERS / nlay:g} to 24 layers"))
    return value, per_step, len(t_all), {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample}


def reference_main(args, rank, world):
    if rank != 0:
        return
    value, per_step, done, cb = cpu_reference_arm(args.steps, args.warmup, LAYERS)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": done, "warmup": args.warmup,
        "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic", "config": workload_config(1), "cpu_baseline": cb,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def workload_config(world):
    return {"workload": "24-layer Maple MoE stack (d=2048, 256 ternary experts 512/2048, top-8), prefill chunk of 2048 tokens per GPU, "
                        "hidden ~N(0,1), random router (near-uniform routing), seeded synthetic weights",
            "tokens_per_step_per_gpu": NB, "layers": LAYERS,
            "parallelism": f"ep{world}: tokens split over the GPUs, {256 // world} experts per GPU, dispatch and combine by peer stores over NVLink" if world > 1 else "single",
            "l2": "inputs larger than L2: 4.9 GB of expert weights are streamed from HBM every step"}


def parity_check(g, ml, nl):
    """Two layers of one chunk against the reference (oracle/_ref; the CPU restatement where that is absent), layer by layer on the
    reference's own inputs: same top-8 indices, hidden state within 1e-5 (max |d| / max |ref|, maple.c:942-946).  Runs each layer three
    times, so that the compared result also comes from a graph replay."""
    from oracle import oracle as orc
    clib = g.lib
    nlay = min(2, nl)
    x = ml.synth_hidden(clib, SEED, 1999, NB)
    use_ref = orc.Reference.available()
    ref = orc.Reference() if use_ref else orc.Oracle()
    if use_ref:
        ref.threads(1)      # one thread: the reference's workers spin for the life of the process (maple.c:89-108) and would sit on
                            # the cores that the CPU baseline leg times later
    worst, same_top = 0.0, True
    for L in range(nlay):
        lay = (ml.synth_router(clib, SEED, L), ml.synth_norm(clib, SEED, L), ml.synth_experts(clib, SEED, L, 0, 256))
        if use_ref:
            ref.set_layer(L, *lay); want, d = ref.moe(L, x, 1)
        else:
            want, d = ref.moe(*lay, x, 1)
        for _ in range(3):
            got = x.copy(); g.forward(got, L, 1)
        same_top = same_top and bool(np.array_equal(g.peek("top", NB).reshape(NB, 8), d["top"]))
        worst = max(worst, float(np.abs(got - want).max() / np.abs(want).max()))
        x = want
    ok = same_top and worst <= 1e-5
    return {"result": "equal" if ok else "DIFFERENT", "against": "oracle/_ref (maple.c compiled here)" if use_ref else "oracle port",
            "layers": nlay, "top8_indices_equal": same_top, "hidden_max_rel": worst, "tolerance": 1e-5,
            "how": "layer by layer on the reference's inputs, third call of each layer (a graph replay)"}


def gpre_moe_leg(g, ml, nl, warm, steps):
    """The chunk through nl calls of gpre_moe (gpu_pre.m:318-385; call site maple.c:763): normalised hidden rows and the grouping tables
    come from the host, the result goes back to the host, every call synchronous.  The tables are the ones this library's own routing
    produced for the chunk (taken layer by layer beforehand); what is timed is only the calls."""
    clib = g.lib
    x = ml.synth_hidden(clib, SEED, 2000, NB)
    g._chk(clib.gmoe_x_upload(x.ctypes.data, NB))
    calls = []
    gloc = ml.gloc_for_contiguous()
    for L in range(nl):
        g._chk(clib.gmoe_forward_dev(NB, L, 1, None)); g._chk(clib.gmoe_sync())
        nu = int(g.peek("nu", NB)[0]); ue = g.peek("ue", NB)[:nu]
        regs = np.array([g.layer_region[L], -1, -1, -1], np.int32)
        calls.append((g.peek("hn", NB).copy(), nu, np.ascontiguousarray(gloc[ue]), regs, g.peek("ustart", NB)[:nu + 1].copy(),
                      g.peek("utok", NB).copy(), g.peek("uw", NB).copy(), g.peek("tp", NB).copy()))
    # maple.c hands every layer's call the same two arrays (HNB in, YB out: static, maple.c:763); so does this loop.  Writing a layer's
    # normalised rows into HNB is the reference's CPU work (its attention and norm) and is not timed.
    hnb, yb = np.empty((NB, H), np.float32), np.empty((NB, H), np.float32)
    clib.gpre_pin_policy(1)         # what GPRE_PIN_HOST=1 does for an unmodified maple.c: HNB and YB are page-locked where they lie
    t_wall, t_gpu = 0.0, 0.0
    for i in range(warm + steps):
        for c in calls:
            hnb[:] = c[0]
            t0 = time.perf_counter()
            tg = g.gpre_moe(hnb, *c[1:], out=yb)[1]
            if i >= warm:
                t_wall += time.perf_counter() - t0; t_gpu += tg
    clib.gpre_pin_policy(0)         # releases the registrations before the arrays go
    return {"value": NB * steps / t_wall, "unit": UNIT, "ms_per_step": t_wall / steps * 1e3, "gpu_ms_per_step": t_gpu / steps * 1e3, "calls_per_step": nl,
            "h2d_bytes_per_step": int(sum(c[0].nbytes + c[2].nbytes + c[4].nbytes + c[5].nbytes + c[6].nbytes + c[7].nbytes for c in calls)),
            "d2h_bytes_per_step": NB * H * 4 * nl,
            "note": "wall clock around the synchronous calls; one input and one output array for all calls (maple.c's static HNB and YB), ordinary "
                    "allocations that the library page-locks in place when it sees them a second time (GPRE_PIN_HOST=1); gpu_ms = the seconds the calls return"}


# ---------------------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=LAYERS, help="fewer layers for small profiling captures (not a bench number)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--capture", choices=["prefill", "decode", "attn"], help="a short run for a profiler, no timing and no JSON line: 2 layers, 3 passes of "
                    "one chunk (2048 tokens, or 64 for decode) with plain launches (no graph replay), so that a capture of a few launches of one kernel stays small")
    ap.add_argument("--zipf", action="store_true", help="skewed routing: a per-expert logit bias from a Zipf(s=1.2) ranking (BASELINE config 4); not the headline line")
    args = ap.parse_args()
    rank, local, world = dist_env()
    if args.impl == "reference":
        return reference_main(args, rank, world)
    if args.capture:
        from maple_runtime_b200 import lib as ml
        nbc = NB if args.capture == "prefill" else 64
        g = ml.Gpre(NB, device=local)
        if args.capture == "attn":      # the head of the attention half alone: 2048 tokens, local layer, 3 launches
            rng = np.random.default_rng(SEED)
            qkv = rng.standard_normal((NB, 3072)).astype(np.float32); pos = np.arange(NB, dtype=np.int32)
            ang = np.arange(NB)[:, None] / np.power(10000.0, (2.0 * np.arange(32)) / 64)[None, :]
            g.rope_table(np.stack([np.cos(ang), np.sin(ang)], -1).astype(np.float32))
            for _ in range(3):
                g.qk_rope(qkv, pos, 0, np.ones(128, np.float32), np.ones(128, np.float32))
            print("capture run done: attn, 2048 tokens, 3 launches", file=sys.stderr)
            return
        for L in range(2):
            g.synth_layer(SEED, L)
        g.lib.gmoe_set_graph(0)
        x = ml.synth_hidden(g.lib, SEED, 2000, nbc)
        for _ in range(3):
            xx = x.copy(); g.forward(xx, 0, 2)
        print(f"capture run done: {args.capture}, {nbc} tokens, 2 layers, 3 passes", file=sys.stderr)
        return
    warm = max(args.warmup, 3)
    dist = init_dist(world)

    from maple_runtime_b200 import lib as ml
    g = ml.Gpre(NB, device=local)
    clib = g.lib
    nl = args.layers
    epr = 256 // world
    for L in range(nl):
        g.synth_layer(SEED, L, rank * epr, epr)        # expert parallel: each GPU holds only its own experts
    if world > 1:
        from maple_runtime_b200 import ep
        ep.setup(g, rank, world, gather_obj(dist))

    bias = ml.synth_zipf_bias(clib, SEED) if args.zipf else None
    bptr = bias.ctypes.data if bias is not None else None

    def forward_chunk(c):
        if world > 1:
            g._chk(clib.gmoe_ep_forward_dev(c, NB, 0, nl, bptr))
        else:
            g._chk(clib.gmoe_forward_chunk(c, NB, 0, nl, bptr))

    def forward_host(ptr):
        return g._chk(clib.gmoe_ep_forward(ptr, NB, 0, nl, bptr) if world > 1 else clib.gmoe_forward(ptr, NB, 0, nl, bptr))
    nring = 4
    ring = np.concatenate([ml.synth_hidden(clib, SEED, 2000 + rank * 16 + c, NB) for c in range(nring)])
    g._chk(clib.gmoe_chunks_upload(ring.ctypes.data, NB, nring))

    # ---- parity on the timed path, before anything is timed ----
    parity = parity_check(g, ml, nl) if (world == 1 and rank == 0) else "not run at N > 1 (every GPU holds a shard of the experts); tests/test_ep.py compares the expert-parallel path"

    # ---- value: chunk resident in HBM, K steps, each device-timed between two events on the library's stream; graph replay, no
    # per-stage events inside ----
    import ctypes as C
    for i in range(warm):
        forward_chunk(i % nring); g._chk(clib.gmoe_sync())
    sampler = ClockSampler(local); sampler.start()
    l0 = clib.gmoe_launch_count()
    barrier(dist)
    t_dev = 0.0
    wall0 = time.perf_counter()
    for i in range(args.steps):
        forward_chunk(i % nring)
        t_dev += g._chk(clib.gmoe_sync())              # device seconds of this step (events on the library's stream)
    wall = time.perf_counter() - wall0
    barrier(dist)
    launches = clib.gmoe_launch_count() - l0
    t_dev = allmax(dist, t_dev)
    value = world * NB * args.steps / t_dev

    # ---- the dominant kernel's own duration: a pass with events around the gate+up launches only (graph replay) ----
    g.profile(1 << 4)                                   # one pass runs plainly, the next is captured with its event records, the rest replay it
    for i in range(5):
        forward_chunk(i % nring); g._chk(clib.gmoe_sync())
    secs, nlaunch = g.profile_read()                    # the plain pass and the last replay
    g.profile(0)

    # ---- stage breakdown (separate pass, all stages timed, plain launches instead of the graph replay) ----
    clib.gmoe_set_graph(0)
    g.profile(0xFF)
    for i in range(2):
        forward_chunk(i % nring)
    st_secs, st_n = g.profile_read()
    g.profile(0)
    clib.gmoe_set_graph(1)
    breakdown = {name: round(float(s) / (2 * nl) * 1e6, 2) for name, s in zip(g.STAGES, st_secs)}   # us per layer

    # ---- e2e: host buffers, copies inside the timed region.  The streaming form (gmoe_forward_submit / gmoe_forward_wait, two chunks
    # outstanding: a chunk's copies run beside the other chunk's kernels) is the headline; the waiting call (gmoe_forward) beside it ----
    hx = clib.gmoe_pinned_alloc(NB * H * 4)
    hbuf = np.ctypeslib.as_array(C.cast(hx, C.POINTER(C.c_float)), shape=(NB, H))
    t_sync = 0.0
    for i in range(warm + args.steps):
        hbuf[:] = ring[(i % nring) * NB:(i % nring + 1) * NB]
        if i == warm:
            barrier(dist)
        t = forward_host(hx)
        if i >= warm:
            t_sync += t
    barrier(dist)
    t_sync = allmax(dist, t_sync)
    hin = [clib.gmoe_pinned_alloc(NB * H * 4) for _ in range(nring)]
    hout = [clib.gmoe_pinned_alloc(NB * H * 4) for _ in range(2)]
    for c in range(nring):
        np.ctypeslib.as_array(C.cast(hin[c], C.POINTER(C.c_float)), shape=(NB, H))[:] = ring[c * NB:(c + 1) * NB]

    def submit(i):
        g._chk(clib.gmoe_forward_submit(hin[i % nring], hout[i % 2], NB, 0, nl, bptr))
    for i in range(warm):
        submit(i); g._chk(clib.gmoe_forward_wait())
    barrier(dist)
    g._chk(clib.gmoe_forward_mark())
    submit(0)
    for i in range(1, args.steps):
        submit(i); g._chk(clib.gmoe_forward_wait())
    t_e2e = g._chk(clib.gmoe_forward_wait())            # device seconds from the mark to the end of the last chunk's copy back
    barrier(dist)
    t_e2e = allmax(dist, t_e2e)
    e2e = world * NB * args.steps / t_e2e
    e2e_sync = world * NB * args.steps / t_sync
    clocks = sampler.summary()          # sampled from the start of the device-timed steps to the end of the host-buffer loops

    # ---- roofline of the dominant kernel ----
    pk = peaks()
    i8_peak = float(clib.gmoe_i8_peak(256, 30000)) if rank == 0 else 0.0      # ~40 ms of MMAs on every SM
    gu_t = float(secs[4]) / max(int(nlaunch[4]), 1)          # stage 4 is one launch per layer: the grouped gate+up GEMM
    gu_tops = GU_OPS_PER_PAIR * NB * 8 / gu_t / 1e12
    traffic, traffic_src = profiled_traffic("gate_up")
    # Which roof binds: the kernel's algorithmic bytes over the measured copy bandwidth against its integer operations over the measured
    # kind::i8 rate.  Per pair 2048 B of int8 activations in and 2 x 512 fp32 values out; per expert its gate and up codes and row scales
    # once (every expert is used at this size).  At 64 pairs per expert that is 291 operations per byte, below the machine balance
    # (~700), so the HBM roof is the binding one; the tensor roof is reported beside it.
    gu_bytes = NB * 8 * (2048 + 2 * 512 * 4) + 256 * 2 * 264192
    gu_gbs = gu_bytes / gu_t / 1e9
    t_hbm, t_tensor = gu_bytes / (pk["hbm_gbs"] * 1e9), (GU_OPS_PER_PAIR * NB * 8 / (i8_peak * 1e12) if i8_peak > 0 else 0.0)
    roofline = {"kernel": "grouped gate+up GEMM (int8 x ternary, tcgen05 kind::i8)", "bound": "hbm" if t_hbm >= t_tensor else "tensor",
                "achieved": gu_gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gu_gbs / pk["hbm_gbs"], "peak_source": pk["src"],
                "algorithmic_bytes_per_launch": gu_bytes, "roof_us": {"hbm": t_hbm * 1e6, "tensor": t_tensor * 1e6},
                "traffic": traffic, "traffic_unit": "bytes per launch",
                "traffic_note": f"dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this workload, from the ncu summary profiles/{traffic_src}" if traffic else "no ncu summary of this kernel under profiles/",
                "launches_timed": int(nlaunch[4]), "avg_launch_us": gu_t * 1e6,
                "tensor": {"achieved": gu_tops, "peak": i8_peak, "unit": "TOP/s (int8)", "frac": gu_tops / i8_peak if i8_peak > 0 else None,
                           "peak_note": "tcgen05.mma kind::i8, M=128 N=256 K=32, operands resident in shared memory, one CTA per SM, measured in this run with CUDA events (gmoe_i8_peak)",
                           "frac_of_2x_bf16_burst": gu_tops / (2.0 * pk["bf16_tflops"]), "frac_of_2x_bf16_sustained": gu_tops / (2.0 * pk["bf16_tflops_sustained"])},
                "bf16_peaks_source": pk["src"], "weights_gbs": 256 * 2 * 264192 / gu_t / 1e9}

    out = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
           "ms_per_step": t_dev / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
           "data": "synthetic", "config": workload_config(world), "clocks": clocks, "gpu_launches": int(launches),
           "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": NB * H * 4, "d2h_bytes_per_step": NB * H * 4,
                   "call": "gmoe_forward_submit / gmoe_forward_wait: pinned host input and output, two chunks outstanding, every chunk's copy in and copy out inside the timed region",
                   "waiting_call": {"value": e2e_sync, "unit": UNIT, "call": "gmoe_forward: copy in, layers, copy out, wait, one chunk at a time"}},
           "roofline": roofline, "stage_us_per_layer": breakdown, "wall_s_timed_region": wall, "parity_check": parity,
           "whole_path_int8_tops_per_gpu": OPS_PER_PAIR * NB * 8 * nl * args.steps / t_dev / 1e12}
    if i8_peak > 0:
        out["whole_path_frac_of_measured_i8_peak"] = out["whole_path_int8_tops_per_gpu"] / i8_peak
    out["whole_path_frac_of_2x_bf16_burst"] = out["whole_path_int8_tops_per_gpu"] / (2.0 * pk["bf16_tflops"])
    if args.zipf:
        out["config"]["routing"] = "router logits + per-expert bias ln(256 p_e), p_e ~ rank^-1.2 over a seeded permutation (skewed load); not the headline configuration"
    if nl != LAYERS:
        out["config"]["layers"] = nl
        out["note"] = "reduced layer count: a profiling run, not a benchmark number"

    # ---- decode shape: 64 conversations x 1 token, one layer at a time over all layers (HBM-bound) ----
    if world > 1:
        out["ep_received_pairs_last_layer"] = [int(v) for v in gather_obj(dist)(clib.gmoe_ep_received())]
        if not args.zipf:
            # the same step with skewed routing (a per-expert logit bias from a Zipf(s=1.2) ranking over a seeded permutation): every rank
            # waits for the rank whose experts are the busiest; not the headline configuration
            zb = ml.synth_zipf_bias(clib, SEED); zp = zb.ctypes.data
            for i in range(3):
                g._chk(clib.gmoe_ep_forward_dev(i % nring, NB, 0, nl, zp)); g._chk(clib.gmoe_sync())
            barrier(dist)
            tz, nz = 0.0, min(args.steps, 5)
            for i in range(nz):
                g._chk(clib.gmoe_ep_forward_dev(i % nring, NB, 0, nl, zp)); tz += g._chk(clib.gmoe_sync())
            barrier(dist)
            tz = allmax(dist, tz)
            recv = [int(v) for v in gather_obj(dist)(clib.gmoe_ep_received())]
            out["skewed_routing"] = {"value": world * NB * nz / tz, "unit": UNIT, "ms_per_step": tz / nz * 1e3, "steps": nz,
                                     "routing": "router logits + per-expert bias ln(256 p_e), p_e ~ rank^-1.2 over a seeded permutation; experts sharded contiguously by index",
                                     "ep_received_pairs_last_layer": recv}
    if rank == 0 and world == 1:
        out["e2e_gpre_moe"] = gpre_moe_leg(g, ml, nl, 1, min(args.steps, 5))
        # the head of the attention half (q/k norm, half-rotary embedding, fp16 cache rows): one launch per layer, bound by HBM
        rng = np.random.default_rng(SEED)
        qkv = rng.standard_normal((NB, 3072)).astype(np.float32); pos = np.arange(NB, dtype=np.int32)
        ang = np.arange(NB)[:, None] / np.power(10000.0, (2.0 * np.arange(32)) / 64)[None, :]
        g.rope_table(np.stack([np.cos(ang), np.sin(ang)], -1).astype(np.float32))
        ones = np.ones(128, np.float32)
        ts = sorted(g.qk_rope(qkv, pos, 0, ones, ones)[3] for _ in range(7))
        ah_bytes = NB * (3072 * 4 + 2048 * 4 + 2 * 512 * 2)
        out["attention_head"] = {"what": "gmoe_qk_rope on one 2048-token chunk: q/k RMS norm, half-rotary embedding, fp16 key and value rows (kernel only, median of 7)",
                                 "us": ts[3] * 1e6, "algorithmic_bytes": ah_bytes, "achieved_gbs": ah_bytes / ts[3] / 1e9, "frac_of_measured_hbm": ah_bytes / ts[3] / 1e9 / pk["hbm_gbs"]}
    if not args.no_decode and rank == 0 and world == 1:
        out["decode"] = decode_leg(g, clib, ml, nl, pk, warm, args.steps)
        out["dense_projections"] = dense_leg(g, ml, pk, warm, args.steps)
    if not args.no_cpu and rank == 0:
        _, _, _, out["cpu_baseline"] = cpu_reference_arm(400, 1, 3, budget_s=12.0)
    if rank == 0:
        print(json.dumps(out))


def dense_leg(g, ml, pk, warm, steps):
    """The attention projections of one layer on the 2048-token chunk (gpre_dense, gpu_pre.m:235-256): q,k,v as one group of 3072
    rows and o (2048 rows), synthetic ternary matrices; GPU seconds of the call (per-token int8 + the grouped kernel), host copies
    outside.  Reported beside the headline, not part of it."""
    rng = np.random.default_rng(SEED & 0xFFFFFFFF)

    def matrix(rows):   # codes 0..2 in every 2-bit field (never 3), scales as for the experts
        c = rng.integers(0, 3, size=(rows, 512, 4), dtype=np.uint8)
        return (c[:, :, 0] | (c[:, :, 1] << 2) | (c[:, :, 2] << 4) | (c[:, :, 3] << 6)).astype(np.uint8), rng.uniform(0.01, 0.05, rows).astype(np.float32)
    for rows in (2048, 512, 512):
        g.dense_add(0, *matrix(rows), rows, 2048)
    g.dense_add(1, *matrix(2048), 2048, 2048)
    g.dense_done(NB)
    x = ml.synth_hidden(g.lib, SEED, 4000, NB)
    out = {}
    for name, grp, rows in (("qkv", 0, 3072), ("o", 1, 2048)):
        ts = [g.dense(grp, x, rows)[1] for _ in range(warm + steps)][warm:]
        t = sum(ts) / len(ts)
        out[name] = {"rows": rows, "us": t * 1e6, "int8_tops": 2.0 * rows * 2048 * NB / t / 1e12, "frac_of_2x_bf16_sustained": 2.0 * rows * 2048 * NB / t / 1e12 / (2.0 * pk["bf16_tflops_sustained"])}
    return out


def decode_leg(g, clib, ml, nl, pk, warm, steps):
    """64 conversations x 1 token through all layers (the --multi 64 shape, maple.c:1189-1199): weight-bandwidth bound."""
    nb = 64
    x = ml.synth_hidden(clib, SEED, 3000, nb)
    g._chk(clib.gmoe_chunks_upload(x.ctypes.data, nb, 1))
    for _ in range(warm):
        g._chk(clib.gmoe_forward_chunk(0, nb, 0, nl, None)); g._chk(clib.gmoe_sync())
    t = 0.0
    for _ in range(steps):                              # the timed steps: graph replay, no per-stage events
        g._chk(clib.gmoe_forward_chunk(0, nb, 0, nl, None)); t += g._chk(clib.gmoe_sync())
    clib.gmoe_set_graph(0); g.profile(0xFF)             # stage breakdown and the weight-stream kernel's own duration: plain launches
    for _ in range(steps):
        g._chk(clib.gmoe_forward_chunk(0, nb, 0, nl, None)); g._chk(clib.gmoe_sync())
    secs, n = g.profile_read(); g.profile(0); clib.gmoe_set_graph(1)
    nu = int(g.peek("nu", nb)[0])                      # used experts of the last layer (others are alike)
    layer_bytes = nu * EXPERT_BYTES + 256 * 2048 * 2 + nb * 2048 * 4 * 3
    gu_bytes = nu * 2 * 264192
    gu_t = float(secs[4]) / max(int(n[4]), 1)
    per_layer = t / steps / nl
    return {"metric": "moe_decode_tokens_per_s_64_conversations", "value": nb * steps / t, "unit": UNIT,
            "ms_per_step": t / steps * 1e3, "used_experts": nu, "bytes_per_layer": layer_bytes,
            "roofline": {"kernel": "gate+up weight stream (register-decode mma.sync)", "bound": "hbm", "achieved": gu_bytes / gu_t / 1e9,
                         "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gu_bytes / gu_t / 1e9 / pk["hbm_gbs"], "traffic": profiled_traffic("decode_gate_up")[0], "traffic_unit": "bytes per launch",
                         "traffic_note": "from the ncu summary under profiles/ (every used expert's gate and up bytes once)",
                         "avg_launch_us": gu_t * 1e6},
            "layer_hbm_frac": layer_bytes / per_layer / 1e9 / pk["hbm_gbs"],
            "stage_us_per_layer": {name: round(float(s) / (steps * nl) * 1e6, 2) for name, s in zip(g.STAGES, secs)}}


if __name__ == "__main__":
    main()
