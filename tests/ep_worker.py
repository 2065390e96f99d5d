"""One rank of the expert-parallel tests (launched by torch.distributed.run, one process per rank).

mode cpu: gloo only, no GPU: the dispatch plan of every rank is consistent (slots form a bijection onto the owner's
          receive buffer, ordered by expert, then source rank, then source order).
mode gpu: every rank runs the expert-parallel stack on its own GPU and compares its hidden state, bit for bit, with the
          single-GPU oracle result for its token slice."""
import os
import sys
import numpy as np
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from maple_runtime_b200 import ep, lib as ml  # noqa: E402

SEED = 20261125


def gather(obj):
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, obj)
    return out


def main():
    mode = sys.argv[1]
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    if mode == "cpu":
        rng = np.random.default_rng(100 + rank)
        nb = 64 + 17 * rank                                     # ragged: ranks hold different token counts
        p = 1.0 / np.arange(1, 257) ** 1.2; p /= p.sum()
        top = np.stack([rng.choice(256, 8, replace=False, p=p) for _ in range(nb)])
        cnt = np.bincount(top.ravel(), minlength=256)
        all_cnt = np.stack(gather(cnt))
        pl = ep.plan(all_cnt, rank, world)
        # this rank's pairs in grouped order: expert ascending, token ascending
        order = np.argsort(top.ravel() * 100000 + np.repeat(np.arange(nb), 8), kind="stable")
        exp_sorted = top.ravel()[order]
        first = np.concatenate([[0], np.cumsum(cnt)])[:-1]
        slots = pl["dst_base"][exp_sorted] + (np.arange(nb * 8) - first[exp_sorted])
        owners = exp_sorted // (256 // world)
        everything = gather((owners, slots, exp_sorted))
        totals = gather(pl["total"])
        for o in range(world):
            got = np.concatenate([s[w == o] for w, s, _ in everything])
            assert np.array_equal(np.sort(got), np.arange(totals[o])), "slots are not a bijection onto the receive buffer"
            e_at = np.empty(totals[o], np.int64); r_at = np.empty(totals[o], np.int64)
            for r, (w, s, e) in enumerate(everything):
                e_at[s[w == o]] = e[w == o]; r_at[s[w == o]] = r
            key = e_at * 16 + r_at
            assert np.all(np.diff(key) >= 0), "receive buffer is not ordered by (expert, source rank)"
        print(f"rank {rank}: plan consistent, {pl['total']} pairs received", flush=True)
    else:
        from oracle import oracle as orc
        nb, layers = int(sys.argv[2]), int(sys.argv[3])
        zipf = len(sys.argv) > 4 and sys.argv[4] == "zipf"
        g = ml.Gpre(max(nb, 64), device=rank)
        clib = g.lib
        epr = 256 // world
        for L in range(layers):
            g.synth_layer(SEED, L, rank * epr, epr)             # only this rank's experts live on this GPU
        ep.setup(g, rank, world, gather)
        g.set_router(1)                                         # exact-order router: the comparison below is bit for bit through all layers
        bias = ml.synth_zipf_bias(clib, SEED) if zipf else None
        x = ml.synth_hidden(clib, SEED, 500 + rank, nb)
        want = x.copy()
        o = orc.Oracle()
        for L in range(layers):
            want, _ = o.moe(ml.synth_router(clib, SEED, L), ml.synth_norm(clib, SEED, L), ml.synth_experts(clib, SEED, L, 0, 256), want, 1, bias, dump=False)
        for path in (1, 2):
            g.set_path(path)
            replays = clib.gmoe_graph_launches()
            for call in range(3):       # the first call runs plain launches, the second captures the layer loop, the third replays it
                got = x.copy()
                secs = clib.gmoe_ep_forward(got.ctypes.data, nb, 0, layers, None if bias is None else bias.ctypes.data)
                assert secs > 0, g.err()
                same = np.array_equal(got.view(np.uint32), want.view(np.uint32))
                rel = float(np.abs(got - want).max() / np.abs(want).max())
                print(f"rank {rank} path {path} call {call}: received {clib.gmoe_ep_received()} pairs in the last layer, equal bits {same}, rel {rel:.2e}", flush=True)
                assert same, f"rank {rank} path {path} call {call}: rel {rel:.3e}"
            assert clib.gmoe_graph_launches() - replays >= 2, "the expert-parallel layer loop was not replayed as a graph"
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
