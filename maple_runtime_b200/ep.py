"""Expert-parallel set-up helpers and a host statement of the dispatch plan (csrc/k_ep.cu) for tests.

The data path is in the C library (gmoe_ep_*); this module only moves the NCCL id and the CUDA IPC handles between the
ranks through whatever all-gather the caller has (torch.distributed with gloo in bench.py and the tests)."""
import ctypes as C
import numpy as np

NE = 256


def plan(all_cnt, rank, world):
    """all_cnt [world][256]: pairs per expert of every rank.  Returns what ep_plan_kernel computes for `rank`:
    dst_base [256] (slot of this rank's first pair of expert e in the owner's receive buffer), and the owner's view
    (used experts, starts, total)."""
    all_cnt = np.asarray(all_cnt, np.int64).reshape(world, NE)
    epr = NE // world
    tot = all_cnt.sum(0)
    before = all_cnt[:rank].sum(0)
    base = np.zeros(NE, np.int64)
    for e in range(NE):
        o = e // epr
        base[e] = tot[o * epr:e].sum()
    mine = np.arange(NE) // epr == rank
    cnt = np.where(mine, tot, 0)
    ue = np.nonzero(cnt)[0]
    ustart = np.concatenate([[0], np.cumsum(cnt[ue])])
    return dict(dst_base=(base + before).astype(np.int32), ue=ue.astype(np.int32), ustart=ustart.astype(np.int32), total=int(cnt.sum()))


def setup(g, rank, world, all_gather):
    """g: maple_runtime_b200.lib.Gpre already initialised on this rank's GPU.  all_gather(obj) -> list of every rank's obj."""
    lib = g.lib
    uid = C.create_string_buffer(128)
    if rank == 0:
        g._chk(lib.gmoe_ep_unique_id(uid))
    uid_raw = all_gather(uid.raw)[0]
    g._chk(lib.gmoe_ep_init(rank, world, uid_raw))
    h = C.create_string_buffer(448)
    g._chk(lib.gmoe_ep_handles(h))
    allh = b"".join(all_gather(h.raw))
    g._chk(lib.gmoe_ep_connect(allh))
    all_gather(b"connected")       # nobody starts storing into a peer before every peer has opened its handles
