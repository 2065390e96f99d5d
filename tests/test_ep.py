"""Expert parallelism: the dispatch plan on CPU ranks (gloo, no GPU), and the whole path on 2 GPUs when the machine has them."""
import os
import subprocess
import sys
import numpy as np
import pytest

from conftest import ROOT


def run_ranks(n, *args, timeout=600):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(29500 + os.getpid() % 1000), os.path.join(ROOT, "tests", "ep_worker.py"), *map(str, args)]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)


def test_plan_statement_small():
    from maple_runtime_b200 import ep
    all_cnt = np.zeros((2, 256), np.int64)
    all_cnt[0, [3, 130]] = [2, 1]; all_cnt[1, [3, 200]] = [4, 5]
    p0, p1 = ep.plan(all_cnt, 0, 2), ep.plan(all_cnt, 1, 2)
    assert p0["total"] == 6 and p1["total"] == 6
    assert p0["dst_base"][3] == 0 and p1["dst_base"][3] == 2          # expert 3 lives on rank 0: rank 0's pairs first, then rank 1's
    assert p0["dst_base"][130] == 0 and p1["dst_base"][200] == 1       # rank 1's buffer: expert 130 (1 pair), then expert 200
    assert list(p1["ue"]) == [130, 200] and list(p1["ustart"]) == [0, 1, 6]


def test_plan_consistent_across_two_cpu_ranks():
    r = run_ranks(2, "cpu")
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("plan consistent") == 2


def _gpus():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=20).stdout
        return out.count("GPU ")
    except Exception:
        return 0


@pytest.mark.gpu
@pytest.mark.parametrize("nb,layers,zipf", [(96, 2, ""), (700, 2, "zipf")])
def test_two_gpus_equal_single_gpu_oracle(nb, layers, zipf):
    if _gpus() < 2:
        pytest.skip("needs 2 GPUs")
    r = run_ranks(2, "gpu", nb, layers, zipf)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("equal bits True") == 12     # 2 ranks x 2 kernel paths x 3 calls (plain, captured, replayed)


@pytest.mark.gpu
def test_rendezvous_gives_up_when_a_rank_never_arrives(gpu):
    """Failure detection of the expert-parallel rendezvous without a GPU fault: a wait on an arrival flag that nothing sets
    ends after its limit with the status the host reads; the context stays usable."""
    import time
    t0 = time.perf_counter()
    assert gpu.lib.gmoe_ep_timeout_selftest(200) == 41
    dt = time.perf_counter() - t0
    assert 0.15 < dt < 5.0
    assert gpu.lib.gmoe_ep_timeout_selftest(20) == 41        # and again: the first give-up left nothing behind
