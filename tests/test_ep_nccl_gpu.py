"""GPU (two or more devices): the expert-parallel host that lives inside the library --
b200moe_ep_unique_id / ep_init / ep_forward / ep_shutdown, NCCL sends and receives, no
torch.distributed. One child process per rank; each compares its output with the single-GPU
operator on the same tokens. Skipped on a box with one GPU."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("shared", [0, 1])
def test_library_side_expert_parallel_host(cuda, tmp_path, shared):
    torch = cuda
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "ep_nccl_worker.py"), str(r), str(world), str(tmp_path), str(shared)],
                              env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(o)
    for r, p in enumerate(procs):
        assert p.returncode == 0, "rank %d failed:\n%s" % (r, outs[r][-3000:])
    for r in range(world):
        res = json.load(open(os.path.join(str(tmp_path), "rank%d.json" % r)))
        assert res["finite"]
        # same products and fp32 accumulators as the single-GPU call; only the combine adds in placed-id order
        assert res["max_abs"] <= 4e-3 and res["mean_rel"] <= 1e-5, res
        assert res["overflow_status"] == 8, res          # B200MOE_ERR_TOO_LARGE on every rank
