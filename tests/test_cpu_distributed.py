"""Distributed API: single-process semantics (world size 1, error strings of the reference's
`tests/test_distributed.py:367-386`) and real multi-process runs on CPU ranks (gloo, world size 2)
for the collectives, DDP buckets/hooks/no_sync, AMP overflow propagation, expert parallelism and
heartbeat failure detection.  Failures are made on the host only."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

import genesis_b200 as genesis
import genesis_b200.nn as nn
from genesis_b200 import distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launch(scenario, world=2, backend="gloo", timeout=240, env=None):
    e = {**os.environ, "OMP_NUM_THREADS": "2", **(env or {})}
    if backend == "gloo":
        e["CUDA_VISIBLE_DEVICES"] = ""
    for attempt in range(3):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
               os.path.join(HERE, "_dist_worker.py"), "--scenario", scenario, "--backend", backend]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e)
        # the port probed as free can be taken again before the rendezvous binds it (another job on the machine):
        # that is not a result of the scenario, so pick another one
        if r.returncode != 0 and "EADDRINUSE" in r.stderr and attempt < 2:
            continue
        break
    assert r.returncode == 0 and r.stdout.count("WORKER_OK") == world, f"stdout:\n{r.stdout[-3000:]}\nstderr:\n{r.stderr[-3000:]}"


def test_single_process_group_and_error_strings():
    assert not dist.is_initialized()
    for fn in (dist.get_world_size, dist.get_rank, dist.barrier):
        with pytest.raises(RuntimeError, match="Process group not initialized"):
            fn()
    with pytest.raises(ValueError, match="Unsupported backend"):
        dist.init_process_group(backend="invalid_backend", world_size=1, rank=0)
    with pytest.raises(NotImplementedError):
        dist.init_process_group(backend="mpi", world_size=1, rank=0)
    dist.init_process_group(backend="nccl", world_size=1, rank=0)
    try:
        assert dist.is_initialized() and dist.get_world_size() == 1 and dist.get_rank() == 0
        t = genesis.ones(4)
        dist.all_reduce(t)
        dist.broadcast(t, 0)
        dist.barrier()
        outs = [genesis.zeros(4)]
        dist.all_gather(outs, t)
        assert np.array_equal(outs[0].numpy(), np.ones(4, np.float32))
        o = genesis.zeros(4)
        dist.reduce_scatter(o, [t])
        assert np.array_equal(o.numpy(), np.ones(4, np.float32))
        model = nn.Sequential(nn.Linear(4, 3), nn.ReLU(), nn.Linear(3, 2))
        ddp = nn.DistributedDataParallel(model)
        assert ddp.module is model and dist.DistributedDataParallel is nn.DistributedDataParallel
        y = ddp(genesis.ones(5, 4))
        y.sum().backward()
        assert all(p.grad is not None for p in ddp.parameters())
        assert set(ddp.state_dict()) == set(model.state_dict())
        ddp.eval()
        assert not model.training
        with ddp.no_sync():
            pass
    finally:
        dist.destroy_process_group()
        dist.destroy_process_group()          # idempotent
    assert not dist.is_initialized()
    with pytest.raises(RuntimeError):
        nn.DistributedDataParallel(nn.Linear(2, 2))
    assert {o.name for o in dist.ReduceOp} >= {"SUM", "PRODUCT", "MAX", "MIN"}


@pytest.mark.parametrize("scenario", ["collectives", "ddp", "ddp_tied", "ddp_amp", "ep", "heartbeat"])
def test_two_cpu_ranks(scenario):
    launch(scenario, world=2, backend="gloo")


def test_rank_that_never_joins_times_out():
    """Rendezvous with a missing peer ends with an error inside the time budget instead of hanging."""
    code = (
        "import sys, os\n"
        f"sys.path.insert(0, {os.path.dirname(HERE)!r})\n"
        "import torch.distributed as tdist, datetime\n"
        "try:\n"
        "    tdist.init_process_group('gloo', init_method='tcp://127.0.0.1:%d', world_size=2, rank=0,\n"
        "                             timeout=datetime.timedelta(seconds=3))\n"
        "    print('JOINED')\n"
        "except Exception as e:\n"
        "    print('TIMED_OUT', type(e).__name__)\n" % _free_port())
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120,
                       env={**os.environ, "CUDA_VISIBLE_DEVICES": ""})
    assert "TIMED_OUT" in r.stdout, r.stdout + r.stderr


def test_rank_that_skips_a_collective_gives_timeout_on_the_others():
    launch("skipped_collective", world=2, backend="gloo", env={"GENESIS_COMM_TIMEOUT_S": "3"}, timeout=120)
