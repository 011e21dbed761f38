"""Multi-GPU runs (one process per GPU, NCCL plumbing, peer-memory kernels on the hot path):
collectives through the fused all-reduce kernel, DDP with symmetric-memory buckets, AMP overflow
propagation through the all-reduce, expert parallelism; plus the single-GPU timeout path of a device
wait (a flag that nothing sets, short budget: the kernel returns a status, the context stays usable)."""
import ctypes
import os

import pytest
import torch

from test_cpu_distributed import launch

pytestmark = pytest.mark.gpu
NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0
ENV = {"NCCL_NVLS_ENABLE": "0"}


@pytest.mark.skipif(NGPU < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("scenario", ["collectives", "ddp", "ddp_tied", "ddp_amp", "ddp_amp_clip", "ddp_wire", "ddp_graph", "ep"])
def test_two_gpu_ranks(scenario):
    launch(scenario, world=2, backend="nccl", env=ENV, timeout=600)


@pytest.mark.skipif(NGPU < 2, reason="needs 2 GPUs")
def test_two_gpu_ranks_nccl_transport():
    launch("ddp", world=2, backend="nccl", env={**ENV, "GENESIS_COMM": "nccl"}, timeout=600)


@pytest.mark.skipif(NGPU < 4, reason="needs 4 GPUs")
@pytest.mark.parametrize("scenario", ["ddp", "ddp_tied", "ddp_wire", "ep"])
def test_four_gpu_ranks(scenario):
    launch(scenario, world=4, backend="nccl", env=ENV, timeout=600)


@pytest.mark.skipif(NGPU < 8, reason="needs 8 GPUs")
@pytest.mark.parametrize("scenario", ["collectives", "ddp", "ddp_tied", "ddp_amp", "ddp_wire", "ddp_graph", "ep"])
def test_eight_gpu_ranks(scenario):
    launch(scenario, world=8, backend="nccl", env=ENV, timeout=900)


def test_device_wait_times_out_with_status():
    from genesis_b200.ops import native as N
    L = N.lib()
    flag = torch.zeros(4, dtype=torch.int32, device="cuda")
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = L.gb_wait_flag(flag.data_ptr(), 1, 20_000_000, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    rec = status.tolist()
    assert rec[0] == 2, rec                      # GB_ERR_FLAG_TIMEOUT
    # the context is still healthy and a satisfied wait reports nothing
    status.zero_()
    flag.fill_(5)
    L.gb_wait_flag(flag.data_ptr(), 3, 20_000_000, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0


def test_expired_peer_wait_reaches_the_training_loop():
    """The communication kernels record an expired wait in the library-wide status word: the next host read of a
    result (`Tensor.item()`) raises `CommTimeout`, and so does DDP's sync-free probe at the next forward."""
    import genesis_b200 as genesis
    from genesis_b200.ops import native as N
    from genesis_b200.distributed.process_group import CommTimeout
    L = N.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    st = N.status_tensor(dev)
    N.check_status(dev)
    flag = torch.zeros(4, dtype=torch.int32, device="cuda")
    L.gb_wait_flag(flag.data_ptr(), 1, 20_000_000, st.data_ptr(), torch.cuda.current_stream().cuda_stream)
    loss = genesis.Tensor(torch.ones(1, device="cuda"))
    with pytest.raises(CommTimeout):
        loss.item()
    assert st.tolist()[0] == 0                        # cleared by the read that raised
    # the probe: armed after the kernel, polled later without blocking
    L.gb_wait_flag(flag.data_ptr(), 1, 20_000_000, st.data_ptr(), torch.cuda.current_stream().cuda_stream)
    probe = N.StatusProbe(dev)
    probe.arm()
    with pytest.raises(CommTimeout):
        probe.poll("probe", wait=True)
    N.check_status(dev)
