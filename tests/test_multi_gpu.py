"""Fused NVLink collectives and tensor-parallel serving on 2+ GPUs (child processes, one per GPU)."""
import pytest
import torch

from test_tp_cpu import fail_text, run_ranks

pytestmark = pytest.mark.gpu

NEED2 = pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
# plain peer loads/stores only in these tests; NVLS is kept off in NCCL as well
ENV = {"NCCL_NVLS_ENABLE": "0"}


def _ngpu():
    n = torch.cuda.device_count()
    return 8 if n >= 8 else 4 if n >= 4 else 2


@NEED2
def test_gemm_allreduce_fused_matches_reference():
    r = run_ranks("gemm_ar", n=_ngpu(), device="cuda", comm="fused", env_extra=ENV)
    assert r.returncode == 0, fail_text(r)


@NEED2
@pytest.mark.parametrize("comm", ["nccl", "fused"])
def test_tp_model_matches_single_gpu(comm):
    r = run_ranks("tp_model", n=2, device="cuda", comm=comm, env_extra=ENV)
    assert r.returncode == 0, fail_text(r)


@NEED2
def test_tp_decode_under_cuda_graphs():
    r = run_ranks("tp_graph", n=2, device="cuda", comm="fused", env_extra=ENV)
    assert r.returncode == 0, fail_text(r)


@NEED2
def test_expert_parallel_moe_matches_single_rank():
    r = run_ranks("ep_model", n=2, device="cuda", comm="fused", env_extra=ENV)
    assert r.returncode == 0, fail_text(r)


@NEED2
def test_engine_with_two_pipeline_stages_on_gpus():
    """pp_size = 2 through the engine: stage-local layers on each GPU, micro-batched steps, NCCL p2p hand-off."""
    r = run_ranks("pp_engine", n=2, device="cuda", comm="nccl", env_extra=ENV)
    assert r.returncode == 0, fail_text(r)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_engine_with_tp2_x_pp2_on_gpus():
    r = run_ranks("pp_engine", n=4, device="cuda", comm="fused", env_extra=ENV)
    assert r.returncode == 0, fail_text(r)


@NEED2
def test_rank_exit_between_steps_is_detected():
    r = run_ranks("rank_exit", n=2, device="cuda", comm="nccl", env_extra=ENV)
    assert r.returncode == 0, fail_text(r)


def test_peer_wait_times_out_and_reports():
    """A peer that never shows up: the bounded flag wait gives up, the status word says so and
    the context stays usable (the missing peer is simulated — nothing is launched for it)."""
    from oxidize_b200.models.weights import LinearWeight, QTensor
    from oxidize_b200.ops import cuda as C
    from oxidize_b200.parallel.fused import FusedComm

    dev = torch.device("cuda", 0)
    comm = FusedComm(dev, max_tokens=64, hidden=1024, timeout_s=0.002)
    # pretend to be rank 0 of 2 with both "peers" mapped onto this GPU's own buffers
    comm.set_peer_pointers([comm.data.data_ptr()] * 2, [comm.flags.data_ptr()] * 2, world=2, rank=0)
    x = torch.randn(8, 256, device=dev).to(torch.bfloat16)
    w = torch.randn(256, 256, device=dev).to(torch.bfloat16)
    C.status()
    comm.linear_allreduce(x, LinearWeight([QTensor("BF16", w, (256, 256))]))
    torch.cuda.synchronize()
    code, detail, count = C.status()
    assert code == 4 and count >= 1
    # the context is still usable
    y = C.gemm_bf16(x, w)
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all() and C.status()[0] == 0
