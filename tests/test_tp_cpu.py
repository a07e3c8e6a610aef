"""Multi-process tensor parallelism and failure detection on CPU ranks (gloo, world 2 and 4)."""
import os
import socket
import subprocess
import sys
import time

import pytest

from oxidize_b200.parallel.health import (Heartbeat, MemoryStore, RunnerStatus, StepWatchdog, eval_with_timeout)

HERE = os.path.dirname(os.path.abspath(__file__))


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def fail_text(r) -> str:
    """What the ranks themselves printed before the launcher's own failure report (which is long and says nothing)."""
    err = r.stderr
    for mark in ("Sending process", "failed (exitcode"):
        i = err.find(mark)
        if i >= 0:
            err = err[:i]
            break
    return r.stdout[-2000:] + "\n" + err[-6000:]


def run_ranks(case, n=2, device="cpu", comm="nccl", timeout=300, env_extra=None):
    env = dict(os.environ)
    env.update({"OMP_NUM_THREADS": "2"})
    env.update(env_extra or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), os.path.join(HERE, "mp_worker.py"), case, "--device", device,
           "--comm", comm]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    return r


def test_tp2_logits_match_tp1_on_cpu():
    r = run_ranks("tp_model")
    assert r.returncode == 0, fail_text(r)
    assert r.stdout.count("OK tp_model") == 2


def test_tp4_logits_match_tp1_on_cpu():
    r = run_ranks("tp_model", n=4)
    assert r.returncode == 0, fail_text(r)
    assert r.stdout.count("OK tp_model") == 4


def test_tp2_gemma3_and_latent_attention_match_single_rank_on_cpu():
    r = run_ranks("tp_families", 2)
    assert r.returncode == 0, fail_text(r)


def test_ep2_moe_logits_match_single_rank_on_cpu():
    r = run_ranks("ep_model")
    assert r.returncode == 0, fail_text(r)
    assert r.stdout.count("OK ep_model") == 2


def test_tp2_with_replicated_experts_matches_single_rank_on_cpu():
    r = run_ranks("ep1_model")
    assert r.returncode == 0, fail_text(r)
    assert r.stdout.count("OK ep1_model") == 2


def test_mismatched_expert_partition_is_rejected():
    import torch

    from oxidize_b200.models.config import preset
    from oxidize_b200.models.transformer import Transformer
    from oxidize_b200.utils.synth import synth_weights

    cfg = preset("mixtral-8x7b", hidden_size=64, n_layers=1, n_heads=2, n_kv_heads=2, head_dim=32, ffn_size=64,
                 expert_ffn_size=32, vocab_size=64, n_experts=4, n_experts_used=2)
    w = synth_weights(cfg, torch.device("cpu"), "F32", ep_rank=0, ep_size=2)
    with pytest.raises(ValueError, match="expert parallelism must span the whole group"):
        Transformer(w)


def test_pp2_tokens_match_single_process_on_cpu():
    r = run_ranks("pp_model")
    assert r.returncode == 0, fail_text(r)
    assert r.stdout.count("OK pp_model") == 2


def test_engine_with_two_pipeline_stages_on_cpu():
    r = run_ranks("pp_engine")
    assert r.returncode == 0, fail_text(r)
    assert r.stdout.count("OK pp_engine") == 2


def test_engine_with_tp2_x_pp2_on_cpu():
    r = run_ranks("pp_engine", n=4)
    assert r.returncode == 0, fail_text(r)
    assert r.stdout.count("OK pp_engine") == 4


def test_rank_exit_detected_by_heartbeat():
    r = run_ranks("rank_exit")
    assert r.returncode == 0, fail_text(r)
    assert r.stdout.count("OK rank_exit") == 2


def test_eval_with_timeout_variants():
    assert eval_with_timeout(lambda: 5, 1.0).value == 5
    seen = []
    res = eval_with_timeout(lambda: time.sleep(3600), 0.05, on_failure=seen.append)
    assert res.status == "timed_out" and seen == ["timed_out"]
    res = eval_with_timeout(lambda: 1 / 0, 1.0, on_failure=seen.append)
    assert res.status == "error" and isinstance(res.error, ZeroDivisionError)


def test_heartbeat_staleness_with_fake_clock():
    store = MemoryStore()
    now = [100.0]
    a = Heartbeat(store, 0, 3, stale_after_s=5.0, clock=lambda: now[0])
    b = Heartbeat(store, 1, 3, stale_after_s=5.0, clock=lambda: now[0])
    a.beat()
    b.beat()
    assert a.dead_ranks() == []  # rank 2 never joined but the grace period has not passed
    now[0] += 6.0
    a.beat()
    assert a.dead_ranks() == [1, 2]  # 1 went stale, 2 never joined
    b.beat()
    assert a.dead_ranks() == [2]
    store.set("exit/1", "1")
    assert a.dead_ranks() == [1, 2]


def test_step_watchdog_trips():
    hits = []
    wd = StepWatchdog(deadline_s=0.1, on_trip=hits.append)
    wd.begin_step()
    wd.end_step()
    time.sleep(0.2)
    assert wd.healthy
    wd.begin_step()
    time.sleep(0.4)
    assert not wd.healthy and wd.status is RunnerStatus.FAILED and len(hits) == 1
    wd.close()
