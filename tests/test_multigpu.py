"""Multi-GPU checks (run as child processes over NCCL + peer memory, NVLS off)."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(script: str, nproc: int, port: int, *args: str, timeout: int = 600, extra_env: dict | None = None) -> str:
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **(extra_env or {}))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, script), *args]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    out = res.stdout + res.stderr
    assert res.returncode == 0, out[-4000:]
    return out


@pytest.mark.parametrize("clip", ["0", "0.5"])
def test_fsdp_matches_single_process(unique_port, clip):
    n = min(torch.cuda.device_count(), 4)
    out = _run("_mp_fsdp_check.py", n, unique_port, clip)
    assert "MP_FSDP_OK" in out, out[-4000:]


def test_resharded_modes_equal_resident_mode(unique_port):
    """reshard_after_forward (pooled slots), shard_every_ith_layer and checkpointing on top give the same numbers."""
    n = 4 if torch.cuda.device_count() >= 4 else 2
    out = _run("_mp_fsdp_modes.py", n, unique_port, timeout=900)
    assert "MP_MODES_OK" in out, out[-4000:]


def test_missing_rank_makes_the_step_raise(unique_port):
    """Host-made failure: one rank skips a step; the other's bounded barrier waits run out, its step raises and its
    optimizer state stays untouched."""
    out = _run("_mp_fsdp_timeout.py", 2, unique_port)
    assert "MP_TIMEOUT_OK" in out, out[-4000:]


def test_hybrid_sharding_replicas_stay_in_sync(unique_port):
    """Two replicas of a one-rank shard group: gradients are summed over the replicate group before the update."""
    out = _run("_mp_fsdp_check.py", 2, unique_port, "0.5", "1")
    assert "MP_FSDP_OK" in out, out[-4000:]


@pytest.mark.parametrize("kind,sp", [("llama", "1"), ("llama", "0"), ("qwen3", "1"), ("olmo3", "1")])
def test_tensor_parallel_matches_unsharded(unique_port, kind, sp):
    """Fused all-gather GEMM / GEMM reduce-scatter / embedding push against the unsharded model."""
    n = 2
    out = _run("_mp_tp_check.py", n, unique_port, "nccl", kind, sp, str(unique_port))
    assert "TP_OK" in out, out[-4000:]


@pytest.mark.parametrize("tp", [2, 4])
def test_tensor_parallel_times_sharded_data_parallel(unique_port, tp):
    """TP (with SP and the sharded loss) composed with the FSDP engine on a (dp_shard, tp) mesh."""
    n = torch.cuda.device_count()
    if n < 2 * tp and not (tp == 2 and n >= 2):
        pytest.skip(f"needs {2 * tp} GPUs")
    nproc = 2 * tp if n >= 2 * tp else tp   # falls back to tp x 1 (engine with a one-rank shard group)
    out = _run("_mp_tp_fsdp_check.py", nproc, unique_port, str(tp))
    assert "MP_TP_FSDP_OK" in out, out[-4000:]


def test_tensor_parallel_fp8(unique_port):
    """Block-scaled FP8 projections under tensor + sequence parallelism stay close to the unsharded bf16 model."""
    out = _run("_mp_tp_check.py", 2, unique_port, "nccl", "llama", "1", str(unique_port), "fp8")
    assert "TP_OK" in out, out[-4000:]


@pytest.mark.parametrize("kind", ["llama", "qwen3"])
def test_tensor_parallel_pull_all_gather(unique_port, kind):
    """The pull form of the fused all-gather (the push form is the default) forced on."""
    out = _run("_mp_tp_check.py", 2, unique_port, "nccl", kind, "1", str(unique_port),
               extra_env={"OB_TP_PUSH_MIN_WORLD": "99"})
    assert "TP_OK" in out, out[-4000:]


def test_fp8_all_gather_gemm_fused(unique_port):
    """Quantise + e4m3 all-gather + GEMM in one launch equals the unfused sequence (block and per-tensor scales)."""
    out = _run("_mp_fp8_ag_check.py", 2, unique_port, str(unique_port))
    assert "FP8_AG_OK" in out
