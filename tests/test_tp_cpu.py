"""Tensor / sequence parallelism on CPU: two Gloo ranks against the unsharded model (fp32).

The same autograd structure runs on GPUs with the fused NVLink kernels; here the collectives are
``torch.distributed`` calls, which checks the sharding plan, the gradient flow (partial gradients of
replicated parameters are summed over the group) and the vocabulary-parallel loss.
"""

import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(port: int, kind: str, sp: str) -> str:
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", CUDA_VISIBLE_DEVICES="")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "_mp_tp_check.py"), "gloo", kind, sp, str(port)],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append(o)
        assert p.returncode == 0, o[-3000:]
    return "\n".join(outs)


@pytest.mark.parametrize("kind,sp", [("llama", "0"), ("llama", "1"), ("qwen3", "1"), ("olmo3", "1")])
def test_tp_matches_unsharded(unique_port, kind, sp):
    assert "TP_OK" in _run(unique_port, kind, sp)


def test_tp_checkpoint_layout_roundtrip(unique_port, tmp_path):
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", CUDA_VISIBLE_DEVICES="")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "_mp_tp_ckpt.py"), str(unique_port), str(tmp_path)],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        o, _ = p.communicate(timeout=600)
        outs.append(o)
        assert p.returncode == 0, o[-3000:]
    assert "TP_CKPT_OK" in "\n".join(outs)
