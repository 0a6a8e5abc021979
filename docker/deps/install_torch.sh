#!/usr/bin/env bash
# PyTorch from source against the system NCCL, compiled for sm_100a only. The package needs torch >= 2.8 for
# torch.distributed._symmetric_memory (symmetric allocations + handle exchange) and DTensor / DCP checkpoints.
set -euo pipefail
TORCH_VERSION="${TORCH_VERSION:-v2.11.0}"
git clone --depth 1 --branch "${TORCH_VERSION}" --recurse-submodules --shallow-submodules \
    https://github.com/pytorch/pytorch.git /opt/pytorch
cd /opt/pytorch
python3 -m pip install --no-cache-dir -r requirements.txt
export TORCH_CUDA_ARCH_LIST="10.0a" USE_SYSTEM_NCCL=1 NCCL_ROOT="${NCCL_ROOT:-/usr/local/nccl}" \
       USE_CUDNN=1 USE_FLASH_ATTENTION=0 USE_MEM_EFF_ATTENTION=0 BUILD_TEST=0 USE_DISTRIBUTED=1 \
       MAX_JOBS="${MAX_JOBS:-$(nproc)}" CMAKE_BUILD_TYPE=Release
python3 setup.py bdist_wheel
python3 -m pip install --no-cache-dir dist/torch-*.whl
cd / && rm -rf /opt/pytorch/build
