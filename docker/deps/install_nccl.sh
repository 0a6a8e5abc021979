#!/usr/bin/env bash
# NCCL from source for Blackwell only (sm_100). The framework's own data plane uses peer loads / stores over the
# symmetric heap; NCCL remains the control plane (process groups, barriers, the DDP and HSDP-replica reductions).
set -euo pipefail
NCCL_VERSION="${NCCL_VERSION:-v2.28.9-1}"
PREFIX="${PREFIX:-/usr/local/nccl}"
git clone --depth 1 --branch "${NCCL_VERSION}" https://github.com/NVIDIA/nccl.git /tmp/nccl
cd /tmp/nccl
make -j"$(nproc)" src.build CUDA_HOME="${CUDA_HOME:-/usr/local/cuda}" \
     NVCC_GENCODE="-gencode=arch=compute_100,code=sm_100"
make install PREFIX="${PREFIX}"
echo "${PREFIX}/lib" > /etc/ld.so.conf.d/nccl.conf && ldconfig
rm -rf /tmp/nccl
