#!/usr/bin/env bash
# GDRCopy user library (multi-node NCCL over InfiniBand benefits from it; single-node NVLink runs do not need it).
set -euo pipefail
GDRCOPY_VERSION="${GDRCOPY_VERSION:-v2.5}"
git clone --depth 1 --branch "${GDRCOPY_VERSION}" https://github.com/NVIDIA/gdrcopy.git /tmp/gdrcopy
make -C /tmp/gdrcopy -j"$(nproc)" lib lib_install prefix=/usr/local CUDA="${CUDA_HOME:-/usr/local/cuda}"
ldconfig && rm -rf /tmp/gdrcopy
