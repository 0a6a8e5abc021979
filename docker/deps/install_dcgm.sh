#!/usr/bin/env bash
# NVIDIA DCGM (datacenter-gpu-manager) for the optional SM-utilisation metrics of core/profile.py. Read-only use:
# the framework never changes clocks, power limits or any other GPU setting through it.
set -euo pipefail
. /etc/os-release
distro="ubuntu${VERSION_ID//./}"
curl -fsSL "https://developer.download.nvidia.com/compute/cuda/repos/${distro}/x86_64/cuda-keyring_1.1-1_all.deb" -o /tmp/keyring.deb
dpkg -i /tmp/keyring.deb && rm /tmp/keyring.deb
apt-get update && apt-get install -y --no-install-recommends datacenter-gpu-manager-4-cuda12
rm -rf /var/lib/apt/lists/*
