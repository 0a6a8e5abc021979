#!/usr/bin/env bash
# Build one of the images from the repository root:  docker/build.sh [ngc|raw] [--push]
set -euo pipefail
cd "$(dirname "$0")/.."
target="${1:-ngc}"
shift || true
case "${target}" in
  ngc|raw) ;;
  *) echo "usage: docker/build.sh [ngc|raw] [--push]" >&2; exit 2 ;;
esac
extra=()
for a in "$@"; do
  case "$a" in
    --push) extra+=(--push) ;;
    *) extra+=("$a") ;;
  esac
done
if docker buildx version >/dev/null 2>&1; then
  exec docker buildx bake -f docker/docker-bake.hcl "${target}" "${extra[@]}"
fi
file=docker/Dockerfile
[ "${target}" = raw ] && file=docker/Dockerfile.raw
exec docker build -f "${file}" -t "optimus-dl-b200:${TAG:-latest}${target/ngc/}" .
