// docker buildx bake -f docker/docker-bake.hcl [ngc|raw]
variable "REGISTRY" { default = "" }
variable "TAG" { default = "latest" }
variable "CUDA_IMAGE" { default = "nvidia/cuda:12.9.1-cudnn-devel-ubuntu24.04" }
variable "NGC_IMAGE" { default = "nvcr.io/nvidia/pytorch:25.09-py3" }
variable "NCCL_VERSION" { default = "v2.28.9-1" }
variable "TORCH_VERSION" { default = "v2.11.0" }

group "default" { targets = ["ngc"] }

target "_common" {
  context   = "."
  platforms = ["linux/amd64"]
}

// short path: NGC PyTorch image + this package
target "ngc" {
  inherits   = ["_common"]
  dockerfile = "docker/Dockerfile"
  args       = { BASE = "${NGC_IMAGE}" }
  tags       = ["${REGISTRY}optimus-dl-b200:${TAG}"]
}

// everything from source, sm_100a only
target "raw" {
  inherits   = ["_common"]
  dockerfile = "docker/Dockerfile.raw"
  args = {
    CUDA_IMAGE    = "${CUDA_IMAGE}"
    NCCL_VERSION  = "${NCCL_VERSION}"
    TORCH_VERSION = "${TORCH_VERSION}"
  }
  tags = ["${REGISTRY}optimus-dl-b200:${TAG}-raw"]
}
