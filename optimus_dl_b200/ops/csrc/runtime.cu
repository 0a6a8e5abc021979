// Per-thread runtime binding.
//
// This library links its own copy of the CUDA runtime.  A host thread that has made no runtime
// call yet (for example an autograd worker thread) has no current context, and a driver-level
// call such as the tensor-map encoder would fail there; binding the device once per thread
// makes the device's primary context current for every later launcher call on that thread.
#include <cuda_runtime.h>

extern "C" int ob_bind_thread(int device) {
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaFree(0);
}
