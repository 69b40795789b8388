// C entry point in front of the reference project's own CUDA launcher, so that its kernel can be
// run (as a checker and as a timed comparator) without the torch extension around it.
// TEST / BENCHMARK INFRASTRUCTURE ONLY: nothing in the product links or loads this.
//
// The reference's launcher is the C++ template
//   template <typename T> cudaError_t flashattention_forward(T* O, const T* Q, const T* K_mat,
//       const T* V, int seq_len, int batch_size, int num_heads);          (src/cpp/v1.cu:4-38)
// explicitly instantiated for __nv_bfloat16 (src/cpp/v1.cu:40-42) and called by the binding
// (src/cpp/torch_bind.cpp:34-39).  build_ref.py compiles the reference's v1.cu where it lies,
// unmodified, together with this file; the declaration below resolves against that instantiation.
// The launcher uses the legacy default stream and device 0's properties (v1.cu:7-8, 33-34): call
// it with device 0 current and synchronise the default stream around it.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

template <typename T>
cudaError_t flashattention_forward(T* O, const T* Q, const T* K_mat, const T* V, int seq_len,
                                   int batch_size, int num_heads);

extern "C" int ref_v1_forward(void* O, const void* Q, const void* K_mat, const void* V, int seq_len,
                              int batch_size, int num_heads) {
  return static_cast<int>(flashattention_forward<__nv_bfloat16>(
      static_cast<__nv_bfloat16*>(O), static_cast<const __nv_bfloat16*>(Q),
      static_cast<const __nv_bfloat16*>(K_mat), static_cast<const __nv_bfloat16*>(V), seq_len,
      batch_size, num_heads));
}
