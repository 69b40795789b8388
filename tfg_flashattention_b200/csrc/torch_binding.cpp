// pybind11 / torch-extension binding of the attention forward: the compiled counterpart of the
// reference's src/cpp/torch_bind.cpp:21-49 (`PYBIND11_MODULE ... m.def("forward", ...)`), in front
// of this library's C ABI (include/fa_b200.h) instead of the reference's launcher template.
//
//   forward(Q, K_mat, V, causal=True, return_lse=False, softmax_scale=None, out=None)
//
// Three positional tensors behave as the reference's binding: CUDA + bfloat16 checked the same way
// (CHECK_CUDA / the dtype branch, torch_bind.cpp:13-19, 33-42), O = empty_like(Q) (:31), causal,
// scale 1/sqrt(64), returns O.  Differences: size(3) is checked (the reference assumes 64), tensors
// need not be contiguous (strides go to the library, which reads `[B,N,H,d]` views in place), the
// launch goes to the current stream of Q's device, the GIL is released around the library call,
// and the library's error code becomes a RuntimeError (the reference drops its cudaError_t).
// PyTorch is used for what it owns: tensors, the current device and stream.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "../../include/fa_b200.h"

namespace {

// Argument and library errors leave as std::runtime_error, which pybind11 turns into the same
// Python RuntimeError that TORCH_CHECK produces in the reference binding.
#define FA_CHECK(cond, ...)                                        \
  do {                                                             \
    if (!(cond)) throw std::runtime_error(c10::str(__VA_ARGS__)); \
  } while (0)

void check_input(const torch::Tensor& t, const char* name) {
  FA_CHECK(t.device().is_cuda(), name, " must be a CUDA tensor");
  FA_CHECK(t.scalar_type() == torch::kBFloat16, "Unsupported tensor dtype. Use bfloat16.");
  FA_CHECK(t.dim() == 4, name, " must have shape [B, H, N, d]");
}

// Element strides {batch, head, row}; strides of size-1 dimensions are never dereferenced, so they
// are replaced by a canonical value that always passes the library's checks.
void strides3(const torch::Tensor& t, const char* name, int64_t out[3]) {
  const int64_t H = t.size(1), N = t.size(2), d = t.size(3);
  FA_CHECK(d <= 1 || t.stride(3) == 1, name, ": the last dimension must be dense (stride 1)");
  int64_t sb = t.stride(0), sh = t.stride(1), sn = t.stride(2);
  if (N == 1) sn = d;
  if (H == 1) sh = std::max<int64_t>(N * sn, 8);
  if (t.size(0) == 1) sb = std::max<int64_t>(std::max(H * sh, N * sn), 8);
  out[0] = sb; out[1] = sh; out[2] = sn;
}

py::object forward(const torch::Tensor& Q, const torch::Tensor& K_mat, const torch::Tensor& V, bool causal,
                   bool return_lse, const c10::optional<double>& softmax_scale,
                   const c10::optional<torch::Tensor>& out) {
  check_input(Q, "Q");
  check_input(K_mat, "K_mat");
  check_input(V, "V");
  FA_CHECK(K_mat.sizes() == Q.sizes() && V.sizes() == Q.sizes(),
              "Q, K_mat and V must have the same shape [B, H, N, d]");
  FA_CHECK(K_mat.device() == Q.device() && V.device() == Q.device(),
              "Q, K_mat and V must be on the same device");
  torch::Tensor O;
  if (out.has_value()) {
    check_input(*out, "out");
    FA_CHECK(out->sizes() == Q.sizes() && out->device() == Q.device(), "out must match Q in shape and device");
    O = *out;
  } else {
    O = torch::empty_like(Q);   // same allocation rule as the reference (torch_bind.cpp:31)
  }
  const c10::cuda::CUDAGuard guard(Q.device());
  torch::Tensor lse;
  if (return_lse) lse = torch::empty({Q.size(0), Q.size(1), Q.size(2)}, Q.options().dtype(torch::kFloat32));

  fa_b200_params p{};
  p.B = static_cast<int32_t>(Q.size(0));
  p.H = static_cast<int32_t>(Q.size(1));
  p.N = static_cast<int32_t>(Q.size(2));
  p.d = static_cast<int32_t>(Q.size(3));
  if (Q.numel() > 0) {
    p.q = Q.data_ptr(); p.k = K_mat.data_ptr(); p.v = V.data_ptr(); p.o = O.data_ptr();
    strides3(Q, "Q", p.q_strides);
    strides3(K_mat, "K_mat", p.k_strides);
    strides3(V, "V", p.v_strides);
    strides3(O, "out", p.o_strides);
  } else {            // empty problem: nothing is read, any valid pointers and strides do
    p.q = p.k = p.v = p.o = reinterpret_cast<void*>(16);
    for (int i = 0; i < 3; ++i) p.q_strides[i] = p.k_strides[i] = p.v_strides[i] = p.o_strides[i] = 8;
  }
  p.lse = return_lse && Q.numel() > 0 ? lse.data_ptr<float>() : nullptr;
  p.softmax_scale = softmax_scale.has_value() ? static_cast<float>(*softmax_scale) : 0.0f;
  p.causal = causal ? 1 : 0;
  p.device = Q.device().index();
  p.stream = c10::cuda::getCurrentCUDAStream(Q.device().index()).stream();
  int rc;
  {
    py::gil_scoped_release release;
    rc = fa_b200_fwd(&p);
  }
  FA_CHECK(rc == 0, "custom_flash_attn.forward failed (", rc, "): ", fa_b200_strerror(rc));
  if (return_lse) return py::make_tuple(O, lse);
  return py::cast(O);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("forward", &forward, "FlashAttention forward on B200 (libfa_b200.so)", py::arg("Q"), py::arg("K_mat"),
        py::arg("V"), py::arg("causal") = true, py::arg("return_lse") = false,
        py::arg("softmax_scale") = py::none(), py::arg("out") = py::none());
  m.attr("abi_version") = FA_B200_ABI_VERSION;   // the header this module was compiled against
}
