// PyTorch extension `ms_blkq4linear_ext`: the host-side mirror of the reference's
// python/ms_blkq4linear_ext/ms_blkq4linear.cpp (quant :13-72, forward :74-117,
// module definition :120-123).  Same function names, argument order and checks;
// tensors are reduced to device pointers and byte sizes and handed to the C ABI in
// include/ms_blkq4gemm.h.  Differences, all additive:
//   - work is enqueued on PyTorch's current CUDA stream (the reference passes the
//     legacy default stream), so the calls compose with CUDA graphs and side streams;
//   - with has_offsets == false `quant` returns an empty uint8 tensor for the zero
//     points (the reference returns an undefined tensor, which its own `forward`
//     cannot accept);
//   - `forward_out` writes into a caller-provided output tensor and takes an optional fp16 bias
//     (added in the kernel epilogue, bit-identical to `output += bias`) and the flags of
//     blkq4_fp16_gemm_sm100.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <cstddef>
#include <cstdint>

#include "ms_blkq4gemm.h"

namespace {

constexpr size_t kHalfBytes = 2;

std::vector<torch::Tensor> blkq4linear_quant(int block_size, bool col_wise, bool has_offsets,
                                             torch::Tensor weights) {
  TORCH_CHECK(weights.scalar_type() == torch::kFloat16, "blkq4linear_quant only supports float16 weights");
  TORCH_CHECK(weights.numel() > 0, "blkq4linear_quant only supports non-empty tensors");
  TORCH_CHECK(weights.is_contiguous(), "blkq4linear_quant only supports contiguous tensors");
  TORCH_CHECK(weights.dim() == 2, "blkq4linear_quant only supports 2D tensors");
  TORCH_CHECK(weights.device().type() == at::kCUDA,
              "blkq4linear_quant only supports CUDA tensors, instead got ", weights.device().str());
  const int64_t out_features = weights.size(0);
  const int64_t in_features = weights.size(1);

  std::string err;
  int64_t w_size = 0, meta_size = 0;
  int rc = blkq4_fp16_quant_size_sm80(block_size, col_wise, int(in_features), int(out_features), w_size,
                                      meta_size, &err);
  TORCH_CHECK(rc == 0, err);

  const c10::cuda::CUDAGuard guard(weights.device());
  auto u8 = torch::TensorOptions().dtype(torch::kUInt8).device(weights.device());
  auto f16 = torch::TensorOptions().dtype(torch::kFloat16).device(weights.device());
  torch::Tensor q_weights = torch::empty({w_size}, u8);
  torch::Tensor q_scales = torch::empty({meta_size}, f16);
  torch::Tensor q_zp = torch::empty({has_offsets ? meta_size : 0}, u8);

  rc = blkq4_fp16_quant_sm80(block_size, col_wise, int(in_features), int(out_features), int(in_features),
                             c10::cuda::getCurrentCUDAStream().stream(), weights.data_ptr(),
                             size_t(weights.numel()) * kHalfBytes, q_weights.data_ptr(), size_t(w_size),
                             q_scales.data_ptr(), size_t(meta_size) * kHalfBytes,
                             has_offsets ? q_zp.data_ptr() : nullptr, has_offsets ? size_t(meta_size) : 0,
                             &err);
  TORCH_CHECK(rc == 0, err);
  return {q_weights, q_scales, q_zp};
}

torch::Tensor blkq4linear_forward_out(int block_size, bool col_wise, int in_features, int out_features,
                                      torch::Tensor input, torch::Tensor q_weights, torch::Tensor q_scales,
                                      torch::Tensor q_zp, torch::Tensor output,
                                      c10::optional<torch::Tensor> bias, int64_t flags,
                                      c10::optional<torch::Tensor> workspace) {
  TORCH_CHECK(input.scalar_type() == torch::kFloat16, "blkq4linear_forward only supports float16 inputs");
  TORCH_CHECK(input.dim() == 2 && input.size(1) == in_features,
              "Activation shape is not compatible with the weights");
  TORCH_CHECK(input.device().type() == torch::kCUDA, "blkq4linear_forward only supports CUDA inputs");
  TORCH_CHECK(input.is_contiguous(), "blkq4linear_forward only supports contiguous inputs");
  const auto dev = input.device();
  TORCH_CHECK(q_weights.device() == dev && q_scales.device() == dev &&
                  (!q_zp.defined() || q_zp.numel() == 0 || q_zp.device() == dev) && output.device() == dev,
              "blkq4linear_forward requires all tensors on the same device");
  TORCH_CHECK(output.scalar_type() == torch::kFloat16 && output.is_contiguous() && output.dim() == 2 &&
                  output.size(0) == input.size(0) && output.size(1) == out_features,
              "Output tensor must be a contiguous float16 [batch, out_features] tensor");

  const bool has_bias = bias.has_value() && bias->defined() && bias->numel() > 0;
  if (has_bias)
    TORCH_CHECK(bias->scalar_type() == torch::kFloat16 && bias->is_contiguous() && bias->device() == dev &&
                    bias->numel() == out_features,
                "Fused bias must be a contiguous float16 [out_features] tensor on the input's device");

  const c10::cuda::CUDAGuard guard(dev);
  const bool has_zp = q_zp.defined() && q_zp.numel() > 0;
  std::string err;
  const bool has_ws = workspace.has_value() && workspace->defined() && workspace->numel() > 0;
  if (has_ws)
    TORCH_CHECK(workspace->device() == dev && workspace->is_contiguous(),
                "The split-K workspace must be a contiguous tensor on the input's device");
  int rc = blkq4_fp16_gemm_ws_sm100(block_size, col_wise, int(input.size(0)), out_features, in_features,
                                 c10::cuda::getCurrentCUDAStream().stream(), input.data_ptr(),
                                 size_t(input.numel()) * kHalfBytes, q_weights.data_ptr(),
                                size_t(q_weights.numel()), q_scales.data_ptr(),
                                size_t(q_scales.numel()) * kHalfBytes, has_zp ? q_zp.data_ptr() : nullptr,
                                has_zp ? size_t(q_zp.numel()) : 0, output.data_ptr(),
                                size_t(output.numel()) * kHalfBytes, has_bias ? bias->data_ptr() : nullptr,
                                has_bias ? size_t(bias->numel()) * kHalfBytes : 0, unsigned(flags),
                                has_ws ? workspace->data_ptr() : nullptr,
                                has_ws ? size_t(workspace->numel()) * workspace->element_size() : 0, &err);
  TORCH_CHECK(rc == 0, err);
  return output;
}

torch::Tensor blkq4linear_forward(int block_size, bool col_wise, int in_features, int out_features,
                                  torch::Tensor input, torch::Tensor q_weights, torch::Tensor q_scales,
                                  torch::Tensor q_zp) {
  TORCH_CHECK(input.dim() == 2, "Activation shape is not compatible with the weights");
  auto output = torch::empty({input.size(0), out_features},
                             torch::TensorOptions().dtype(torch::kFloat16).device(input.device()));
  return blkq4linear_forward_out(block_size, col_wise, in_features, out_features, input, q_weights, q_scales,
                                 q_zp, output, c10::nullopt, 0, c10::nullopt);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("quant", &blkq4linear_quant, "Quantize float 16 weights");
  m.def("forward", &blkq4linear_forward, "Forward pass for block quantized linear layer");
  m.def("forward_out", &blkq4linear_forward_out, "Forward pass into a caller-provided output tensor",
        py::arg("block_size"), py::arg("col_wise"), py::arg("in_features"), py::arg("out_features"),
        py::arg("input"), py::arg("q_weights"), py::arg("q_scales"), py::arg("q_zp"), py::arg("output"),
        py::arg("bias") = py::none(), py::arg("flags") = 0, py::arg("workspace") = py::none());
  m.def("gemm_workspace_size", [](int m_, int n_, int k_) { return int64_t(blkq4_gemm_workspace_size(m_, n_, k_)); },
        "Bytes of zeroed workspace with which the tensor-core kernel splits K (0: it does not)");
  m.attr("EARLY_WEIGHT_FETCH") = int(BLKQ4_GEMM_EARLY_WEIGHT_FETCH);
  m.def("library_version", []() { return std::string(blkq4_version()); });
}
