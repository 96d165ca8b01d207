// torch.ops.xpool.ffn_shim as a native operator: the schema of the reference's op (src/cext-bindings/ops.cpp:1-44)
// with a CUDA implementation that goes straight to the Instance transport (kernels/instance.cu) on the caller's
// current stream, so a serving engine can capture it into its decode graphs. The CPU key is left to Python
// (integrations/sglang/shim.py registers a callable there for engine-less tests).
#include <ATen/cuda/CUDAContext.h>
#include <torch/library.h>

#include "xpool/api.h"

namespace {

void ffn_shim_cuda(const at::Tensor& hidden_states, const c10::optional<at::Tensor>& dp_rank_payload_rows, at::Tensor& output,
                   int64_t layer_ordinal, int64_t forward_mode, int64_t output_requirement, int64_t dp_row_layout) {
  TORCH_CHECK(hidden_states.dim() == 2 && output.dim() == 2, "xpool::ffn_shim: hidden_states and output must be [rows, hidden]");
  TORCH_CHECK(hidden_states.scalar_type() == at::kBFloat16 && output.scalar_type() == at::kBFloat16,
              "xpool::ffn_shim: the payload dtype of this build is bfloat16");
  TORCH_CHECK(hidden_states.stride(1) == 1 && output.stride(1) == 1, "xpool::ffn_shim: rows must be contiguous");
  TORCH_CHECK(hidden_states.size(0) == output.size(0) && hidden_states.size(1) == output.size(1), "xpool::ffn_shim: shape mismatch");
  TORCH_CHECK(!dp_rank_payload_rows.has_value() || dp_row_layout != 0, "xpool::ffn_shim: a row table needs a data-parallel layout");
  const int handle = xp_instance_current();
  TORCH_CHECK(handle >= 0, "xpool::ffn_shim called before an Instance runtime was bound");
  const int rc = xp_instance_submit(handle, hidden_states.data_ptr(), static_cast<int>(hidden_states.size(0)),
                                    static_cast<int>(hidden_states.stride(0)), output.data_ptr(), static_cast<int>(output.stride(0)),
                                    static_cast<int>(layer_ordinal), static_cast<int>(forward_mode),
                                    static_cast<int>(output_requirement), static_cast<int>(dp_row_layout),
                                    at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "xpool::ffn_shim: submit failed with code ", rc);
}

}  // namespace

TORCH_LIBRARY(xpool, m) {
  m.def(
      "ffn_shim(Tensor hidden_states, Tensor? dp_rank_payload_rows, Tensor(a!) output, int layer_ordinal, int forward_mode, "
      "int output_requirement, int dp_row_layout) -> ()");
}

TORCH_LIBRARY_IMPL(xpool, CUDA, m) { m.impl("ffn_shim", &ffn_shim_cuda); }
