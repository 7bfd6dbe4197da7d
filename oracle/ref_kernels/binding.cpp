// Python binding for two of the reference's own CUDA kernels, compiled from the reference checkout where it lies
// (never copied): kernels/chipmunk/csrc/indexed_io/mask_to_indices.cu and topk_indices.cu.  Test infrastructure
// only: the GPU tests run them beside this package's kernels to pin the oracle's restatement of their output.
#include <torch/extension.h>

#include <vector>

namespace chipmunk {
std::vector<at::Tensor> mask_to_indices(at::Tensor mask, int64_t multiple_of, int64_t pad_to_multiple_of);
void topk_indices(at::Tensor activation, at::Tensor indices, at::Tensor counts, double sparsity_amount,
                  int64_t multiple_of, double random_amount);
}  // namespace chipmunk

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("mask_to_indices", &chipmunk::mask_to_indices, "reference mask -> (indices, counts)");
  m.def("topk_indices", &chipmunk::topk_indices, "reference sampled-quantile top-k");
}
