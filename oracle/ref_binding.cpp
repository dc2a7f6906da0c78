// Exposes the reference's own CPU implementations (grm/csrc/grm_cuda.cpp,
// compiled from where it lies in the reference checkout) under the op
// namespace torch.ops.grm_ref.* so that tests and the benchmark can call the
// unmodified reference math on CPU tensors.  TEST INFRASTRUCTURE ONLY: the
// product package never loads this library.
//
// The reference's own registration file (grm/csrc/bindings.cpp) is not used:
// it also binds the CUDA entry points, which are not compiled here.
#include <torch/extension.h>

#include "grm_cuda.h"

TORCH_LIBRARY(grm_ref, m) {
  m.def("chunk_update_forward(Tensor keys, Tensor values, Tensor queries, Tensor memory, float memory_decay) -> (Tensor, Tensor, Tensor)");
  m.def("chunk_update_backward(Tensor grad_hidden, Tensor grad_memory_out, Tensor keys, Tensor values, Tensor queries, Tensor memory, Tensor aux, float memory_decay) -> (Tensor, Tensor, Tensor, Tensor)");
  m.def("apply_query_forward(Tensor memories, Tensor queries) -> Tensor");
  m.def("apply_query_backward(Tensor grad_hidden, Tensor memories, Tensor queries) -> (Tensor, Tensor)");
  m.def("batched_memory_gather(Tensor memories_per_batch, Tensor topk_indices) -> Tensor");
}

TORCH_LIBRARY_IMPL(grm_ref, CPU, m) {
  m.impl("chunk_update_forward", grm::chunk_update_forward);
  m.impl("chunk_update_backward", grm::chunk_update_backward);
  m.impl("apply_query_forward", grm::apply_query_forward);
  m.impl("apply_query_backward", grm::apply_query_backward);
  m.impl("batched_memory_gather", grm::batched_memory_gather);
}
