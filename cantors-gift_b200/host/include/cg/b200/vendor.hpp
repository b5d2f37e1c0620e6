// vendor.hpp - how tensors reach VendorKernel::execute on the B200 path.
//
// The reference's interface is execute(const Operation&, void* stream)
// (include/cg/vendor/dispatch.hpp:59-61): no tensors. The cg_b200 kernels registered with the
// VendorDispatcher read device addresses from integer attributes on the operation.
#pragma once

#include <vector>

#include "cg/ir/operation.hpp"
#include "cg/vendor/dispatch.hpp"

namespace cg::b200 {

// Sets "b200.in<i>", "b200.out0" and, when given, "b200.workspace" (scratch for an fp32 matmul: without
// it the kernel allocates and frees its own, synchronising the stream).
void bind_pointers(Operation& op, const std::vector<void*>& inputs, void* output, void* workspace = nullptr);

// The registered cg_b200 kernel that can execute `op`, or nullptr. VendorDispatcher::find_best ranks by
// estimated runtime and the descriptor-only kernels of the reference win that for matmul.
VendorKernel* find_executable(const Operation& op);

}  // namespace cg::b200
