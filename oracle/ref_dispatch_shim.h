// Test infrastructure only. Force-included when compiling the unmodified
// reference extension sources against a current PyTorch: the reference passes
// `tensor.type()` (a DeprecatedTypeProperties) to AT_DISPATCH_FLOATING_TYPES,
// which newer PyTorch no longer converts to a ScalarType. This overload
// restores that conversion without touching the reference sources.
#pragma once
#include <ATen/ATen.h>
#include <ATen/Dispatch.h>
namespace detail {
inline at::ScalarType scalar_type(const at::DeprecatedTypeProperties& t) {
    return t.scalarType();
}
}  // namespace detail
