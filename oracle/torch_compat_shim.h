// Force-included (-include) when the reference's SpMM / SpCONV CUDA sources are compiled into
// oracle/_ref (test infrastructure only).  Those sources dispatch with
// AT_DISPATCH_FLOATING_TYPES(tensor.type(), ...); the overload of ::detail::scalar_type that takes
// the deprecated type-properties object was removed from newer ATen releases.  Restoring it here
// lets the reference sources compile unmodified, where they lie.
#pragma once
#include <ATen/ATen.h>
#include <ATen/Dispatch.h>
#include <ATen/core/DeprecatedTypeProperties.h>

namespace detail {
inline at::ScalarType scalar_type(const at::DeprecatedTypeProperties &t) { return t.scalarType(); }
}  // namespace detail
