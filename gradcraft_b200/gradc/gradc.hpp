// Umbrella header: `#include "gradc/gradc.hpp"` as programs written against GradCraft do.
#pragma once
#include "base.hpp"     // IWYU pragma: keep
#include "runtime.hpp"  // IWYU pragma: keep
#include "tensor.hpp"   // IWYU pragma: keep
#include "ops.hpp"      // IWYU pragma: keep
#include "nn.hpp"       // IWYU pragma: keep
