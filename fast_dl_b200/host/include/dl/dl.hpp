// Umbrella header: everything a user of the library includes.
#pragma once

#include <dl/core/Types.hpp>
#include <dl/nn/nn.hpp>
#include <dl/ops/Ops.hpp>
#include <dl/tensor/Tensor.hpp>
