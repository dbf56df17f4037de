#pragma once
#include <dl/core/Types.hpp>  // DType lives there
