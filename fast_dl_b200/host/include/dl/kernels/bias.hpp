#pragma once
#include <dl/kernels/kernels.hpp>  // all dl::kernels declarations live there
