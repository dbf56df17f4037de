#pragma once
#include <dl/nn/nn.hpp>  // all dl::nn classes live there
