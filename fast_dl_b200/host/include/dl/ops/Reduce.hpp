#pragma once
#include <dl/ops/Ops.hpp>  // all dl::ops declarations live there
