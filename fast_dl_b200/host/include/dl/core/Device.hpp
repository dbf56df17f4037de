#pragma once
#include <dl/core/Types.hpp>  // Device lives there
