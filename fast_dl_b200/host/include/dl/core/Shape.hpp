#pragma once
#include <dl/core/Types.hpp>  // Shape lives there
