#pragma once
// Kept for include-path compatibility; the declarations live in legacy_interfaces.hpp.
#include "legacy_interfaces.hpp"
