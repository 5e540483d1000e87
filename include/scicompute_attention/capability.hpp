// Forwarding header: the whole public API lives in sca_api.hpp.
#pragma once
#include "scicompute_attention/sca_api.hpp"
