// Forwarding header: the detail:: helpers live in sca_api.hpp.
#pragma once
#include "scicompute_attention/sca_api.hpp"
