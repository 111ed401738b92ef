// Forwarding header: this include path of the reference API is served by <ccglib/b200_api.hpp>.
#pragma once
#include <ccglib/b200_api.hpp>
#include <ccglib/gemm/reference.h>
