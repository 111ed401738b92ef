// Forwarding header: 8-bit float storage types used by callers of the reference API.
#pragma once
#include <cuda_fp8.h>
using fp8_e4m3 = __nv_fp8_e4m3;
using fp8_e5m2 = __nv_fp8_e5m2;
