// Forwarding header: bfloat16 storage type used by callers of the reference API.
#pragma once
#include <cuda_bf16.h>
using bf16 = __nv_bfloat16;
