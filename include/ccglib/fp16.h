// Forwarding header: half-precision storage type used by callers of the reference API.
#pragma once
#include <cuda_fp16.h>
