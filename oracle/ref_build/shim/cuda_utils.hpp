// Stands in for the reference's include/cuda_utils.hpp when its host-only flash attention oracle is
// compiled on its own: that oracle needs nothing from the real header except the fp16 type.
#pragma once
#include <cuda_fp16.h>

#include <cmath>
