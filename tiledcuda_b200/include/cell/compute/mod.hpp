#pragma once

#include "cell/compute/broadcast.hpp"
#include "cell/compute/gemm.hpp"
#include "cell/compute/map.hpp"
#include "cell/compute/math_functor.hpp"
#include "cell/compute/reduce.hpp"
#include "cell/compute/softmax.hpp"
