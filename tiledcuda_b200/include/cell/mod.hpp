// Device-side building blocks ("macro kernels") of the B200-native TiledCUDA surface; same include path
// as the reference's include/cell/mod.hpp:3-10.
#pragma once

#include "cell/compute/mod.hpp"
#include "cell/copy/mod.hpp"
#include "cell/sync.hpp"
#include "cell/traits/base.hpp"
#include "cell/warp.hpp"
