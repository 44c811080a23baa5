// Tile vocabulary of the B200-native TiledCUDA surface (same include path as the reference's
// include/types/mod.hpp:3-9, plus the TMEM tile that tcgen05 adds).
#pragma once

#include "types/global.hpp"
#include "types/global_tile_iterator.hpp"
#include "types/layout.hpp"
#include "types/register.hpp"
#include "types/shared.hpp"
#include "types/shared_tile_iterator.hpp"
#include "types/tile_shape.hpp"
#include "types/tmem.hpp"
