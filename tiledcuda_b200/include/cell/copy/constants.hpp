// Copy vocabulary kept from the reference (include/cell/copy/constants.hpp:7-26).
//
// WarpReuse says which warps of a WarpLayout grid load the same data. With mma.sync every warp needs its
// own register copy of the A / B sub-tiles it multiplies, hence kRowReuse / kColReuse. tcgen05.mma reads
// its operands straight from shared memory, so no operand is ever replicated into registers; the enum is
// accepted by the loaders for source compatibility and only kCont has an effect.
#pragma once

namespace tiledcuda::cell::copy {

enum class CopyInst {
    kLoadMat = 0,     // ldmatrix in the reference; here: operands stay in shared memory (descriptor)
    kStoreMat = 1,
    kLoadShared32 = 2,
    kLoadShared128 = 3,
    kTma = 4,         // cp.async.bulk.tensor through a CUtensorMap
    kTmemLoad = 5     // tcgen05.ld
};

enum class WarpReuse {
    kCont = 0,      // every warp handles its own contiguous part
    kCir = 1,
    kRowReuse = 2,  // accepted, treated as kCont
    kColReuse = 3,  // accepted, treated as kCont
    kRowReuseCont = 4,
    kRowReuseCir = 5,
    kColReuseCont = 6,
    kColReuseCir = 7
};

}  // namespace tiledcuda::cell::copy
