// Function-space macros shared by the tile headers. The headers under types/ compile as plain C++ too
// (layout arithmetic is usable on the host); everything under cell/ is device code for sm_100a.
// Same role as the reference's include/config.hpp:3-15.
#pragma once

#if defined(__CUDACC__)
#define HOST_DEVICE __forceinline__ __host__ __device__
#define DEVICE __forceinline__ __device__
#define HOST __forceinline__ __host__
#else
#define HOST_DEVICE inline
#define DEVICE inline
#define HOST inline
#endif
