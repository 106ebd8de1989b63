// Qualifier macros shared by the cusync headers.  Same macro names as the
// reference (src/include/cusync/cusync_defines.h) so user code written against
// it keeps compiling.
#pragma once

#if defined(__CUDACC__) || defined(__NVCC__)
  #define CUSYNC_DEVICE      __device__ __forceinline__
  #define CUSYNC_HOST        __host__ __forceinline__
  #define CUSYNC_DEVICE_HOST __device__ __host__ __forceinline__
  #define CUSYNC_GLOBAL      __global__
#else
  #define CUSYNC_DEVICE      inline
  #define CUSYNC_HOST        inline
  #define CUSYNC_DEVICE_HOST inline
  #define CUSYNC_GLOBAL
#endif
