// Host side of the bounds-check build: the device record of the first out-of-range index.
#include "axb_common.cuh"

#ifdef AXB_BOUNDS_CHECK
__device__ unsigned long long axb_bounds_record[4] = {0ull, 0ull, 0ull, 0ull};
#endif

extern "C" int axb_bounds_check_enabled() {
#ifdef AXB_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}

// out[0..3] = site (0 = no violation), index, limit, number of violations seen
extern "C" int axb_bounds_fetch(long long* out) {
#ifdef AXB_BOUNDS_CHECK
  unsigned long long h[4];
  cudaError_t e = cudaMemcpyFromSymbol(h, axb_bounds_record, sizeof(h));
  if (e != cudaSuccess) return (int)e;
  for (int i = 0; i < 4; ++i) out[i] = (long long)h[i];
  return 0;
#else
  for (int i = 0; i < 4; ++i) out[i] = 0;
  return 0;
#endif
}

extern "C" int axb_bounds_reset() {
#ifdef AXB_BOUNDS_CHECK
  const unsigned long long z[4] = {0ull, 0ull, 0ull, 0ull};
  return (int)cudaMemcpyToSymbol(axb_bounds_record, z, sizeof(z));
#else
  return 0;
#endif
}
