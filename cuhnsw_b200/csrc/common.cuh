// Shared device-side definitions: (distance, id) keys, warp helpers, launch constants.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hnsw {

constexpr unsigned FULL = 0xffffffffu;
constexpr int DIST_DOT = 0;
constexpr int DIST_L2 = 1;

// A candidate is one 64-bit key: order-preserving image of the fp32 distance
// in the high word, node id in the low 31 bits, and bit 31 of the low word as
// the "expanded" flag (the reference keeps `checked` in its Neighbor struct,
// cpp/include/types.hpp:43-47).  Comparisons always mask the flag, so the
// order is the total order (distance, id).
constexpr unsigned long long KEY_FLAG = 0x80000000ull;
constexpr unsigned long long KEY_MASK = ~KEY_FLAG;
constexpr unsigned long long KEY_MAX = 0xffffffffffffffffull & KEY_MASK;

__device__ __forceinline__ unsigned f2ord(float x) {
  x = x + 0.0f;  // -0 -> +0: equal floats get equal keys
  unsigned u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ord2f(unsigned o) {
  unsigned u = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
  return __uint_as_float(u);
}
__device__ __forceinline__ unsigned long long mkkey(float dist, int id) {
  return ((unsigned long long)f2ord(dist) << 32) | (unsigned)id;
}
__device__ __forceinline__ int key_id(unsigned long long k) { return (int)((unsigned)k & 0x7fffffffu); }
__device__ __forceinline__ float key_dist(unsigned long long k) { return ord2f((unsigned)(k >> 32)); }

__device__ __forceinline__ unsigned long long shfl64(unsigned long long v, int src) {
  unsigned lo = __shfl_sync(FULL, (unsigned)v, src);
  unsigned hi = __shfl_sync(FULL, (unsigned)(v >> 32), src);
  return ((unsigned long long)hi << 32) | lo;
}

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// Compacts the lanes selected by `mask`: lane r (r < popc(mask)) receives the
// value held by the r-th selected lane, in lane order.
__device__ __forceinline__ int compact_i32(unsigned mask, int v) {
  int src = __fns(mask, 0, lane_id() + 1);
  return __shfl_sync(FULL, v, src & 31);
}

}  // namespace hnsw
