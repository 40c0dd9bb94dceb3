// Test vehicles for the two shared-memory structures of the walk kernels, so that they can be checked in
// isolation against a host model: the sorted candidate/result list (semantics of PushNodeToSearchPq,
// cpp/include/cuda_utils_kernels.cuh:212-227 of the reference: insert while there is room, else replace the
// largest key if the new one is smaller; CheckAlreadyExists, :50-103: no key twice) and the visited table
// (CheckVisited, :185-210: may forget, must never report an id it has not seen).
// One warp, one CTA; not used by any search or build.
#include "beam.cuh"
#include "kernels.h"

namespace hnsw {

// Merges `nbatches` batches of up to 32 (distance, id) pairs into a list of capacity `cap`.  After batch b
// ends, out_minpos[b] = what merge() returned.  Before batch b the first `expand[b]` unexpanded keys are
// flagged as expanded through the cursor, as a walk would, so that flags have to survive the shifts.
__global__ void __launch_bounds__(32) selftest_list_kernel(int cap, const float* dist, const int* ids,
                                                           const int* batch_begin, int nbatches, const int* expand,
                                                           unsigned long long* out_keys, int* out_size,
                                                           int* out_minpos, int* out_cursor) {
  extern __shared__ __align__(16) unsigned char smem[];
  WarpList wl;
  wl.bind(smem, cap, 64, 1 << 20);
  wl.reset();
  WalkCounters wc{0, 0, 0, 0};
  const int lane = lane_id();
  for (int b = 0; b < nbatches; ++b) {
    for (int e = 0; e < expand[b]; ++e) {
      wl.advance();
      if (wl.cursor >= wl.size) break;
      if (lane == 0) wl.keys[wl.cursor] |= KEY_FLAG;
      __syncwarp();
    }
    const int lo = batch_begin[b], n = batch_begin[b + 1] - lo;
    const bool active = lane < n;
    const unsigned long long key = active ? mkkey(dist[lo + lane], ids[lo + lane]) : 0ull;
    const int mp = wl.merge(key, active, wc);
    if (lane == 0) out_minpos[b] = mp;
    __syncwarp();
  }
  wl.advance();
  for (int i = lane; i < wl.size; i += 32) out_keys[i] = wl.keys[i];
  if (lane == 0) {
    *out_size = wl.size;
    *out_cursor = wl.cursor;
  }
}

// Feeds `count` ids to a visited table of `entries` entries for an index of n nodes, one after the other;
// seen[i] = 1 when the table claimed to have seen ids[i] before.
__global__ void __launch_bounds__(32) selftest_visited_kernel(int entries, long long n, const int* ids, int count,
                                                              int* seen) {
  extern __shared__ __align__(16) unsigned char smem[];
  WarpList wl;
  wl.bind(smem, 32, entries, n);
  wl.reset();
  if (lane_id() == 0)
    for (int i = 0; i < count; ++i) seen[i] = wl.test_and_set(ids[i]) ? 1 : 0;
}

namespace {
// device copy of a host array for the lifetime of one self-test call
template <class T>
struct Mirror {
  T* d = nullptr;
  size_t n = 0;
  cudaError_t up(const T* h, size_t count) {
    n = count;
    cudaError_t e = cudaMalloc(&d, (count ? count : 1) * sizeof(T));
    if (e == cudaSuccess && h && count) e = cudaMemcpy(d, h, count * sizeof(T), cudaMemcpyHostToDevice);
    return e;
  }
  cudaError_t down(T* h) const { return n ? cudaMemcpy(h, d, n * sizeof(T), cudaMemcpyDeviceToHost) : cudaSuccess; }
  ~Mirror() { cudaFree(d); }
};
}  // namespace

cudaError_t launch_selftest_list(int cap, const float* dist, const int* ids, const int* batch_begin, int nbatches,
                                 const int* expand, unsigned long long* out_keys, int* out_size, int* out_minpos,
                                 int* out_cursor, cudaStream_t stream) {
  const size_t smem = WarpList::smem_bytes(cap, 64, 1 << 20);
  cudaError_t e = cudaFuncSetAttribute(selftest_list_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  selftest_list_kernel<<<1, 32, smem, stream>>>(cap, dist, ids, batch_begin, nbatches, expand, out_keys, out_size,
                                                out_minpos, out_cursor);
  return cudaGetLastError();
}

cudaError_t launch_selftest_visited(int entries, long long n, const int* ids, int count, int* seen,
                                    cudaStream_t stream) {
  const size_t smem = WarpList::smem_bytes(32, entries, n);
  cudaError_t e =
      cudaFuncSetAttribute(selftest_visited_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  selftest_visited_kernel<<<1, 32, smem, stream>>>(entries, n, ids, count, seen);
  return cudaGetLastError();
}

#define ST(call)                    \
  do {                              \
    cudaError_t e__ = (call);       \
    if (e__ != cudaSuccess) return e__; \
  } while (0)

cudaError_t selftest_list_host(int cap, const float* dist, const int* ids, const int* batch_begin, int nbatches,
                               const int* expand, unsigned long long* out_keys, int* out_size, int* out_minpos,
                               int* out_cursor) {
  const size_t total = (size_t)batch_begin[nbatches];
  Mirror<float> d_dist;
  Mirror<int> d_ids, d_begin, d_expand, d_size, d_minpos, d_cursor;
  Mirror<unsigned long long> d_keys;
  ST(d_dist.up(dist, total));
  ST(d_ids.up(ids, total));
  ST(d_begin.up(batch_begin, (size_t)nbatches + 1));
  ST(d_expand.up(expand, (size_t)nbatches));
  ST(d_keys.up(nullptr, (size_t)cap));
  ST(d_size.up(nullptr, 1));
  ST(d_minpos.up(nullptr, (size_t)nbatches));
  ST(d_cursor.up(nullptr, 1));
  ST(cudaMemset(d_keys.d, 0, (size_t)cap * sizeof(unsigned long long)));
  ST(launch_selftest_list(cap, d_dist.d, d_ids.d, d_begin.d, nbatches, d_expand.d, d_keys.d, d_size.d, d_minpos.d,
                          d_cursor.d, nullptr));
  ST(cudaDeviceSynchronize());
  ST(d_keys.down(out_keys));
  ST(d_size.down(out_size));
  ST(d_minpos.down(out_minpos));
  return d_cursor.down(out_cursor);
}

cudaError_t selftest_visited_host(int entries, long long n, const int* ids, int count, int* seen) {
  Mirror<int> d_ids, d_seen;
  ST(d_ids.up(ids, (size_t)count));
  ST(d_seen.up(nullptr, (size_t)count));
  ST(launch_selftest_visited(entries, n, d_ids.d, count, d_seen.d, nullptr));
  ST(cudaDeviceSynchronize());
  return d_seen.down(seen);
}
#undef ST

}  // namespace hnsw
