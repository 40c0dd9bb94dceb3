// Pairwise distances between stored rows: the unit-test vehicle of the distance
// primitive (the reference's counterpart is BatchDistanceKernel,
// cpp/include/cuda_dist_kernels.cuh:143-156).
#include "kernels.h"
#include "beam.cuh"

namespace hnsw {

template <class Dist>
__global__ void __launch_bounds__(64) batch_distance_kernel(GraphView g, const int* src, const int* dst,
                                                            long long npairs, float* out) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Dist de;
  const VecTable tab = make_table(g);
  de.init(tab, smem + (size_t)warp * Dist::smem_bytes(g.d));
  const long long nwarps = (long long)gridDim.x * 2;
  for (long long base = ((long long)blockIdx.x * 2 + warp) * 32; base < npairs; base += nwarps * 32) {
    // one source per step of the outer loop; 32 destinations are evaluated per source when they share it,
    // here simply pair by pair so that every pair exercises load_query_row + eval
    for (int k = 0; k < 32 && base + k < npairs; ++k) {
      de.load_query_row(__ldg(src + base + k));
      float dd = de.eval(__ldg(dst + base + k), 1);
      dd = __shfl_sync(FULL, dd, 0);
      if (lane == 0) out[base + k] = dd;
    }
  }
}

template <class Dist>
static cudaError_t batch_distance_t(const GraphView& g, const int* src, const int* dst, long long npairs, float* out,
                                    cudaStream_t stream) {
  size_t smem = 2 * Dist::smem_bytes(g.d);
  cudaError_t e = cudaFuncSetAttribute(batch_distance_kernel<Dist>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem);
  if (e != cudaSuccess) return e;
  long long blocks = (npairs + 63) / 64;
  if (blocks > 148 * 8) blocks = 148 * 8;
  batch_distance_kernel<Dist><<<(unsigned)blocks, 64, smem, stream>>>(g, src, dst, npairs, out);
  return cudaGetLastError();
}

template <class Row>
static cudaError_t batch_distance_rows(const GraphView& g, const int* src, const int* dst, long long npairs, float* out,
                                       cudaStream_t stream) {
  using E = Pick<Row>;
  if (g.d <= 32) return batch_distance_t<typename E::D32>(g, src, dst, npairs, out, stream);
  if (g.d <= 64) return batch_distance_t<typename E::D64>(g, src, dst, npairs, out, stream);
  if (g.d <= 96) return batch_distance_t<typename E::D96>(g, src, dst, npairs, out, stream);
  if (g.d <= 128) return batch_distance_t<typename E::D128>(g, src, dst, npairs, out, stream);
  return batch_distance_t<typename E::Wide>(g, src, dst, npairs, out, stream);
}

int row_stride_elements(int d, int rows16) { return rows16 ? RowF16::stride(d) : RowF32::stride(d); }

cudaError_t launch_batch_distance(const GraphView& g, const int* src, const int* dst, long long npairs, float* out,
                                  cudaStream_t stream) {
  if (npairs <= 0) return cudaSuccess;
#define CALL(R) batch_distance_rows<R>(g, src, dst, npairs, out, stream)
  return HNSW_WITH_ROWS(g.rows16, CALL);
#undef CALL
}

}  // namespace hnsw
