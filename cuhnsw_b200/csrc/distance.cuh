// Canonical fp32 distance for warps (replaces cpp/include/cuda_dist_kernels.cuh:13-140
// of the reference: block-strided scalar loads + shared-memory broadcast).
//
// Summation order (identical in the CPU oracle, so distances are bit-equal):
//   W = 32 accumulators when d <= 128, else 128.  Element i is fused-multiply-
//   added into accumulator (i mod W) in increasing i.  A "team" of T = W/4
//   lanes owns one row; lane t owns accumulators 4t..4t+3, i.e. the float4
//   chunks t, t+T, t+2T, ... of the row, so every load is a 16-byte vector and
//   a team reads T*16 contiguous bytes per instruction.  The four accumulators
//   of a lane fold as (a0+a1)+(a2+a3); lanes fold by an xor butterfly with
//   offsets T/2..1.  DOT returns -sum, L2 the squared distance
//   (cuda_dist_kernels.cuh:112-124).
//
// fp32 rows are stored in element order, padded with zeros to a multiple of 8 floats (32-byte sectors).
//
// 16-bit rows (IEEE half or bfloat16, round to nearest even of the input) keep the same lanes, accumulators and order of
// additions, so they give exactly the canonical fp32 distance over the rounded values; only the layout
// differs, so that a lane still loads 16 bytes at a time: a chunk is four consecutive elements, a lane owns
// chunk columns c = 0, 1, 2, ... (chunk number lane + T*c), and the 8 halves of its columns 2p and 2p + 1
// are stored side by side at 16-byte slot p*T + lane of the row.  Rows are padded with zeros to whole pairs
// of columns (T*16 bytes).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace hnsw {

struct VecTable {
  const unsigned char* vec;  // n rows
  size_t row_bytes;          // row stride
  int nchunk;                // ceil(d / 4): chunks that hold data
  int d;
  int dist_type;
};

// Storage types of a row.  load<N, T>(row, lane, c0, nchunk, v): chunk columns c0 .. c0 + N - 1 of team
// lane `lane` (team of T lanes) as floats in v[0 .. N - 1]; columns past the end of the row read zeros.
// kInner: the caller knows that only column c0 + N - 1 can reach past the end.
struct RowF32 {
  // elements per row for d dimensions
  __host__ __device__ static int stride(int d) { return (d + 7) / 8 * 8; }
  template <int N, int T, bool kInner = false>
  static __device__ __forceinline__ void load(const unsigned char* row, int lane, int c0, int nchunk, float4* v) {
#pragma unroll
    for (int cc = 0; cc < N; ++cc) {
      const int ch = lane + T * (c0 + cc);
      v[cc] = ((kInner && cc < N - 1) || ch < nchunk) ? __ldg(reinterpret_cast<const float4*>(row) + ch)
                                                      : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
};
// two packed 16-bit values -> two floats
template <bool kBf16>
__device__ __forceinline__ float2 unpack2(unsigned w) {
  if (kBf16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));  // a bfloat16 is the upper half of a float
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <bool kBf16>
struct Row16 {
  __host__ __device__ static int team(int d) { return d <= 128 ? 8 : 32; }
  __host__ __device__ static int stride(int d) {
    const int t = team(d), nchunk = (d + 3) / 4;
    return (nchunk + 2 * t - 1) / (2 * t) * t * 8;  // pairs of columns x T slots x 8 halves
  }
  // position (in halves) of element e of a row
  __host__ __device__ static int position(int d, int e) {
    const int t = team(d), ch = e >> 2, c = ch / t, lane = ch % t;
    return ((c >> 1) * t + lane) * 8 + (c & 1) * 4 + (e & 3);
  }
  template <int N, int T, bool kInner = false>
  static __device__ __forceinline__ void load(const unsigned char* row, int lane, int c0, int nchunk, float4* v) {
    const int npair = (nchunk + 2 * T - 1) / (2 * T);
#pragma unroll
    for (int jj = 0; jj < (N + 1) / 2; ++jj) {  // c0 is even
      const int p = (c0 >> 1) + jj;
      uint4 u = make_uint4(0u, 0u, 0u, 0u);
      if (kInner || p < npair) u = __ldg(reinterpret_cast<const uint4*>(row) + p * T + lane);
      const float2 a = unpack2<kBf16>(u.x);
      const float2 b = unpack2<kBf16>(u.y);
      v[2 * jj] = make_float4(a.x, a.y, b.x, b.y);
      if (2 * jj + 1 < N) {
        const float2 c = unpack2<kBf16>(u.z);
        const float2 e = unpack2<kBf16>(u.w);
        v[2 * jj + 1] = make_float4(c.x, c.y, e.x, e.y);
      }
    }
  }
};
using RowF16 = Row16<false>;
using RowBF16 = Row16<true>;
// row storage of an index: GraphView::rows16
constexpr int kRowsF32 = 0, kRowsF16 = 1, kRowsBF16 = 2;
// CALL(Row) with the row type that `kind` names
#define HNSW_WITH_ROWS(kind, CALL) \
  ((kind) == ::hnsw::kRowsF16 ? CALL(::hnsw::RowF16) : (kind) == ::hnsw::kRowsBF16 ? CALL(::hnsw::RowBF16) : CALL(::hnsw::RowF32))

__device__ __forceinline__ void fma4(float4& acc, const float4& a, const float4& b, int dist_type) {
  if (dist_type == DIST_DOT) {
    acc.x = fmaf(a.x, b.x, acc.x);
    acc.y = fmaf(a.y, b.y, acc.y);
    acc.z = fmaf(a.z, b.z, acc.z);
    acc.w = fmaf(a.w, b.w, acc.w);
  } else {
    float dx = a.x - b.x, dy = a.y - b.y, dz = a.z - b.z, dw = a.w - b.w;
    acc.x = fmaf(dx, dx, acc.x);
    acc.y = fmaf(dy, dy, acc.y);
    acc.z = fmaf(dz, dz, acc.z);
    acc.w = fmaf(dw, dw, acc.w);
  }
}

__device__ __forceinline__ float fold4(const float4& a) { return (a.x + a.y) + (a.z + a.w); }

// ---------------------------------------------------------------------------
// d <= 128: teams of 8 lanes, four rows per warp pass, query chunks in registers.
// C = ceil(d / 32) chunks per lane.
// ---------------------------------------------------------------------------
template <int C, class Row = RowF32>
struct DistSmall {
  static constexpr int kTeam = 8;
  static constexpr int kRowsPerPass = 4;
  // Passes whose loads are issued together: one.  Measured on a B200 (1.18 M x 50, 10 000 queries, ef 200):
  // 1.50 ms per launch with one pass in flight, 1.69 ms with two, 2.04 ms with three (all at 64 registers):
  // every added instruction costs more than the shorter gather saves.
  static constexpr int kBatch = 1;
  // Resident CTAs (of 2 warps) per SM the walk kernels are compiled for.
  // search: 16 CTAs = 64 registers; 17 or 18 CTAs (56 registers, spills) gain nothing even where they save a
  // wave of warps (1.51 ms and 2.08 ms on the same launch); rows of 97..128 floats spill at 64 registers and run
  // 37 % faster with 14 CTAs = 72 registers (1 M x 128, 10 000 queries, ef 256: 3.52 ms against 5.57 ms)
  static constexpr int kSearchMinCtas = C <= 3 ? 16 : 14;
  // construction: 16 CTAs (64 registers) measured 6 % faster than 12 for rows of up to 64 floats
  // (1.18 M x 50: 0.208 s against 0.222 s) and 2.5 % faster for 96 (2 M x 96: 0.310 against 0.318 s);
  // rows of 128 floats are 15 % slower there (1 M x 128: 0.477 against 0.415 s)
  static constexpr int kBuildMinCtas = C <= 3 ? 16 : 12;
  static constexpr int kWarpsPerSmTarget = 32;
  __host__ __device__ static constexpr size_t smem_bytes(int) { return 0; }

  VecTable t;
  float4 q[C];

  __device__ __forceinline__ void init(const VecTable& tab, void*) { t = tab; }

  // query from an unpadded row of d floats in global memory
  __device__ __forceinline__ void load_query(const float* qp) {
    const int tl = lane_id() & 7;
#pragma unroll
    for (int c = 0; c < C; ++c) {
      int e = 4 * (tl + 8 * c);
      q[c].x = (e + 0 < t.d) ? __ldg(qp + e + 0) : 0.0f;
      q[c].y = (e + 1 < t.d) ? __ldg(qp + e + 1) : 0.0f;
      q[c].z = (e + 2 < t.d) ? __ldg(qp + e + 2) : 0.0f;
      q[c].w = (e + 3 < t.d) ? __ldg(qp + e + 3) : 0.0f;
    }
  }
  // query = stored (padded) row `id`
  __device__ __forceinline__ void load_query_row(int id) {
    Row::template load<C, 8>(t.vec + (size_t)id * t.row_bytes, lane_id() & 7, 0, t.nchunk, q);
  }

  // Lane r (r < n <= 32, n >= 1) holds a row id; returns the distance to it in lane r.
  __device__ __forceinline__ float eval(int id, int n) {
    return t.dist_type == DIST_DOT ? eval_t<true, kBatch>(id, n) : eval_t<false, kBatch>(id, n);
  }
  template <bool kDot, int kB>
  __device__ __forceinline__ float eval_t(int id, int n) {
    const int lane = lane_id();
    const int team = lane >> 3, tl = lane & 7;
    float result = 0.0f;
    for (int r0 = 0; r0 < n; r0 += 4 * kB) {
      float4 v[kB][C];
#pragma unroll
      for (int u = 0; u < kB; ++u) {
        // rows past n are folded onto row 0 of the list: a harmless repeated load whose result nobody selects
        const int r = r0 + 4 * u + team;
        const int rid = __shfl_sync(FULL, id, r < n ? r : 0);
        // only the last chunk column can lie past the end of the row
        Row::template load<C, 8, true>(t.vec + (size_t)rid * t.row_bytes, tl, 0, t.nchunk, v[u]);
      }
#pragma unroll
      for (int u = 0; u < kB; ++u) {
        if (u == 0 || r0 + 4 * u < n) {  // warp-uniform
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int c = 0; c < C; ++c) fma4(acc, q[c], v[u][c], kDot ? DIST_DOT : DIST_L2);
          float s = fold4(acc);
          s += __shfl_xor_sync(FULL, s, 4);
          s += __shfl_xor_sync(FULL, s, 2);
          s += __shfl_xor_sync(FULL, s, 1);
          if (kDot) s = -s;
          const float mine = __shfl_sync(FULL, s, (lane & 3) << 3);
          if ((lane >> 2) == (r0 >> 2) + u) result = mine;
        }
      }
    }
    return result;
  }
};

// ---------------------------------------------------------------------------
// d > 128: the whole warp owns one row (T = 32), query chunks in shared memory.
// ---------------------------------------------------------------------------
// kChunksT = chunk columns per row whose loads are in flight together, kRowsT = rows; kMinCtasT = resident
// CTAs per SM the search kernel is compiled for.  <4, 8> (16 float4 in flight, ~125 registers) suits large batches;
// <8, 4> (32 float4 in flight) is 23 % faster on 1000 queries of d = 960, where resident warps do not
// matter because there are fewer queries than warp slots.
template <int kChunksT, int kMinCtasT, class Row = RowF32, int kRowsT = 4>
struct DistLargeT {
  static constexpr int kRows = kRowsT;        // rows whose loads are in flight together
  static constexpr int kChunks = kChunksT;    // chunk columns per row per step
  static constexpr int kSearchMinCtas = kMinCtasT;
  static constexpr int kBuildMinCtas = 8;
  static constexpr int kWarpsPerSmTarget = 16;
  __host__ __device__ static constexpr size_t smem_bytes(int d) { return (size_t)((d + 127) / 128) * 128 * sizeof(float); }

  VecTable t;
  float4* sq;  // per-warp, (C * 32) float4, zero padded
  int C;

  __device__ __forceinline__ void init(const VecTable& tab, void* smem) {
    t = tab;
    sq = reinterpret_cast<float4*>(smem);
    C = (tab.d + 127) / 128;
  }
  __device__ __forceinline__ void load_query(const float* qp) {
    float* s = reinterpret_cast<float*>(sq);
    for (int e = lane_id(); e < C * 128; e += 32) s[e] = (e < t.d) ? __ldg(qp + e) : 0.0f;
    __syncwarp();
  }
  __device__ __forceinline__ void load_query_row(int id) {
    const unsigned char* row = t.vec + (size_t)id * t.row_bytes;
    for (int c0 = 0; c0 < C; c0 += 2) {
      float4 v[2];
      Row::template load<2, 32>(row, lane_id(), c0, t.nchunk, v);
      sq[lane_id() + 32 * c0] = v[0];
      if (c0 + 1 < C) sq[lane_id() + 32 * (c0 + 1)] = v[1];
    }
    __syncwarp();
  }
  __device__ __forceinline__ float eval(int id, int n) {
    const int lane = lane_id();
    float result = 0.0f;
    for (int r0 = 0; r0 < n; r0 += kRows) {
      float4 acc[kRows];
      int rid[kRows];
#pragma unroll
      for (int u = 0; u < kRows; ++u) {
        acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        rid[u] = __shfl_sync(FULL, id, (r0 + u) & 31);
        if (r0 + u >= n) rid[u] = -1;
      }
      for (int c0 = 0; c0 < C; c0 += kChunks) {
        float4 v[kRows][kChunks];
#pragma unroll
        for (int u = 0; u < kRows; ++u) {
          // rows past n are folded onto row 0: a harmless repeated load whose result nobody selects
          Row::template load<kChunks, 32>(t.vec + (size_t)(rid[u] >= 0 ? rid[u] : 0) * t.row_bytes, lane, c0, t.nchunk,
                                          v[u]);
        }
#pragma unroll
        for (int cc = 0; cc < kChunks; ++cc) {
          if (c0 + cc < C) {
            float4 qq = sq[lane + 32 * (c0 + cc)];
#pragma unroll
            for (int u = 0; u < kRows; ++u) fma4(acc[u], qq, v[u][cc], t.dist_type);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kRows; ++u) {
        float s = fold4(acc[u]);
        s += __shfl_xor_sync(FULL, s, 16);
        s += __shfl_xor_sync(FULL, s, 8);
        s += __shfl_xor_sync(FULL, s, 4);
        s += __shfl_xor_sync(FULL, s, 2);
        s += __shfl_xor_sync(FULL, s, 1);
        if (t.dist_type == DIST_DOT) s = -s;
        if (lane == r0 + u) result = s;
      }
    }
    return result;
  }
};

using DistLarge = DistLargeT<4, 8>;      // default: build kernels, large query batches
using DistLargeDeep = DistLargeT<8, 4>;  // few queries: more loads in flight per warp

// Engines by row width (floats) and storage type: Pick<Row>::D32 ... ::Wide, ::WideDeep
template <class Row>
struct Pick {
  using D32 = DistSmall<1, Row>;
  using D64 = DistSmall<2, Row>;
  using D96 = DistSmall<3, Row>;
  using D128 = DistSmall<4, Row>;
  using Wide = DistLargeT<4, 8, Row>;
  using WideDeep = DistLargeT<8, 4, Row>;
  // a warp of a four-warp CTA per query sees one or two rows of most requests: two rows, eight columns of
  // each in flight (a 3840-byte row in one round trip) measured 8 % faster there than four rows of four
  using Team = DistLargeT<8, 8, Row, 2>;
};

}  // namespace hnsw
