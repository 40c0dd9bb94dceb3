// Host layer of the engine: options, device-resident index, level orchestration,
// hnswlib-format file I/O.  Mirrors the public methods of the reference's host
// class (cpp/include/cuhnsw.hpp:50-113) but keeps the whole index in flat device
// arrays instead of per-level host adjacency lists (cpp/include/level_graph.hpp).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <string>
#include <vector>

#include "kernels.h"

namespace hnsw {

enum Status {
  kOk = 0,
  kInvalidArgument = -1,
  kIoError = -2,
  kParseError = -3,
  kInvalidOption = -4,
  kCudaError = -5,
  kBadState = -6,
  kUnsupported = -7,
};

// Field names and defaults follow cuhnsw/proto/config.proto:9-27.
struct Options {
  int seed = 777;
  int c_log_level = 2;
  int max_m = 12;
  int max_m0 = 24;
  int ef_construction = 150;
  double level_mult = 0.0;
  bool save_remains = false;
  double hyper_threads = 10.0;
  int block_dim = 32;
  std::string dist_type = "dot";
  int visited_table_size = 0;
  int visited_list_size = 8192;
  bool nrz = false;
  bool reverse_cand = false;
  int search_team = -1;  // d > 128: 1 = CTA per query, 0 = warp per query, -1 = chosen by batch size
  std::string row_dtype = "f32";  // "f16" / "bf16": rows stored in 16 bits, distances in fp32 over the stored values
  bool search_schedule = true;  // batches of more than one wave: serve the queries with the farthest entry first
  bool zero_copy = true;        // host-buffer searches on page-locked buffers: the kernels read and write them in place
  double heuristic_coef = 0.25;
  // extensions (absent from the reference's schema; optional keys of the option file)
  long long batch_max = 0;  // nodes per insertion batch; 0 = hyper_threads * (SMs * 128 / block_dim)
  // A batch never exceeds (nodes already linked on the level) / ramp_div.  Every batch, however small, costs
  // the latency of one insertion (~0.4 ms: a 110-step walk, selection, one reverse update), and with 16 the
  // ~190 ramp-up batches of the five levels were 40 % of a 1.18 M-row build: 0.192 s with 16, 0.154 s with 4,
  // 0.147 s with 2, 0.144 s with 1; recall@10 and the work per search do not move beyond their scatter from one
  // schedule to the next (0.955-0.961 at ef 300; 100 000 x 50: 0.990 / 0.993 / 0.987 / 0.995 with 16 / 4 / 2 / 1).
  long long ramp_div = 4;
  int device_id = -1;       // -1 = current device
  // GPUs that each hold a replica of the index; a host-buffer search is split over them.  Empty: one GPU.
  std::vector<int> devices;
};

template <class T>
class DevBuf {
 public:
  DevBuf() = default;
  DevBuf(const DevBuf&) = delete;
  DevBuf& operator=(const DevBuf&) = delete;
  ~DevBuf() { release(); }
  void release() {
    if (p_) cudaFree(p_);
    p_ = nullptr;
    n_ = 0;
  }
  cudaError_t alloc(size_t n) {
    release();
    if (n == 0) return cudaSuccess;
    cudaError_t e = cudaMalloc(&p_, n * sizeof(T));
    if (e == cudaSuccess) n_ = n;
    else p_ = nullptr;
    return e;
  }
  cudaError_t reserve(size_t n) { return n <= n_ ? cudaSuccess : alloc(n); }
  T* get() const { return p_; }
  size_t size() const { return n_; }

 private:
  T* p_ = nullptr;
  size_t n_ = 0;
};

class Engine {
 public:
  Engine();
  ~Engine();

  // device_override >= 0: use that GPU whatever the option file says (replicas of a multi-GPU handle)
  int Init(const char* opt_path, int device_override = -1);
  // makes this engine a copy of src's index on its own GPU (device-to-device)
  int CloneFrom(const Engine& src);
  bool has_graph() const { return has_graph_; }
  long long num_data() const { return n_; }
  int num_dims() const { return d_; }
  int SetData(const float* data, long long num_data, int num_dims);
  int SetRandomLevels(const int* levels);
  int BuildGraph();
  int SaveIndex(const char* path);
  int LoadIndex(const char* path);
  // host buffers in, host buffers out; blocks until the results are in place
  int SearchGraph(const float* qdata, long long num_queries, int topk, int ef_search, int* nns, float* distances,
                  int* found_cnt);
  // host buffers in/out, copies and kernels enqueued on the engine's stream, returns without waiting: the
  // results are in place once the stream has reached this point
  int SearchGraphAsync(const float* qdata, long long num_queries, int topk, int ef_search, int* nns, float* distances,
                       int* found_cnt);
  // device buffers in/out; enqueued on the engine's stream, returns without waiting
  int SearchGraphDevice(const float* d_qdata, long long num_queries, int topk, int ef_search, int* d_nns,
                        float* d_distances, int* d_found_cnt);
  // host buffers in/out like SearchGraph, but no allocation: staging lives in a fixed device array
  int SearchGraphStatic(const float* qdata, long long num_queries, int topk, int ef_search, int* nns,
                        float* distances, int* found_cnt);
  // distances between stored rows (host index arrays, host output)
  int BatchDistance(const int* src, const int* dst, long long npairs, float* out);
  int SetStream(void* stream);
  void* stream() const { return stream_; }
  int Synchronize();
  // a stream on this engine's GPU / page-locked host memory, for hosts that have no CUDA binding of their own
  int CreateStream(void** out);
  int SyncStream(void* stream);
  int DestroyStream(void* stream);
  void* HostAlloc(size_t bytes);
  void HostFree(void* ptr);
  int EnableStats(int on);
  int GetStats(unsigned long long* out4);
  int GetGraph(int* levels, int* rows0, int* rows_upper);  // host copies, for tests
  int Describe(long long* out8);
  double last_build_seconds() const { return last_build_seconds_; }
  const char* last_error() const { return err_.c_str(); }
  const Options& options() const { return opt_; }

 private:
  int Fail(int code, const std::string& msg);
  int FailCuda(cudaError_t e, const char* what);
  int EnsureDevice();
  int AllocRows(long long num_data, int num_dims);
  int AllocGraph();
  int ResolveVsize(int requested_cap, long long nq, int* vsize) const;  // nq < 0: construction
  GraphView View() const;
  void Log(int level, const char* fmt, ...) const;

  Options opt_;
  bool inited_ = false;
  std::string err_;
  int device_ = -1;
  int sm_count_ = 0;
  size_t smem_optin_ = 0;
  cudaStream_t stream_ = nullptr;  // legacy default stream unless SetStream is called

  long long n_ = 0;
  int d_ = 0;
  int vstride_ = 0;
  int rows16_ = 0;  // 0 fp32 rows, 1 IEEE half, 2 bfloat16
  void* RowPtr(long long row) const {
    return reinterpret_cast<unsigned char*>(vec_.get()) + (size_t)row * vstride_ * (rows16_ ? 2 : 4);
  }
  int dist_type_ = 0;
  int stride0_ = 0, strideU_ = 0;
  int max_level_ = 0, enter_point_ = 0;
  long long total_upper_ = 0;
  bool has_data_ = false, has_levels_ = false, has_graph_ = false, labelled_ = false;
  std::vector<int> levels_h_;
  std::vector<int> upper_base_h_;
  std::vector<long long> labels_h_;

  DevBuf<float> vec_;
  DevBuf<int> rows0_, rowsU_, levels_d_, upper_base_d_, labels_d_;
  DevBuf<unsigned long long> counters_;  // [0] search ticket, [1..2] build tickets, [4..7] stats
  bool stats_on_ = false;
  // Scratch of one search in flight: its ticket counter and the grow-only arrays of the
  // longest-first schedule (six words per query + sort storage).  A search uses the set that belongs to the
  // stream it is enqueued on, so searches enqueued on different streams can run at the same time: the tail of
  // one batch (a launch lasts as long as its longest walk) overlaps with the next batch.  A stream beyond
  // kSearchLanes takes over the least recently used set after waiting for the search that used it last (through
  // the set's own event, which outlives a stream the caller has destroyed since).
  struct SearchLane {
    cudaStream_t stream = nullptr;
    bool used = false;
    unsigned long long stamp = 0;
    cudaEvent_t done = nullptr;  // recorded behind the last thing a search put on the stream
    bool pending = false;
    DevBuf<unsigned long long> ticket;
    DevBuf<unsigned> sched;
    DevBuf<unsigned char> sched_tmp;
    long long capacity = 0;
    // grow-only device copies of the host-buffer searches' queries and results
    DevBuf<float> q, dist;
    DevBuf<int> ids, found;
  };
  static constexpr int kSearchLanes = 8;
  SearchLane lanes_[kSearchLanes];
  unsigned long long lane_clock_ = 0;
  int LaneFor(cudaStream_t stream, SearchLane** lane);
  int MarkLane(SearchLane* lane);  // records `done` on the engine's stream
  int WaitForSearches();           // every search enqueued so far, on whatever stream, is over
  int PrepareSchedule(long long nq, SearchLane* lane, SearchSchedule* s);
  double last_build_seconds_ = 0.0;
};

}  // namespace hnsw
