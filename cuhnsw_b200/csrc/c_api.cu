// extern "C" surface of the engine; see include/cuhnsw_b200.h for the contract.
#include <exception>
#include <new>

#include "../../include/cuhnsw_b200.h"
#include "engine.h"
#include "replicas.h"

struct cuhnsw_handle {
  hnsw::Engine engine;         // the index on the first (or only) GPU
  hnsw::ReplicaSet replicas;   // copies on the other GPUs of the option `devices`
  std::string fatal;
};

namespace {
template <class F>
int guarded(cuhnsw_handle* h, F f) {
  if (!h) return CUHNSW_INVALID_ARGUMENT;
  h->fatal.clear();  // the text of an earlier exception must not outlive the call that raised it
  try {
    return f(h->engine);
  } catch (const std::bad_alloc&) {
    h->fatal = "out of host memory";
    return CUHNSW_OUT_OF_MEMORY;
  } catch (const std::exception& e) {
    h->fatal = e.what();
  } catch (...) {
    h->fatal = "unknown failure";
  }
  return CUHNSW_INTERNAL_ERROR;
}
int null_argument(cuhnsw_handle* h, const char* what) {
  if (h) h->fatal = std::string("null pointer: ") + what;
  return CUHNSW_INVALID_ARGUMENT;
}
}  // namespace

extern "C" {

cuhnsw_handle* cuhnsw_create(void) {
  try {
    return new cuhnsw_handle();
  } catch (...) {
    return nullptr;
  }
}
void cuhnsw_destroy(cuhnsw_handle* h) { delete h; }
const char* cuhnsw_last_error(const cuhnsw_handle* h) {
  if (!h) return "null handle";
  return h->fatal.empty() ? h->engine.last_error() : h->fatal.c_str();
}
int cuhnsw_init(cuhnsw_handle* h, const char* opt_path) {
  return guarded(h, [&](hnsw::Engine& e) {
    int rc = e.Init(opt_path);
    if (rc == hnsw::kOk) rc = h->replicas.Configure(e, opt_path, &h->fatal);
    return rc;
  });
}
int cuhnsw_set_data(cuhnsw_handle* h, const float* data, int64_t num_data, int32_t num_dims) {
  return guarded(h, [&](hnsw::Engine& e) {
    h->replicas.Invalidate();
    return e.SetData(data, num_data, num_dims);
  });
}
int cuhnsw_set_random_levels(cuhnsw_handle* h, const int32_t* levels) {
  return guarded(h, [&](hnsw::Engine& e) {
    h->replicas.Invalidate();
    return e.SetRandomLevels(levels);
  });
}
int cuhnsw_build_graph(cuhnsw_handle* h) {
  return guarded(h, [&](hnsw::Engine& e) {
    h->replicas.Invalidate();
    int rc = e.BuildGraph();
    if (rc == hnsw::kOk && h->replicas.active()) rc = h->replicas.Sync(e, &h->fatal);
    return rc;
  });
}
int cuhnsw_save_index(cuhnsw_handle* h, const char* fpath) {
  return guarded(h, [&](hnsw::Engine& e) { return e.SaveIndex(fpath); });
}
int cuhnsw_load_index(cuhnsw_handle* h, const char* fpath) {
  return guarded(h, [&](hnsw::Engine& e) {
    h->replicas.Invalidate();
    int rc = e.LoadIndex(fpath);
    if (rc == hnsw::kOk && h->replicas.active()) rc = h->replicas.Sync(e, &h->fatal);
    return rc;
  });
}
int cuhnsw_search_knn(cuhnsw_handle* h, const float* qdata, int64_t num_queries, int32_t topk, int32_t ef_search,
                      int32_t* nns, float* distances, int32_t* found_cnt) {
  return guarded(h, [&](hnsw::Engine& e) {
    if (h->replicas.active() && e.has_graph() && num_queries > 0 && qdata && nns && distances && found_cnt)
      return h->replicas.Search(e, qdata, num_queries, topk, ef_search, nns, distances, found_cnt, &h->fatal);
    return e.SearchGraph(qdata, num_queries, topk, ef_search, nns, distances, found_cnt);
  });
}
int cuhnsw_search_knn_device(cuhnsw_handle* h, const float* d_qdata, int64_t num_queries, int32_t topk,
                             int32_t ef_search, int32_t* d_nns, float* d_distances, int32_t* d_found_cnt) {
  return guarded(h, [&](hnsw::Engine& e) {
    return e.SearchGraphDevice(d_qdata, num_queries, topk, ef_search, d_nns, d_distances, d_found_cnt);
  });
}
int cuhnsw_search_knn_async(cuhnsw_handle* h, const float* qdata, int64_t num_queries, int32_t topk, int32_t ef_search,
                            int32_t* nns, float* distances, int32_t* found_cnt) {
  return guarded(h, [&](hnsw::Engine& e) {
    return e.SearchGraphAsync(qdata, num_queries, topk, ef_search, nns, distances, found_cnt);
  });
}
namespace {
// A call on another replica makes that replica's GPU the thread's current device; the caller (who may be in the
// middle of its own CUDA work) gets its device back.
struct DeviceRestore {
  int before = -1;
  DeviceRestore() {
    if (cudaGetDevice(&before) != cudaSuccess) {
      cudaGetLastError();
      before = -1;
    }
  }
  ~DeviceRestore() {
    if (before >= 0) cudaSetDevice(before);
  }
};
}  // namespace
int cuhnsw_replica_count(const cuhnsw_handle* h) { return h ? h->replicas.count() : 0; }
int cuhnsw_stream_create_on(cuhnsw_handle* h, int32_t replica, void** out_stream) {
  return guarded(h, [&](hnsw::Engine& e) {
    int rc = hnsw::kOk;
    hnsw::Engine* r = h->replicas.Fresh(e, replica, &rc, &h->fatal);
    if (!r) return rc;
    DeviceRestore restore;
    rc = r->CreateStream(out_stream);
    if (rc != hnsw::kOk && r != &e) h->fatal = r->last_error();
    return rc;
  });
}
int cuhnsw_search_knn_async_on(cuhnsw_handle* h, int32_t replica, void* cuda_stream, const float* qdata,
                               int64_t num_queries, int32_t topk, int32_t ef_search, int32_t* nns, float* distances,
                               int32_t* found_cnt) {
  return guarded(h, [&](hnsw::Engine& e) {
    int rc = hnsw::kOk;
    hnsw::Engine* r = h->replicas.Fresh(e, replica, &rc, &h->fatal);
    if (!r) return rc;
    DeviceRestore restore;
    void* before = r->stream();
    r->SetStream(cuda_stream);
    rc = r->SearchGraphAsync(qdata, num_queries, topk, ef_search, nns, distances, found_cnt);
    r->SetStream(before);
    if (rc != hnsw::kOk && r != &e) h->fatal = r->last_error();
    return rc;
  });
}
int cuhnsw_search_knn_noalloc(cuhnsw_handle* h, const float* qdata, int64_t num_queries, int32_t topk,
                              int32_t ef_search, int32_t* nns, float* distances, int32_t* found_cnt) {
  return guarded(h, [&](hnsw::Engine& e) {
    return e.SearchGraphStatic(qdata, num_queries, topk, ef_search, nns, distances, found_cnt);
  });
}
int cuhnsw_batch_distance(cuhnsw_handle* h, const int32_t* src, const int32_t* dst, int64_t num_pairs, float* out) {
  return guarded(h, [&](hnsw::Engine& e) { return e.BatchDistance(src, dst, num_pairs, out); });
}
int cuhnsw_set_stream(cuhnsw_handle* h, void* cuda_stream) {
  return guarded(h, [&](hnsw::Engine& e) { return e.SetStream(cuda_stream); });
}
int cuhnsw_synchronize(cuhnsw_handle* h) {
  return guarded(h, [&](hnsw::Engine& e) { return e.Synchronize(); });
}
int cuhnsw_stream_create(cuhnsw_handle* h, void** out_stream) {
  return guarded(h, [&](hnsw::Engine& e) { return e.CreateStream(out_stream); });
}
int cuhnsw_stream_synchronize(cuhnsw_handle* h, void* cuda_stream) {
  return guarded(h, [&](hnsw::Engine& e) { return e.SyncStream(cuda_stream); });
}
int cuhnsw_stream_destroy(cuhnsw_handle* h, void* cuda_stream) {
  return guarded(h, [&](hnsw::Engine& e) { return e.DestroyStream(cuda_stream); });
}
void* cuhnsw_host_alloc(cuhnsw_handle* h, size_t bytes) {
  void* p = nullptr;
  guarded(h, [&](hnsw::Engine& e) {
    p = e.HostAlloc(bytes);
    return hnsw::kOk;
  });
  return p;
}
void cuhnsw_host_free(cuhnsw_handle* h, void* ptr) {
  guarded(h, [&](hnsw::Engine& e) {
    e.HostFree(ptr);
    return hnsw::kOk;
  });
}
int cuhnsw_enable_stats(cuhnsw_handle* h, int32_t on) {
  return guarded(h, [&](hnsw::Engine& e) { return e.EnableStats(on); });
}
int cuhnsw_get_stats(cuhnsw_handle* h, uint64_t* out4) {
  if (!out4) return null_argument(h, "out4");
  return guarded(h, [&](hnsw::Engine& e) { return e.GetStats(reinterpret_cast<unsigned long long*>(out4)); });
}
int cuhnsw_describe(cuhnsw_handle* h, int64_t* out8) {
  if (!out8) return null_argument(h, "out8");
  return guarded(h, [&](hnsw::Engine& e) { return e.Describe(reinterpret_cast<long long*>(out8)); });
}
int cuhnsw_get_graph(cuhnsw_handle* h, int32_t* levels, int32_t* rows0, int32_t* rows_upper) {
  return guarded(h, [&](hnsw::Engine& e) { return e.GetGraph(levels, rows0, rows_upper); });
}
double cuhnsw_last_build_seconds(const cuhnsw_handle* h) { return h ? h->engine.last_build_seconds() : 0.0; }

int cuhnsw_merge_topk_device(const int32_t* d_ids, const float* d_distances, int32_t parts, int64_t num_queries,
                             int32_t topk, int32_t* d_out_ids, float* d_out_distances, int32_t* d_out_found,
                             void* cuda_stream) {
  if (parts < 1 || topk < 1 || num_queries < 0) return CUHNSW_INVALID_ARGUMENT;
  if (num_queries > 0 && (!d_ids || !d_distances || !d_out_ids || !d_out_distances)) return CUHNSW_INVALID_ARGUMENT;
  cudaError_t e = hnsw::launch_merge_topk(d_ids, d_distances, (long long)num_queries * topk, nullptr, parts,
                                          num_queries, topk, d_out_ids, d_out_distances, d_out_found,
                                          reinterpret_cast<cudaStream_t>(cuda_stream));
  return e == cudaSuccess ? CUHNSW_OK : CUHNSW_CUDA_ERROR;
}

int cuhnsw_merge_topk_gathered_device(const int32_t* d_gathered, const int32_t* d_id_offsets, int32_t parts,
                                      int64_t num_queries, int32_t topk, int32_t* d_out_ids, float* d_out_distances,
                                      int32_t* d_out_found, void* cuda_stream) {
  if (parts < 1 || topk < 1 || num_queries < 0) return CUHNSW_INVALID_ARGUMENT;
  if (num_queries > 0 && (!d_gathered || !d_out_ids || !d_out_distances)) return CUHNSW_INVALID_ARGUMENT;
  const long long block = (long long)num_queries * topk;
  cudaError_t e = hnsw::launch_merge_topk(d_gathered, reinterpret_cast<const float*>(d_gathered + block), 2 * block,
                                          d_id_offsets, parts, num_queries, topk, d_out_ids, d_out_distances,
                                          d_out_found, reinterpret_cast<cudaStream_t>(cuda_stream));
  return e == cudaSuccess ? CUHNSW_OK : CUHNSW_CUDA_ERROR;
}

int cuhnsw_selftest_list_merge(int32_t capacity, const float* distances, const int32_t* ids,
                               const int32_t* batch_begin, int32_t num_batches, const int32_t* expand_before,
                               uint64_t* out_keys, int32_t* out_size, int32_t* out_first_position,
                               int32_t* out_cursor) {
  if (capacity < 1 || capacity > 8192 || num_batches < 0 || !batch_begin || !expand_before || !out_keys || !out_size ||
      !out_first_position || !out_cursor)
    return CUHNSW_INVALID_ARGUMENT;
  for (int b = 0; b < num_batches; ++b)
    if (batch_begin[b + 1] < batch_begin[b] || batch_begin[b + 1] - batch_begin[b] > 32) return CUHNSW_INVALID_ARGUMENT;
  if (batch_begin[num_batches] > 0 && (!distances || !ids)) return CUHNSW_INVALID_ARGUMENT;
  cudaError_t e = hnsw::selftest_list_host(capacity, distances, ids, batch_begin, num_batches, expand_before,
                                           reinterpret_cast<unsigned long long*>(out_keys), out_size,
                                           out_first_position, out_cursor);
  return e == cudaSuccess ? CUHNSW_OK : CUHNSW_CUDA_ERROR;
}

int cuhnsw_selftest_visited(int32_t entries, int64_t num_nodes, const int32_t* ids, int32_t count, int32_t* out_seen) {
  if (entries < 64 || entries > 32768 || (entries & (entries - 1)) || num_nodes < 1 || count < 0 ||
      (count > 0 && (!ids || !out_seen)))
    return CUHNSW_INVALID_ARGUMENT;
  for (int i = 0; i < count; ++i)
    if (ids[i] < 0 || ids[i] >= num_nodes) return CUHNSW_INVALID_ARGUMENT;
  cudaError_t e = hnsw::selftest_visited_host(entries, num_nodes, ids, count, out_seen);
  return e == cudaSuccess ? CUHNSW_OK : CUHNSW_CUDA_ERROR;
}

}  // extern "C"
