// C entry points over the reference's own host class (cpp/include/cuhnsw.hpp:50-113), so that
// the unmodified reference kernels can be driven from ctypes to produce golden vectors.
// TEST INFRASTRUCTURE ONLY; compiled by oracle/build_ref.sh together with the reference's
// sources where they lie; nothing of the reference is copied into this repository.
#include <exception>
#include <string>

#include "cuhnsw.hpp"

static std::string g_err;

extern "C" {
void* ref_create() {
  try { return new cuhnsw::CuHNSW(); } catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}
void ref_destroy(void* h) { delete static_cast<cuhnsw::CuHNSW*>(h); }
const char* ref_error() { return g_err.c_str(); }
#define GUARD(stmt) try { stmt; return 0; } catch (const std::exception& e) { g_err = e.what(); return -1; }
int ref_init(void* h, const char* path) {
  try { return static_cast<cuhnsw::CuHNSW*>(h)->Init(path) ? 0 : -2; } catch (const std::exception& e) { g_err = e.what(); return -1; }
}
int ref_set_data(void* h, const float* data, int n, int d) { GUARD(static_cast<cuhnsw::CuHNSW*>(h)->SetData(data, n, d)) }
int ref_set_random_levels(void* h, const int* levels) { GUARD(static_cast<cuhnsw::CuHNSW*>(h)->SetRandomLevels(levels)) }
int ref_build_graph(void* h) { GUARD(static_cast<cuhnsw::CuHNSW*>(h)->BuildGraph()) }
int ref_save_index(void* h, const char* path) { GUARD(static_cast<cuhnsw::CuHNSW*>(h)->SaveIndex(path)) }
int ref_load_index(void* h, const char* path) { GUARD(static_cast<cuhnsw::CuHNSW*>(h)->LoadIndex(path)) }
int ref_search(void* h, const float* q, int nq, int topk, int ef, int* nns, float* dist, int* found) {
  GUARD(static_cast<cuhnsw::CuHNSW*>(h)->SearchGraph(q, nq, topk, ef, nns, dist, found))
}
}
