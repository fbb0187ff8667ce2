// Per-device cache of uploaded index maps, error bookkeeping.
#include <cstdlib>
#include <map>
#include <mutex>
#include <atomic>
#include <stdexcept>
#include <utility>
#include <vector>

#include "../../include/mellin_b200.h"
#include "mellin_internal.h"

namespace mellin {

namespace {
thread_local std::string g_last_error;
std::atomic<int64_t> g_launches{0};
std::atomic<int> g_tensor_cores{1};

struct CachedTable {
  void *block = nullptr;
  DeviceTable view;
};
std::mutex g_mutex;
std::map<std::pair<int, IndexMapKey>, CachedTable> g_tables;
std::map<int, int> g_sm_count;
struct Arena {
  void *ptr = nullptr;
  size_t bytes = 0;
};
std::map<std::pair<int, cudaStream_t>, Arena> g_arenas;
}  // namespace

// Scratch owned by the library for the operator-level entry points, whose
// reference signatures have no workspace argument: one arena per (device,
// stream), grown on demand (growing synchronises the stream and reallocates --
// a set-up cost of the first call of a larger geometry) and kept until
// mellin_clear_tables().  Returns nullptr when the allocation fails.
void *scratch_arena(size_t bytes, cudaStream_t stream) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  Arena &a = g_arenas[std::make_pair(dev, stream)];
  if (a.bytes >= bytes) return a.ptr;
  if (a.ptr != nullptr) {
    if (cudaStreamSynchronize(stream) != cudaSuccess) return nullptr;  // earlier calls may still be using it
    cudaFree(a.ptr);
    a.ptr = nullptr, a.bytes = 0;
  }
  const size_t want = bytes + bytes / 8;  // a little head-room: geometries of one model differ slightly
  if (cudaMalloc(&a.ptr, want) != cudaSuccess) {
    cudaGetLastError();
    a.ptr = nullptr;
    return nullptr;
  }
  a.bytes = want;
  return a.ptr;
}

void set_error(const std::string &msg) { g_last_error = msg; }
int fail(int code, const std::string &msg) {
  g_last_error = msg;
  return code;
}
const std::string &last_error() { return g_last_error; }
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }

namespace {
std::atomic<int> g_dependent_launch{-1};  // -1: not decided yet (the environment is read on first use)
}
bool dependent_launch_enabled() {
  int v = g_dependent_launch.load(std::memory_order_relaxed);
  if (v < 0) {
    const char *env = getenv("MELLIN_DEPENDENT_LAUNCH");
    v = (env != nullptr && env[0] == '0') ? 0 : 1;
    g_dependent_launch.store(v, std::memory_order_relaxed);
  }
  return v != 0;
}
int set_dependent_launch(int enable) {
  const int before = dependent_launch_enabled() ? 1 : 0;
  g_dependent_launch.store(enable ? 1 : 0, std::memory_order_relaxed);
  return before;
}

bool tensor_cores_enabled() { return g_tensor_cores.load(std::memory_order_relaxed) != 0; }
int set_tensor_cores(int enable) { return g_tensor_cores.exchange(enable ? 1 : 0); }

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  std::lock_guard<std::mutex> lock(g_mutex);
  auto it = g_sm_count.find(dev);
  if (it != g_sm_count.end()) return it->second;
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  g_sm_count[dev] = n;
  return n;
}

int get_device_table(const IndexMapKey &key, DeviceTable *out) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("cudaGetDevice: ") + cudaGetErrorString(err));
  std::lock_guard<std::mutex> lock(g_mutex);
  auto it = g_tables.find(std::make_pair(dev, key));
  if (it != g_tables.end()) {
    *out = it->second.view;
    return MELLIN_OK;
  }
  IndexMap m;
  try {
    m = build_index_map(key);
  } catch (const std::invalid_argument &e) {
    return fail(MELLIN_ERR_BAD_ARGUMENT, e.what());
  }
  // one block: row_ptr | order | entries (entries 8-byte aligned)
  const size_t n_ptr = m.row_ptr.size(), n_ord = m.order.size(), n_ent = m.entries.size();
  size_t ints = n_ptr + n_ord;
  ints += ints & 1;
  const size_t bytes = ints * sizeof(int32_t) + n_ent * sizeof(Entry);
  std::vector<int32_t> host(ints + 2 * n_ent, 0);
  std::copy(m.row_ptr.begin(), m.row_ptr.end(), host.begin());
  std::copy(m.order.begin(), m.order.end(), host.begin() + n_ptr);
  for (size_t i = 0; i < n_ent; ++i) {
    host[ints + 2 * i] = m.entries[i].a;
    host[ints + 2 * i + 1] = m.entries[i].b;
  }
  CachedTable c;
  err = cudaMalloc(&c.block, bytes > 0 ? bytes : 16);
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("cudaMalloc(index table): ") + cudaGetErrorString(err));
  err = cudaMemcpy(c.block, host.data(), bytes, cudaMemcpyHostToDevice);
  // A copy from pageable memory returns once the bytes are staged; the transfer
  // itself is ordered on the legacy default stream only.  The caller's kernels
  // may run on a stream that does not synchronise with it, so wait here.
  if (err == cudaSuccess) err = cudaStreamSynchronize(cudaStreamLegacy);
  if (err != cudaSuccess) {
    cudaFree(c.block);
    return fail(MELLIN_ERR_LAUNCH, std::string("cudaMemcpy(index table): ") + cudaGetErrorString(err));
  }
  const int32_t *base = static_cast<const int32_t *>(c.block);
  c.view.row_ptr = base;
  c.view.order = base + n_ptr;
  c.view.entries = reinterpret_cast<const int2 *>(base + ints);
  c.view.rows = m.rows;
  c.view.max_row = m.max_row;
  c.view.triples = m.triples;
  c.view.num_entries = static_cast<int64_t>(n_ent);
  g_tables.emplace(std::make_pair(dev, key), c);
  *out = c.view;
  return MELLIN_OK;
}

int clear_device_tables() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return MELLIN_ERR_LAUNCH;
  cudaDeviceSynchronize();  // nothing in flight may still read what is freed below
  std::lock_guard<std::mutex> lock(g_mutex);
  for (auto it = g_arenas.begin(); it != g_arenas.end();) {
    if (it->first.first == dev) {
      cudaFree(it->second.ptr);
      it = g_arenas.erase(it);
    } else {
      ++it;
    }
  }
  for (auto it = g_tables.begin(); it != g_tables.end();) {
    if (it->first.first == dev) {
      cudaFree(it->second.block);
      it = g_tables.erase(it);
    } else {
      ++it;
    }
  }
  return MELLIN_OK;
}

}  // namespace mellin
