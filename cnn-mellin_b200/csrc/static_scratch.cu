// Weight-gradient entry point for callers that must not allocate device memory.
//
// Some hosts cannot call cudaMalloc at the point where they need this gradient:
// an inference- or training-runtime plugin whose execute hook is handed a fixed
// arena and is forbidden to grow it, a real-time loop whose memory is pinned
// down at start-up so that no step can fail or stall on an allocation
// (cudaMalloc and cudaFree synchronise the device), a framework that forbids
// allocation inside its backward pass.  The regular entry point needs two kinds
// of device memory besides its operands -- caller-provided scratch for the
// per-block partial sums, and index tables that this library allocates and
// caches on first use.  The variant below needs neither: both live in ONE
// fixed array that is part of the library image, so every GPU that loads the
// library holds those bytes until the process exits.
//
// Limits and rules
//   * the partial sums of the geometry must fit kScratchBytes (8 MiB) and its
//     index tables kTableBytes (256 KiB); otherwise the call is rejected with
//     MELLIN_ERR_WORKSPACE and a message naming both numbers;
//   * the first call on each device resolves the array's device address
//     (cudaGetSymbolAddress) and synchronises the device once; make that call
//     before any stream capture;
//   * the index tables are copied into the array on the caller's stream whenever
//     the Mellin-axis geometry differs from the one the previous call on this
//     device staged (a small host-to-device copy from memory the library keeps
//     alive); calls that repeat the geometry enqueue kernels only;
//   * every call shares the array and finds in it whatever the previous call
//     left there.  Nothing needs clearing -- each kernel writes every partial sum
//     it later reads -- but two calls that overlap on the GPU (different streams,
//     or different host threads) race on it.  Serialise them.
//   * no cudaMalloc / cudaFree / allocating library routine is called; the host
//     side uses ordinary heap memory while it builds the index tables.
#include <cstdint>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/mellin_b200.h"
#include "mellin_internal.h"

namespace {

constexpr size_t kScratchBytes = 8u << 20;   // partial sums
constexpr size_t kTableBytes = 256u << 10;   // the two index tables of the geometry
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes + kTableBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
unsigned char *g_device_ptr[kMaxDevices] = {nullptr};

// What the table region of each device's array holds: the geometry last staged,
// the views handed to the kernels, and the host copy the transfer reads from
// (kept until the next geometry replaces it).
struct StagedTables {
  bool valid = false;
  int64_t key[7] = {0, 0, 0, 0, 0, 0, 0};
  mellin::DeviceTable by_f, by_h;
  std::vector<int32_t> host_f, host_h;
};
StagedTables g_staged[kMaxDevices];

// The array's name is a host-side stand-in, not a device address: resolve it
// once per device, with that device current, and hand the result to kernels.
int resolve_scratch(unsigned char **out, int *device) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return mellin::fail(MELLIN_ERR_LAUNCH, std::string("cudaGetDevice: ") + cudaGetErrorString(err));
  if (dev < 0 || dev >= kMaxDevices) return mellin::fail(MELLIN_ERR_UNSUPPORTED, "device ordinal above 63");
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_device_ptr[dev] == nullptr) {
    void *ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess || ptr == nullptr)
      return mellin::fail(MELLIN_ERR_LAUNCH, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(err));
    // the array comes into being when the library image is loaded on this device;
    // let that finish before the first stream-ordered use
    err = cudaDeviceSynchronize();
    if (err != cudaSuccess)
      return mellin::fail(MELLIN_ERR_LAUNCH, std::string("cudaDeviceSynchronize(static scratch): ") + cudaGetErrorString(err));
    g_device_ptr[dev] = static_cast<unsigned char *>(ptr);
  }
  *out = g_device_ptr[dev];
  *device = dev;
  return MELLIN_OK;
}

// Copies one host-built index map into the array at `offset` and returns a view of it.
int stage_table(const mellin::IndexMapKey &key, unsigned char *base, size_t *offset, mellin::DeviceTable *view,
                std::vector<int32_t> &host, cudaStream_t stream) {
  mellin::IndexMap m;
  try {
    m = mellin::build_index_map(key);
  } catch (const std::invalid_argument &e) {
    return mellin::fail(MELLIN_ERR_BAD_ARGUMENT, e.what());
  }
  const size_t n_ptr = m.row_ptr.size(), n_ord = m.order.size(), n_ent = m.entries.size();
  size_t ints = n_ptr + n_ord;
  ints += ints & 1;  // entries are 8-byte aligned
  const size_t bytes = (ints + 2 * n_ent) * sizeof(int32_t);
  const size_t begin = (*offset + 255) / 256 * 256;
  if (begin + bytes > kScratchBytes + kTableBytes)
    return mellin::fail(MELLIN_ERR_WORKSPACE, "index tables of this geometry need more than the " +
                                                  std::to_string(kTableBytes) + " bytes reserved in the static scratch");
  host.assign(ints + 2 * n_ent, 0);
  for (size_t i = 0; i < n_ptr; ++i) host[i] = m.row_ptr[i];
  for (size_t i = 0; i < n_ord; ++i) host[n_ptr + i] = m.order[i];
  for (size_t i = 0; i < n_ent; ++i) {
    host[ints + 2 * i] = m.entries[i].a;
    host[ints + 2 * i + 1] = m.entries[i].b;
  }
  // `host` lives in g_staged until another geometry replaces it
  cudaError_t err = cudaMemcpyAsync(base + begin, host.data(), bytes, cudaMemcpyHostToDevice, stream);
  if (err != cudaSuccess) return mellin::fail(MELLIN_ERR_LAUNCH, std::string("cudaMemcpyAsync(index table): ") + cudaGetErrorString(err));
  const int32_t *dev = reinterpret_cast<const int32_t *>(base + begin);
  view->row_ptr = dev;
  view->order = dev + n_ptr;
  view->entries = reinterpret_cast<const int2 *>(dev + ints);
  view->rows = m.rows;
  view->max_row = m.max_row;
  view->triples = m.triples;
  view->num_entries = static_cast<int64_t>(n_ent);
  *offset = begin + bytes;
  return MELLIN_OK;
}

}  // namespace

extern "C" int mellin_mcorrlcorr_grad_weight_noalloc_f32(const float *x, const float *grad_y, MELLIN_LAYER_GEOMETRY,
                                                         float *grad_w, float *grad_b, void *stream) {
  using namespace mellin;
  const char *who = "mcorrlcorr_grad_weight_noalloc";
  const int64_t extents[] = {batch, c_in, c_out, nfx, nfy, ngx, ngy, nhx, nhy};
  for (int64_t e : extents)
    if (e < 1 || e > (1LL << 29) - 1) return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": every extent must be in [1, 2^29)");
  if (px < 0 || uy < 1) return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": Mellin p must be >= 0 and linear u >= 1");
  if (x == nullptr || grad_y == nullptr || grad_w == nullptr)
    return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": null pointer");
  GradWProblem<float> p;
  p.in = x, p.go = grad_y, p.gw = grad_w, p.gb = grad_b;
  p.N = (int)batch, p.A = (int)c_out, p.B = (int)c_in;
  p.nkx = (int)nfx, p.nky = (int)nfy, p.nix = (int)ngx, p.niy = (int)ngy, p.nox = (int)nhx, p.noy = (int)nhy;
  p.Ay = (int)sy, p.By = (int)dy, p.Cy = -(int)py, p.Dy = (int)uy;
  // size check first: nothing is touched when the geometry does not fit
  // (the row-streaming kernel's need where it covers the problem: a faster kernel that wants more than the built-in
  // scratch holds simply declines, and the launch below falls through to this one)
  const size_t rows_need = gradw_rows_workspace_floats(p, nullptr) * sizeof(float);
  const size_t need = rows_need > 0 ? rows_need : gradw_workspace_bytes<float>(p);
  if (need > kScratchBytes)
    return fail(MELLIN_ERR_WORKSPACE, std::string(who) + ": the partial sums of this geometry need " + std::to_string(need) +
                                          " bytes, above the " + std::to_string(kScratchBytes) +
                                          " bytes of the built-in scratch; use mellin_mcorrlcorr_grad_weight_f32 with your own workspace");
  unsigned char *base = nullptr;
  int dev = 0;
  int rc = resolve_scratch(&base, &dev);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    StagedTables &st = g_staged[dev];
    const int64_t key[7] = {nfx, ngx, nhx, sx, dx, px, ux};
    bool same = st.valid;
    for (int i = 0; i < 7 && same; ++i) same = st.key[i] == key[i];
    if (!same) {
      st.valid = false;
      size_t offset = kScratchBytes;  // tables sit behind the partial sums
      rc = stage_table(IndexMapKey{Relation::Corr, SortBy::F, nfx, ngx, nhx, sx, dx, px, ux}, base, &offset, &st.by_f,
                       st.host_f, s);
      if (rc) return rc;
      rc = stage_table(IndexMapKey{Relation::Corr, SortBy::H, nfx, ngx, nhx, sx, dx, px, ux}, base, &offset, &st.by_h,
                       st.host_h, s);
      if (rc) return rc;
      for (int i = 0; i < 7; ++i) st.key[i] = key[i];
      st.valid = true;
    }
    p.table = st.by_f, p.table_h = st.by_h;
  }
  return launch_gradw<float>(p, base, kScratchBytes, s);
}
