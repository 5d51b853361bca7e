// C-ABI layer of libb2fil.so: error convention, forest lifetime, prediction entry points.
// Declarations and the reference interfaces they replace are in include/b2fil.h.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include "forest.hpp"
#include "kernels.hpp"
#include "kernels_q.hpp"

using namespace b2fil;

namespace {

thread_local std::string g_last_error;
std::atomic<int64_t> g_launches{0};

int set_error(int code, const std::string& msg)
{
  g_last_error = msg;
  return code;
}
int cuda_error(const char* what, cudaError_t e)
{
  return set_error(B2FIL_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

#define B2FIL_CUDA(call)                                  \
  do {                                                    \
    const cudaError_t e_ = (call);                        \
    if (e_ != cudaSuccess) return cuda_error(#call, e_);  \
  } while (0)

// Makes a device current for the lifetime of the guard and restores the previous one.
struct DeviceGuard {
  int prev = -1;
  bool ok  = false;
  explicit DeviceGuard(int dev)
  {
    if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    ok = cudaSetDevice(dev) == cudaSuccess;
  }
  ~DeviceGuard()
  {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

// Peer access is a per-process setting of a device pair.  It is switched on the first time a pair
// is used (forest replication, output gather) and remembered: 1 = `dev` maps `peer`'s memory
// directly (copies between them do not pass through host memory), 0 = it cannot.
std::mutex g_peer_mu;
std::map<std::pair<int, int>, int> g_peer;

int enable_peer_one_way(int dev, int peer)
{
  if (dev == peer) return 1;
  std::lock_guard<std::mutex> lock(g_peer_mu);
  const auto key = std::make_pair(dev, peer);
  const auto it  = g_peer.find(key);
  if (it != g_peer.end()) return it->second;
  int can = 0;
  if (cudaDeviceCanAccessPeer(&can, dev, peer) != cudaSuccess) {
    cudaGetLastError();
    can = 0;
  }
  if (can) {
    DeviceGuard guard(dev);
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
      cudaGetLastError();  // somebody else in the process (e.g. the array library) did it already
    } else if (e != cudaSuccess) {
      cudaGetLastError();
      can = 0;
    }
  }
  g_peer[key] = can;
  return can;
}

// Both directions: a peer copy is direct when either side can issue it, the library enables both.
int enable_peer_pair(int a, int b)
{
  const int ab = enable_peer_one_way(a, b);
  const int ba = enable_peer_one_way(b, a);
  return (ab && ba) ? 1 : 0;
}

// Device times of the calling thread's last b2fil_predict_sharded call.
struct ShardTiming {
  double compute_ms = 0, gather_ms = 0, wall_ms = 0;
  int direct = 0, valid = 0;
};
thread_local ShardTiming g_shard_timing;

// Pipeline shape of b2fil_predict_host (tuning aids B2FIL_HOST_BLOCK_MB / B2FIL_HOST_SLOTS, read
// from the environment once).
constexpr int kMaxHostSlots = 4;
struct HostPipeCfg {
  size_t block_bytes = size_t(256) << 20;
  int slots          = 2;
  // pageable arrays: smaller blocks through three pinned staging buffers, filled by a few threads
  size_t staged_block_bytes = size_t(64) << 20;
  int staged_slots          = 3;
  int copy_threads          = 0;
  HostPipeCfg()
  {
    const unsigned hw = std::thread::hardware_concurrency();
    copy_threads      = static_cast<int>(std::max(1u, std::min(8u, hw / 2)));
    if (const char* e = getenv("B2FIL_HOST_COPY_THREADS")) {
      const long n = atol(e);
      if (n >= 1 && n <= 64) copy_threads = static_cast<int>(n);
    }
    if (const char* e = getenv("B2FIL_HOST_STAGED_BLOCK_MB")) {
      const long mb = atol(e);
      if (mb >= 1 && mb <= 1024) staged_block_bytes = static_cast<size_t>(mb) << 20;
    }
    if (const char* e = getenv("B2FIL_HOST_BLOCK_MB")) {
      const long mb = atol(e);
      if (mb >= 1 && mb <= 4096) block_bytes = static_cast<size_t>(mb) << 20;
    }
    if (const char* e = getenv("B2FIL_HOST_SLOTS")) {
      const long n = atol(e);
      if (n >= 1 && n <= kMaxHostSlots) slots = static_cast<int>(n);
    }
  }
};
const HostPipeCfg& host_pipe_cfg()
{
  static const HostPipeCfg cfg;
  return cfg;
}

}  // namespace

// One slot of the host-buffer pipeline: device staging buffers and the stream that orders them.
struct HostSlot {
  cudaStream_t stream = nullptr;
  void* x             = nullptr;
  void* out           = nullptr;
  size_t x_bytes      = 0;
  size_t out_bytes    = 0;
  cudaEvent_t ev[3]   = {nullptr, nullptr, nullptr};  // sharded prediction: begin, kernels done, gathered
  // pageable host arrays: pinned staging on the host side of the copies
  void* pin_in         = nullptr;
  void* pin_out        = nullptr;
  size_t pin_in_bytes  = 0;
  size_t pin_out_bytes = 0;
  int64_t pending_r0   = -1;  // rows whose results sit in pin_out, not yet handed to the caller
  int64_t pending_n    = 0;
};

struct b2fil_forest {
  ForestView view{};
  int32_t precision = B2FIL_F32, storage = 0, layout = 0, align_bytes = 0, node_bytes = 0;
  int32_t device = 0, sm_count = 0, default_chunk = 0;
  int64_t n_nodes_in = 0, n_nodes_packed = 0, device_bytes = 0;
  int32_t* status = nullptr;
  cudaMemPool_t pool = nullptr;  // stream-ordered scratch of the rank-quantised path
  std::vector<uint32_t> q_top;   // host copy of the three top nodes per tree (may be empty)
  struct Block {
    void* ptr;
    size_t bytes;
    size_t view_offset;  // offset of the pointer member inside ForestView
  };
  std::vector<Block> blocks;
  int32_t clone_src_device = -1;  // device this forest was replicated from, or -1
  int32_t clone_direct     = -1;  // 1: that replication went over a direct peer path
  std::mutex host_mu;  // serialises the calls that use the slots below
  HostSlot slots[kMaxHostSlots];
  ~b2fil_forest()
  {
    DeviceGuard g(device);
    for (auto& b : blocks) cudaFree(b.ptr);
    if (status) cudaFree(status);
    if (pool) cudaMemPoolDestroy(pool);
    for (auto& s : slots) {
      if (s.x) cudaFree(s.x);
      if (s.out) cudaFree(s.out);
      if (s.stream) cudaStreamDestroy(s.stream);
      for (auto& e : s.ev)
        if (e) cudaEventDestroy(e);
      if (s.pin_in) cudaFreeHost(s.pin_in);
      if (s.pin_out) cudaFreeHost(s.pin_out);
    }
  }
};

namespace {

template <typename V>
int upload(b2fil_forest* f, const V& host, size_t view_offset)
{
  if (host.empty()) return B2FIL_OK;
  const size_t bytes = host.size() * sizeof(typename V::value_type);
  void* d            = nullptr;
  cudaError_t e      = cudaMalloc(&d, bytes);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    return set_error(B2FIL_ERR_NO_MEMORY, "device allocation of " + std::to_string(bytes) +
                                            " bytes for the forest failed");
  }
  if (e != cudaSuccess) return cuda_error("cudaMalloc", e);
  f->blocks.push_back({d, bytes, view_offset});
  f->device_bytes += static_cast<int64_t>(bytes);
  B2FIL_CUDA(cudaMemcpy(d, host.data(), bytes, cudaMemcpyHostToDevice));
  std::memcpy(reinterpret_cast<char*>(&f->view) + view_offset, &d, sizeof(void*));
  return B2FIL_OK;
}

int init_device_state(b2fil_forest* f)
{
  cudaDeviceProp prop;
  B2FIL_CUDA(cudaGetDeviceProperties(&prop, f->device));
  f->sm_count = prop.multiProcessorCount;
  B2FIL_CUDA(cudaMalloc(&f->status, sizeof(int32_t)));
  B2FIL_CUDA(cudaMemset(f->status, 0, sizeof(int32_t)));
  // a pool of its own keeps freed scratch cached between predictions without touching the
  // settings of the device's default pool
  cudaMemPoolProps props{};
  props.allocType     = cudaMemAllocationTypePinned;
  props.handleTypes   = cudaMemHandleTypeNone;
  props.location.type = cudaMemLocationTypeDevice;
  props.location.id   = f->device;
  B2FIL_CUDA(cudaMemPoolCreate(&f->pool, &props));
  uint64_t keep = ~uint64_t(0);
  B2FIL_CUDA(cudaMemPoolSetAttribute(f->pool, cudaMemPoolAttrReleaseThreshold, &keep));
  return B2FIL_OK;
}

size_t elem_bytes(const b2fil_forest* f) { return f->precision == B2FIL_F32 ? 4 : 8; }

int64_t out_elems(const b2fil_forest* f, int kind)
{
  switch (kind) {
    case B2FIL_INFER_DEFAULT: return f->view.n_outputs;
    case B2FIL_INFER_PER_TREE:
      return static_cast<int64_t>(f->view.n_trees) *
             (f->view.leaf_vector_len > 1 ? f->view.n_outputs : 1);
    case B2FIL_INFER_LEAF_ID: return f->view.n_trees;
    case B2FIL_INFER_CLASS: return 1;
    case B2FIL_INFER_PROBA2: return 2;
    default: return 0;
  }
}
size_t out_elem_bytes(const b2fil_forest* f, int kind)
{
  if (kind == B2FIL_INFER_LEAF_ID || kind == B2FIL_INFER_CLASS) return 4;
  return elem_bytes(f);
}

int check_predict_args(const b2fil_forest* f, int kind, const void* X, int64_t n_rows,
                       int64_t row_stride, const void* out)
{
  if (!f) return set_error(B2FIL_ERR_INVALID_ARG, "forest is NULL");
  if (out_elems(f, kind) == 0) return set_error(B2FIL_ERR_INVALID_ARG, "unknown infer_kind");
  if (n_rows < 0) return set_error(B2FIL_ERR_INVALID_ARG, "n_rows is negative");
  if (n_rows > 0 && (!X || !out)) return set_error(B2FIL_ERR_INVALID_ARG, "NULL buffer");
  if (row_stride < f->view.n_features)
    return set_error(B2FIL_ERR_INVALID_ARG, "row_stride is smaller than n_features");
  if (kind == B2FIL_INFER_PROBA2 && f->view.n_outputs != 1)
    return set_error(B2FIL_ERR_INVALID_ARG, "B2FIL_INFER_PROBA2 needs a forest with one output");
  return B2FIL_OK;
}

int enqueue(const b2fil_forest* f, int kind, const void* X, int64_t n_rows, int64_t row_stride,
            void* out, int chunk_size, double threshold, cudaStream_t stream)
{
  PredictParams p{};
  p.f          = f->view;
  p.X          = X;
  p.n_rows     = n_rows;
  p.row_stride = row_stride;
  p.out        = out;
  p.kind       = kind;
  p.threshold  = threshold;
  p.status     = f->status;
  p.q_top      = f->q_top.empty() ? nullptr : f->q_top.data();
  std::string err;
  int64_t n = 0;
  const int rc =
    launch_predict(p, chunk_size > 0 ? chunk_size : f->default_chunk, f->sm_count, stream, f->pool,
                   err, &n);
  g_launches += n;
  if (rc != B2FIL_OK) return set_error(rc, err);
  return B2FIL_OK;
}

int ensure_slot(b2fil_forest* f, HostSlot& s, size_t x_bytes, size_t out_bytes)
{
  if (!s.stream) B2FIL_CUDA(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking));
  if (s.x_bytes < x_bytes) {
    if (s.x) cudaFree(s.x);
    s.x = nullptr;
    s.x_bytes = 0;
    B2FIL_CUDA(cudaMalloc(&s.x, x_bytes));
    s.x_bytes = x_bytes;
  }
  if (s.out_bytes < out_bytes) {
    if (s.out) cudaFree(s.out);
    s.out = nullptr;
    s.out_bytes = 0;
    B2FIL_CUDA(cudaMalloc(&s.out, out_bytes));
    s.out_bytes = out_bytes;
  }
  (void)f;
  return B2FIL_OK;
}

// Read and clear the status word.  The caller has already waited for the work it cares about.
int read_status_word(const b2fil_forest* f, int32_t* status)
{
  B2FIL_CUDA(cudaMemcpy(status, f->status, sizeof(int32_t), cudaMemcpyDeviceToHost));
  if (*status != 0) {
    // reported once: the next prediction starts from a clean word
    B2FIL_CUDA(cudaMemset(f->status, 0, sizeof(int32_t)));
    static const char* const where[] = {"", "tree ring (producer)", "tree ring (consumer)",
                                        "row-tile buffer", "rank tables", "self test"};
    const char* w = (*status >= 1 && *status <= 5) ? where[*status] : "unknown";
    return set_error(B2FIL_ERR_TIMEOUT, std::string("a bounded wait inside a kernel ran out: ") +
                                          w + " (status " + std::to_string(*status) + ")");
  }
  return B2FIL_OK;
}

// True when the CUDA runtime does not know the host pointer: ordinary (pageable) memory.  Copies
// from such memory are staged by the driver through a small internal buffer and run at a
// fraction of the link; the library stages them itself instead.
bool is_pageable(const void* p)
{
  cudaPointerAttributes a{};
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return true;
  }
  return a.type == cudaMemoryTypeUnregistered;
}

int ensure_pinned(void** buf, size_t* have, size_t want)
{
  if (*have >= want) return B2FIL_OK;
  if (*buf) cudaFreeHost(*buf);
  *buf  = nullptr;
  *have = 0;
  const cudaError_t e = cudaHostAlloc(buf, want, cudaHostAllocDefault);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return set_error(B2FIL_ERR_NO_MEMORY, std::string("pinned staging buffer: ") + cudaGetErrorString(e));
  }
  *have = want;
  return B2FIL_OK;
}

// Copy `n_rows` rows of `row_bytes` bytes (source rows `src_stride` bytes apart) into a dense
// buffer with `threads` host threads: one thread cannot fill a PCIe 5 link from pageable memory.
void parallel_rows_copy(char* dst, const char* src, int64_t n_rows, size_t row_bytes,
                        size_t src_stride, int threads)
{
  auto work = [=](int64_t b, int64_t e) {
    if (src_stride == row_bytes) {
      std::memcpy(dst + static_cast<size_t>(b) * row_bytes, src + static_cast<size_t>(b) * src_stride,
                  static_cast<size_t>(e - b) * row_bytes);
    } else {
      for (int64_t r = b; r < e; ++r)
        std::memcpy(dst + static_cast<size_t>(r) * row_bytes, src + static_cast<size_t>(r) * src_stride,
                    row_bytes);
    }
  };
  const int64_t min_rows = std::max<int64_t>(1, static_cast<int64_t>((size_t(4) << 20) / std::max<size_t>(1, row_bytes)));
  const int t = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(threads, n_rows / min_rows)));
  if (t <= 1) {
    work(0, n_rows);
    return;
  }
  std::vector<std::thread> pool;
  pool.reserve(t - 1);
  for (int i = 1; i < t; ++i) pool.emplace_back(work, n_rows * i / t, n_rows * (i + 1) / t);
  work(0, n_rows / t);
  for (auto& th : pool) th.join();
}

// Host-array prediction for pageable inputs: row blocks are gathered into pinned staging buffers
// by several host threads while the previous blocks are copied and predicted; results come back
// through pinned buffers too.  The caller holds the forest's host mutex and has made its device
// current.
int predict_host_staged(b2fil_forest* f, int infer_kind, const char* xin, int64_t n_rows,
                        int64_t row_stride, char* yout, int chunk_size, double threshold)
{
  const HostPipeCfg& pipe = host_pipe_cfg();
  const size_t es        = elem_bytes(f);
  const int64_t F        = f->view.n_features;
  const size_t in_row_b  = static_cast<size_t>(F) * es;
  const size_t out_row_b = static_cast<size_t>(out_elems(f, infer_kind)) * out_elem_bytes(f, infer_kind);
  int64_t block_rows = static_cast<int64_t>(
    std::max<size_t>(1, pipe.staged_block_bytes / std::max(in_row_b, out_row_b)));
  block_rows = std::max<int64_t>(block_rows / 128 * 128, 128);
  block_rows = std::min(block_rows, n_rows);
  const int S = pipe.staged_slots;
  int rc      = B2FIL_OK;
  for (int i = 0; i < S && rc == B2FIL_OK; ++i) {
    HostSlot& s = f->slots[i];
    rc = ensure_slot(f, s, static_cast<size_t>(block_rows) * in_row_b,
                     static_cast<size_t>(block_rows) * out_row_b);
    if (rc == B2FIL_OK) rc = ensure_pinned(&s.pin_in, &s.pin_in_bytes, static_cast<size_t>(block_rows) * in_row_b);
    if (rc == B2FIL_OK) rc = ensure_pinned(&s.pin_out, &s.pin_out_bytes, static_cast<size_t>(block_rows) * out_row_b);
    s.pending_r0 = -1;
  }
  if (rc != B2FIL_OK) return rc;  // nothing has been enqueued yet
  // hand a slot's finished results to the caller (after its stream has drained)
  auto flush = [&](HostSlot& s) -> int {
    if (s.pending_r0 < 0) return B2FIL_OK;
    const cudaError_t e = cudaStreamSynchronize(s.stream);
    if (e != cudaSuccess) return cuda_error("cudaStreamSynchronize", e);
    std::memcpy(yout + static_cast<size_t>(s.pending_r0) * out_row_b, s.pin_out,
                static_cast<size_t>(s.pending_n) * out_row_b);
    s.pending_r0 = -1;
    return B2FIL_OK;
  };
  int which = 0;
  for (int64_t r0 = 0; r0 < n_rows && rc == B2FIL_OK; r0 += block_rows, which = (which + 1) % S) {
    HostSlot& s     = f->slots[which];
    const int64_t n = std::min(block_rows, n_rows - r0);
    if ((rc = flush(s)) != B2FIL_OK) break;  // also frees the slot's staging buffers for reuse
    parallel_rows_copy(static_cast<char*>(s.pin_in), xin + static_cast<size_t>(r0) * row_stride * es,
                       n, in_row_b, static_cast<size_t>(row_stride) * es, pipe.copy_threads);
    cudaError_t e = cudaMemcpyAsync(s.x, s.pin_in, static_cast<size_t>(n) * in_row_b,
                                    cudaMemcpyHostToDevice, s.stream);
    if (e != cudaSuccess) {
      rc = cuda_error("host-to-device copy of a row block", e);
      break;
    }
    rc = enqueue(f, infer_kind, s.x, n, F, s.out, chunk_size, threshold, s.stream);
    if (rc != B2FIL_OK) break;
    e = cudaMemcpyAsync(s.pin_out, s.out, static_cast<size_t>(n) * out_row_b, cudaMemcpyDeviceToHost,
                        s.stream);
    if (e != cudaSuccess) {
      rc = cuda_error("device-to-host copy of a result block", e);
      break;
    }
    s.pending_r0 = r0;
    s.pending_n  = n;
  }
  // drain every slot, also after an error: copies in flight still use the staging buffers
  for (int i = 0; i < S; ++i) {
    HostSlot& s = f->slots[i];
    if (rc == B2FIL_OK) {
      rc = flush(s);
    } else if (s.stream) {
      cudaStreamSynchronize(s.stream);
      s.pending_r0 = -1;
    }
  }
  if (rc != B2FIL_OK) return rc;
  int32_t status = 0;
  return read_status_word(f, &status);
}

}  // namespace

extern "C" {

const char* b2fil_last_error(void) { return g_last_error.c_str(); }

int b2fil_version(void) { return 100; }

int64_t b2fil_kernel_launches(void) { return g_launches.load(); }

int b2fil_forest_create(const b2fil_forest_desc* desc, const b2fil_create_opts* opts,
                        b2fil_forest** out)
{
  if (!desc || !opts || !out) return set_error(B2FIL_ERR_INVALID_ARG, "NULL argument");
  *out = nullptr;
  try {
    int n_dev = 0;
    cudaError_t e = cudaGetDeviceCount(&n_dev);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return set_error(B2FIL_ERR_CUDA, std::string("no usable CUDA device: ") +
                                         cudaGetErrorString(e));
    }
    if (opts->device_id < 0 || opts->device_id >= n_dev)
      return set_error(B2FIL_ERR_INVALID_ARG, "device_id " + std::to_string(opts->device_id) +
                                                " out of range (" + std::to_string(n_dev) +
                                                " devices)");
    PackedForest pf;
    std::string err;
    int rc = pack_forest(*desc, *opts, dense_ok, pf, err);
    if (rc != B2FIL_OK) return set_error(rc, err);

    std::unique_ptr<b2fil_forest> f(new b2fil_forest());
    f->device = opts->device_id;
    DeviceGuard guard(f->device);
    if (!guard.ok) return set_error(B2FIL_ERR_CUDA, "cudaSetDevice failed");
    f->view           = pf.view;
    f->precision      = pf.precision;
    f->storage        = pf.storage;
    f->layout         = opts->layout;
    f->align_bytes    = pf.align_bytes;
    f->node_bytes     = pf.node_bytes;
    f->n_nodes_in     = pf.n_nodes_in;
    f->n_nodes_packed = pf.n_nodes_packed;
    f->default_chunk  = std::max(0, opts->default_chunk_size);
    if ((rc = init_device_state(f.get())) != B2FIL_OK) return rc;
    if ((rc = upload(f.get(), pf.nodes, offsetof(ForestView, nodes))) != B2FIL_OK) return rc;
    if ((rc = upload(f.get(), pf.roots, offsetof(ForestView, roots))) != B2FIL_OK) return rc;
    if ((rc = upload(f.get(), pf.leaf_ids, offsetof(ForestView, leaf_ids))) != B2FIL_OK) return rc;
    if ((rc = upload(f.get(), pf.cat_pool, offsetof(ForestView, cat_pool))) != B2FIL_OK) return rc;
    if ((rc = upload(f.get(), pf.tree_class, offsetof(ForestView, tree_class))) != B2FIL_OK)
      return rc;
    if ((rc = upload(f.get(), pf.tree_orig, offsetof(ForestView, tree_orig))) != B2FIL_OK)
      return rc;
    if ((rc = upload(f.get(), pf.leaf_vectors, offsetof(ForestView, leaf_vectors))) != B2FIL_OK)
      return rc;
    if ((rc = upload(f.get(), pf.out_scale, offsetof(ForestView, out_scale))) != B2FIL_OK)
      return rc;
    if ((rc = upload(f.get(), pf.out_bias, offsetof(ForestView, out_bias))) != B2FIL_OK) return rc;
    if (pf.view.c_enabled) {
      if ((rc = upload(f.get(), pf.c_nodes, offsetof(ForestView, c_nodes))) != B2FIL_OK) return rc;
      if ((rc = upload(f.get(), pf.c_exact, offsetof(ForestView, c_exact))) != B2FIL_OK) return rc;
      if ((rc = upload(f.get(), pf.c_leaf_payload, offsetof(ForestView, c_leaf_payload))) != B2FIL_OK)
        return rc;
      if ((rc = upload(f.get(), pf.c_leaf_ids, offsetof(ForestView, c_leaf_ids))) != B2FIL_OK)
        return rc;
      if ((rc = upload(f.get(), pf.c_top, offsetof(ForestView, c_top))) != B2FIL_OK) return rc;
      if ((rc = upload(f.get(), pf.c_top_src, offsetof(ForestView, c_top_src))) != B2FIL_OK)
        return rc;
    }
    if (pf.view.q_enabled) {
      if ((rc = upload(f.get(), pf.q_nodes, offsetof(ForestView, q_nodes))) != B2FIL_OK) return rc;
      if ((rc = upload(f.get(), pf.q_nodes_ids, offsetof(ForestView, q_nodes_ids))) != B2FIL_OK)
        return rc;
      if ((rc = upload(f.get(), pf.q_blob, offsetof(ForestView, q_blob))) != B2FIL_OK) return rc;
      if ((rc = upload(f.get(), pf.q_groups, offsetof(ForestView, q_groups))) != B2FIL_OK)
        return rc;
      f->q_top = std::move(pf.q_top);
    }
    *out = f.release();
    return B2FIL_OK;
  } catch (const std::bad_alloc&) {
    return set_error(B2FIL_ERR_NO_MEMORY, "host allocation failed while packing the forest");
  } catch (const std::exception& ex) {
    return set_error(B2FIL_ERR_INVALID_ARG, std::string("unexpected failure: ") + ex.what());
  }
}

int b2fil_forest_clone_to_device(const b2fil_forest* src, int device_id, b2fil_forest** out)
{
  if (!src || !out) return set_error(B2FIL_ERR_INVALID_ARG, "NULL argument");
  *out = nullptr;
  try {
    int n_dev = 0;
    B2FIL_CUDA(cudaGetDeviceCount(&n_dev));
    if (device_id < 0 || device_id >= n_dev)
      return set_error(B2FIL_ERR_INVALID_ARG, "device_id out of range");
    std::unique_ptr<b2fil_forest> f(new b2fil_forest());
    f->view           = src->view;
    f->precision      = src->precision;
    f->storage        = src->storage;
    f->layout         = src->layout;
    f->align_bytes    = src->align_bytes;
    f->node_bytes     = src->node_bytes;
    f->n_nodes_in     = src->n_nodes_in;
    f->n_nodes_packed = src->n_nodes_packed;
    f->default_chunk  = src->default_chunk;
    f->q_top          = src->q_top;
    f->device         = device_id;
    DeviceGuard guard(device_id);
    if (!guard.ok) return set_error(B2FIL_ERR_CUDA, "cudaSetDevice failed");
    int rc;
    if ((rc = init_device_state(f.get())) != B2FIL_OK) return rc;
    f->clone_src_device = src->device;
    f->clone_direct     = enable_peer_pair(device_id, src->device);
    for (const auto& b : src->blocks) {
      void* d       = nullptr;
      cudaError_t e = cudaMalloc(&d, b.bytes);
      if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        return set_error(B2FIL_ERR_NO_MEMORY, "device allocation for the forest copy failed");
      }
      if (e != cudaSuccess) return cuda_error("cudaMalloc", e);
      f->blocks.push_back({d, b.bytes, b.view_offset});
      f->device_bytes += static_cast<int64_t>(b.bytes);
      // direct over the peer path when it could be enabled above, staged through the host
      // otherwise
      B2FIL_CUDA(cudaMemcpyPeer(d, device_id, b.ptr, src->device, b.bytes));
      std::memcpy(reinterpret_cast<char*>(&f->view) + b.view_offset, &d, sizeof(void*));
    }
    *out = f.release();
    return B2FIL_OK;
  } catch (const std::bad_alloc&) {
    return set_error(B2FIL_ERR_NO_MEMORY, "host allocation failed");
  }
}

int b2fil_forest_free(b2fil_forest* f)
{
  delete f;
  return B2FIL_OK;
}

int b2fil_forest_info(const b2fil_forest* f, b2fil_info* info)
{
  if (!f || !info) return set_error(B2FIL_ERR_INVALID_ARG, "NULL argument");
  std::memset(info, 0, sizeof(*info));
  info->precision          = f->precision;
  info->layout             = f->layout;
  info->storage            = f->storage;
  info->device_id          = f->device;
  info->n_trees            = f->view.n_trees;
  info->n_features         = f->view.n_features;
  info->n_outputs          = f->view.n_outputs;
  info->leaf_vector_len    = f->view.leaf_vector_len;
  info->max_depth          = f->view.max_depth;
  info->dense_depth        = f->view.dense_depth;
  info->node_bytes         = f->node_bytes;
  info->has_categorical    = f->view.has_categorical;
  info->n_nodes_in         = f->n_nodes_in;
  info->n_nodes_packed     = f->n_nodes_packed;
  info->device_bytes       = f->device_bytes;
  info->default_chunk_size = f->default_chunk;
  info->row_quantization   = f->view.q_enabled;
  info->compact_image      = f->view.c_enabled;
  info->top_levels         = f->view.c_enabled ? f->view.c_top_levels : 0;
  info->peer_direct        = f->clone_direct;
  info->clone_src_device   = f->clone_src_device;
  if (f->pool) {
    uint64_t reserved = 0;
    if (cudaMemPoolGetAttribute(f->pool, cudaMemPoolAttrReservedMemCurrent, &reserved) == cudaSuccess)
      info->scratch_pool_bytes = static_cast<int64_t>(reserved);
    else
      cudaGetLastError();
  }
  return B2FIL_OK;
}

int64_t b2fil_output_elems_per_row(const b2fil_forest* f, int infer_kind)
{
  if (!f) {
    set_error(B2FIL_ERR_INVALID_ARG, "forest is NULL");
    return 0;
  }
  const int64_t n = out_elems(f, infer_kind);
  if (n == 0) set_error(B2FIL_ERR_INVALID_ARG, "unknown infer_kind");
  return n;
}


int b2fil_forest_status(const b2fil_forest* f, int32_t* status)
{
  if (!f || !status) return set_error(B2FIL_ERR_INVALID_ARG, "NULL argument");
  DeviceGuard guard(f->device);
  if (!guard.ok) return set_error(B2FIL_ERR_CUDA, "cudaSetDevice failed");
  // every stream of the device, the non-blocking ones included: a plain copy on the default
  // stream would not wait for them
  B2FIL_CUDA(cudaDeviceSynchronize());
  return read_status_word(f, status);
}

int b2fil_forest_selftest_timeout(b2fil_forest* f, int tries, void* cuda_stream)
{
  if (!f) return set_error(B2FIL_ERR_INVALID_ARG, "forest is NULL");
  if (tries < 1 || tries > 4096)
    return set_error(B2FIL_ERR_INVALID_ARG, "tries must be between 1 and 4096");
  DeviceGuard guard(f->device);
  if (!guard.ok) return set_error(B2FIL_ERR_CUDA, "cudaSetDevice failed");
  std::string err;
  const int rc = launch_bounded_wait_selftest(f->status, static_cast<uint32_t>(tries),
                                              static_cast<cudaStream_t>(cuda_stream), err);
  if (rc != B2FIL_OK) return set_error(rc, err);
  return B2FIL_OK;
}

int b2fil_enable_peer_access(int device_a, int device_b)
{
  int n_dev = 0;
  B2FIL_CUDA(cudaGetDeviceCount(&n_dev));
  if (device_a < 0 || device_b < 0 || device_a >= n_dev || device_b >= n_dev)
    return set_error(B2FIL_ERR_INVALID_ARG, "device ordinal out of range");
  return enable_peer_pair(device_a, device_b);
}

int b2fil_set_tuning(const char* key, int value)
{
  if (!key) return set_error(B2FIL_ERR_INVALID_ARG, "key is NULL");
  set_tuning_value(key, value);
  return B2FIL_OK;
}

int b2fil_last_variant(char* buf, size_t buf_bytes)
{
  if (!buf || buf_bytes == 0) return set_error(B2FIL_ERR_INVALID_ARG, "NULL or empty buffer");
  const std::string v = last_launch_variant();
  const size_t n      = std::min(v.size(), buf_bytes - 1);
  std::memcpy(buf, v.data(), n);
  buf[n] = 0;
  return static_cast<int>(v.size());
}

int b2fil_last_sharded_timing(double* compute_ms, double* gather_ms, double* wall_ms,
                              int* gather_direct)
{
  const ShardTiming& t = g_shard_timing;
  if (!t.valid) return set_error(B2FIL_ERR_INVALID_ARG, "no sharded prediction on this thread yet");
  if (compute_ms) *compute_ms = t.compute_ms;
  if (gather_ms) *gather_ms = t.gather_ms;
  if (wall_ms) *wall_ms = t.wall_ms;
  if (gather_direct) *gather_direct = t.direct;
  return B2FIL_OK;
}

int b2fil_predict(const b2fil_forest* f, int infer_kind, const void* X_dev, int64_t n_rows,
                  int64_t row_stride, void* out_dev, int chunk_size, double threshold,
                  void* cuda_stream)
{
  int rc = check_predict_args(f, infer_kind, X_dev, n_rows, row_stride, out_dev);
  if (rc != B2FIL_OK) return rc;
  DeviceGuard guard(f->device);
  if (!guard.ok) return set_error(B2FIL_ERR_CUDA, "cudaSetDevice failed");
  return enqueue(f, infer_kind, X_dev, n_rows, row_stride, out_dev, chunk_size, threshold,
                 static_cast<cudaStream_t>(cuda_stream));
}

int b2fil_predict_fixed_scratch(const b2fil_forest* f, int infer_kind, const void* X_dev,
                                int64_t n_rows, int64_t row_stride, void* out_dev, int chunk_size,
                                double threshold, void* cuda_stream)
{
  int rc = check_predict_args(f, infer_kind, X_dev, n_rows, row_stride, out_dev);
  if (rc != B2FIL_OK) return rc;
  DeviceGuard guard(f->device);
  if (!guard.ok) return set_error(B2FIL_ERR_CUDA, "cudaSetDevice failed");
  PredictParams p{};
  p.f          = f->view;
  p.X          = X_dev;
  p.n_rows     = n_rows;
  p.row_stride = row_stride;
  p.out        = out_dev;
  p.kind       = infer_kind;
  p.threshold  = threshold;
  p.status     = f->status;
  p.q_top      = f->q_top.empty() ? nullptr : f->q_top.data();
  std::string err;
  int64_t n = 0;
  rc = launch_predict_fixed_scratch(p, chunk_size > 0 ? chunk_size : f->default_chunk,
                                    f->sm_count, f->device,
                                    static_cast<cudaStream_t>(cuda_stream), err, &n);
  g_launches += n;
  if (rc != B2FIL_OK) return set_error(rc, err);
  return B2FIL_OK;
}

int b2fil_predict_host(b2fil_forest* f, int infer_kind, const void* X_host, int64_t n_rows,
                       int64_t row_stride, void* out_host, int chunk_size, double threshold)
{
  int rc = check_predict_args(f, infer_kind, X_host, n_rows, row_stride, out_host);
  if (rc != B2FIL_OK) return rc;
  if (n_rows == 0) return B2FIL_OK;
  std::lock_guard<std::mutex> lock(f->host_mu);
  DeviceGuard guard(f->device);
  if (!guard.ok) return set_error(B2FIL_ERR_CUDA, "cudaSetDevice failed");
  const size_t es        = elem_bytes(f);
  const int64_t F        = f->view.n_features;
  const size_t in_row_b  = static_cast<size_t>(F) * es;
  const size_t out_row_b = static_cast<size_t>(out_elems(f, infer_kind)) * out_elem_bytes(f, infer_kind);
  // ordinary (pageable) arrays of some size go through the library's own pinned staging
  if (static_cast<size_t>(n_rows) * in_row_b >= (size_t(8) << 20) && is_pageable(X_host))
    return predict_host_staged(f, infer_kind, static_cast<const char*>(X_host), n_rows, row_stride,
                               static_cast<char*>(out_host), chunk_size, threshold);
  // row blocks of about 256 MiB of input (and at most 256 MiB of output) keep both copy engines
  // and the SMs busy while two blocks are in flight
  const HostPipeCfg& pipe = host_pipe_cfg();
  const size_t budget     = pipe.block_bytes;
  int64_t block_rows  = static_cast<int64_t>(std::max<size_t>(1, budget / std::max(in_row_b, out_row_b)));
  block_rows          = std::max<int64_t>(block_rows / 128 * 128, 128);
  block_rows          = std::min(block_rows, n_rows);
  for (int i = 0; i < pipe.slots; ++i) {
    rc = ensure_slot(f, f->slots[i], static_cast<size_t>(block_rows) * in_row_b,
                     static_cast<size_t>(block_rows) * out_row_b);
    if (rc != B2FIL_OK) return rc;  // nothing has been enqueued yet
  }
  const char* xin = static_cast<const char*>(X_host);
  char* yout      = static_cast<char*>(out_host);
  int which       = 0;
  for (int64_t r0 = 0; r0 < n_rows && rc == B2FIL_OK; r0 += block_rows, which = (which + 1) % pipe.slots) {
    HostSlot& s     = f->slots[which];
    const int64_t n = std::min(block_rows, n_rows - r0);
    // stream order makes the slot's previous block finish before its buffers are reused
    cudaError_t e;
    if (row_stride == F) {
      e = cudaMemcpyAsync(s.x, xin + static_cast<size_t>(r0) * in_row_b,
                          static_cast<size_t>(n) * in_row_b, cudaMemcpyHostToDevice, s.stream);
    } else {
      e = cudaMemcpy2DAsync(s.x, in_row_b, xin + static_cast<size_t>(r0) * row_stride * es,
                            static_cast<size_t>(row_stride) * es, in_row_b, static_cast<size_t>(n),
                            cudaMemcpyHostToDevice, s.stream);
    }
    if (e != cudaSuccess) {
      rc = cuda_error("host-to-device copy of a row block", e);
      break;
    }
    rc = enqueue(f, infer_kind, s.x, n, F, s.out, chunk_size, threshold, s.stream);
    if (rc != B2FIL_OK) break;
    e = cudaMemcpyAsync(yout + static_cast<size_t>(r0) * out_row_b, s.out,
                        static_cast<size_t>(n) * out_row_b, cudaMemcpyDeviceToHost, s.stream);
    if (e != cudaSuccess) rc = cuda_error("device-to-host copy of a result block", e);
  }
  // Also after an error: copies already enqueued still read and write the caller's buffers, so
  // the call may not return before they are done.
  for (int i = 0; i < pipe.slots; ++i) {
    if (!f->slots[i].stream) continue;
    const cudaError_t e = cudaStreamSynchronize(f->slots[i].stream);
    if (e != cudaSuccess && rc == B2FIL_OK) rc = cuda_error("cudaStreamSynchronize", e);
  }
  if (rc != B2FIL_OK) return rc;
  int32_t status = 0;
  return read_status_word(f, &status);
}

int b2fil_predict_sharded(b2fil_forest* const* forests, int n_devices, int infer_kind,
                          const void* const* X_shards, const int64_t* shard_rows,
                          int64_t row_stride, void* out_dev0, int chunk_size, double threshold)
{
  if (!forests || !X_shards || !shard_rows || n_devices <= 0)
    return set_error(B2FIL_ERR_INVALID_ARG, "NULL argument or no devices");
  for (int i = 0; i < n_devices; ++i) {
    if (!forests[i]) return set_error(B2FIL_ERR_INVALID_ARG, "forest is NULL");
    const int rc = check_predict_args(forests[i], infer_kind, X_shards[i], shard_rows[i],
                                      row_stride, out_dev0);
    if (rc != B2FIL_OK) return rc;
  }
  for (int i = 0; i < n_devices; ++i) {
    for (int j = 0; j < i; ++j) {
      if (forests[i] == forests[j] || forests[i]->device == forests[j]->device)
        return set_error(B2FIL_ERR_INVALID_ARG, "every shard needs its own forest on its own device");
    }
  }
  b2fil_forest* f0       = forests[0];
  const size_t out_row_b = static_cast<size_t>(out_elems(f0, infer_kind)) * out_elem_bytes(f0, infer_kind);
  // every device predicts its shard on its own stream; shards of devices other than the first
  // land in a staging buffer on their device and are pushed to device 0 by a peer copy.
  // The forests' locks are taken in address order, so two callers that pass the same forests in
  // different orders cannot wait for each other.
  std::vector<b2fil_forest*> by_address(forests, forests + n_devices);
  std::sort(by_address.begin(), by_address.end(), std::less<b2fil_forest*>());
  std::vector<std::unique_lock<std::mutex>> locks;
  for (b2fil_forest* f : by_address) locks.emplace_back(f->host_mu);
  int direct = 1;
  for (int i = 1; i < n_devices; ++i)
    direct &= enable_peer_pair(forests[i]->device, f0->device);

  const auto t0  = std::chrono::steady_clock::now();
  int rc_final   = B2FIL_OK;
  int64_t row_off = 0;
  std::vector<int> fed;  // devices that have work enqueued
  for (int i = 0; i < n_devices && rc_final == B2FIL_OK; ++i) {
    b2fil_forest* f = forests[i];
    DeviceGuard guard(f->device);
    if (!guard.ok) {
      rc_final = set_error(B2FIL_ERR_CUDA, "cudaSetDevice failed");
      break;
    }
    HostSlot& s     = f->slots[0];
    const int64_t n = shard_rows[i];
    char* dst0      = static_cast<char*>(out_dev0) + static_cast<size_t>(row_off) * out_row_b;
    row_off += n;
    if (n == 0) continue;
    const bool local = f->device == f0->device;
    int rc = ensure_slot(f, s, 0, local ? 0 : static_cast<size_t>(n) * out_row_b);
    for (auto& ev : s.ev) {
      if (rc == B2FIL_OK && !ev && cudaEventCreate(&ev) != cudaSuccess)
        rc = set_error(B2FIL_ERR_CUDA, "cudaEventCreate failed");
    }
    if (rc != B2FIL_OK) {
      rc_final = rc;
      break;
    }
    fed.push_back(i);
    cudaEventRecord(s.ev[0], s.stream);
    rc = enqueue(f, infer_kind, X_shards[i], n, row_stride, local ? static_cast<void*>(dst0) : s.out,
                 chunk_size, threshold, s.stream);
    cudaEventRecord(s.ev[1], s.stream);
    if (rc == B2FIL_OK && !local) {
      const cudaError_t e = cudaMemcpyPeerAsync(dst0, f0->device, s.out, f->device,
                                                static_cast<size_t>(n) * out_row_b, s.stream);
      if (e != cudaSuccess) rc = cuda_error("cudaMemcpyPeerAsync", e);
    }
    cudaEventRecord(s.ev[2], s.stream);
    if (rc != B2FIL_OK) rc_final = rc;
  }
  // Wait for every device that was fed, also after an error on a later device: their kernels and
  // copies still write into the caller's output.
  ShardTiming timing;
  for (int i : fed) {
    b2fil_forest* f = forests[i];
    DeviceGuard guard(f->device);
    HostSlot& s         = f->slots[0];
    const cudaError_t e = cudaStreamSynchronize(s.stream);
    if (e != cudaSuccess) {
      if (rc_final == B2FIL_OK) rc_final = cuda_error("cudaStreamSynchronize", e);
      continue;
    }
    float ms = 0;
    if (cudaEventElapsedTime(&ms, s.ev[0], s.ev[1]) == cudaSuccess)
      timing.compute_ms = std::max(timing.compute_ms, static_cast<double>(ms));
    if (cudaEventElapsedTime(&ms, s.ev[1], s.ev[2]) == cudaSuccess)
      timing.gather_ms = std::max(timing.gather_ms, static_cast<double>(ms));
    int32_t status = 0;
    const int rc   = read_status_word(f, &status);
    if (rc != B2FIL_OK && rc_final == B2FIL_OK) rc_final = rc;
  }
  timing.wall_ms =
    std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
  timing.direct  = direct;
  timing.valid   = 1;
  g_shard_timing = timing;
  return rc_final;
}

}  // extern "C"
