// Device-side building blocks shared by every kernel translation unit: shared-memory and
// mbarrier primitives (inline PTX), per-precision traits, the node test, row staging, the CTA
// epilogue (reduction over tree groups, averaging, base score, postprocessor, output
// conversion) and the leaf bookkeeping.  Everything lives in an unnamed namespace: each
// translation unit that includes this file gets its own copy.
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <type_traits>
#include <utility>

#include "kernels.hpp"

namespace b2fil {
namespace {


#ifndef B2FIL_SPIN_NS
#define B2FIL_SPIN_NS 256  // sleep between two tries of a bounded mbarrier wait
#endif
constexpr uint32_t kSpinLimit = 1u << 22;  // tries of a bounded mbarrier wait
constexpr int kBarBytes       = 256;       // room for the mbarriers at the start of shared memory
constexpr int kMaxStages      = 8;

// ---------------------------------------------------------------------------------------------
// shared-memory and mbarrier primitives (inline PTX)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p)
{
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init()
{
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
  uint32_t ok;
  asm volatile(
    "{\n"
    ".reg .pred p;\n"
    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
    "selp.u32 %0, 1, 0, p;\n"
    "}\n"
    : "=r"(ok)
    : "r"(bar), "r"(parity)
    : "memory");
  return ok != 0;
}
// Bounded wait: false when the barrier did not complete within `limit` tries (each try blocks
// for a hardware-defined short time, then the warp sleeps briefly).
__device__ __forceinline__ bool mbar_wait_limited(uint32_t bar, uint32_t parity, uint32_t limit)
{
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    // a waiting warp must not compete for issue slots with the warps that are walking trees
#if B2FIL_SPIN_NS > 0
    __nanosleep(B2FIL_SPIN_NS);
#endif
  }
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity)
{
  return mbar_wait_limited(bar, parity, kSpinLimit);
}
// Position in a ring of S stages: the stage index and the parity of its current use, advanced
// without a division.
struct RingPos {
  uint32_t stage = 0, phase = 0;
  __device__ __forceinline__ void advance(int S)
  {
    if (++stage == static_cast<uint32_t>(S)) {
      stage = 0;
      phase ^= 1u;
    }
  }
};

// Bulk asynchronous copy global -> shared memory of this CTA, completing `bytes` on `bar`.
// Both addresses are 16-byte aligned and `bytes` is a multiple of 16.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                              uint32_t bar)
{
  asm volatile(
    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
      dst),
    "l"(src), "r"(bytes), "r"(bar)
    : "memory");
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t a)
{
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t a)
{
  uint32_t v;  // a 16-bit load into a 32-bit register zero-extends
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
// Barrier among the consumer threads only (the producer warp never joins it).
__device__ __forceinline__ void consumer_sync(int n_threads)
{
  asm volatile("bar.sync 1, %0;" ::"r"(n_threads) : "memory");
}

// ---------------------------------------------------------------------------------------------
// per-precision traits
// ---------------------------------------------------------------------------------------------
template <typename T>
struct Traits;

template <>
struct Traits<float> {
  using Val                    = uint32_t;
  static constexpr uint32_t NB = 8;  // dense node bytes
  static constexpr uint32_t ES = 4;  // element bytes (rows, leaves, outputs)
  static __device__ __forceinline__ void ld_node(uint32_t a, Val& v, uint32_t& m)
  {
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v), "=r"(m) : "r"(a));
  }
  static __device__ __forceinline__ float ld_real(uint32_t a)
  {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
  }
  // read-only global load that stays where it is written (the compiler may not sink it)
  static __device__ __forceinline__ float ldg_here(const float* ptr)
  {
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(ptr));
    return v;
  }
  template <uint32_t OFF>
  static __device__ __forceinline__ float ld_real_at(uint32_t a)  // [a + OFF], OFF an immediate
  {
    float v;
    asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(a), "n"(OFF));
    return v;
  }
  // a += inc when t <= x (false for NaN), as one predicated add
  static __device__ __forceinline__ void add_if_le(uint32_t& a, float t, float x, uint32_t inc)
  {
    asm("{\n.reg .pred p;\nsetp.le.f32 p, %1, %2;\n@p add.u32 %0, %0, %3;\n}"
        : "+r"(a)
        : "f"(t), "f"(x), "r"(inc));
  }
  static __device__ __forceinline__ void st_real(uint32_t a, float v)
  {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory");
  }
  static __device__ __forceinline__ Val ld_val(uint32_t a)
  {
    Val v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
  }
  static __device__ __forceinline__ float as_real(Val v) { return __uint_as_float(v); }
  static __device__ __forceinline__ uint32_t low32(Val v) { return v; }
  static __device__ __forceinline__ float exp_(float x) { return expf(x); }
  static __device__ __forceinline__ float exp2_(float x) { return exp2f(x); }
  static __device__ __forceinline__ float log1p_(float x) { return log1pf(x); }
};

template <>
struct Traits<double> {
  using Val                    = uint64_t;
  static constexpr uint32_t NB = 16;
  static constexpr uint32_t ES = 8;
  static __device__ __forceinline__ void ld_node(uint32_t a, Val& v, uint32_t& m)
  {
    uint64_t second;
    asm volatile("ld.shared.v2.u64 {%0, %1}, [%2];" : "=l"(v), "=l"(second) : "r"(a));
    m = static_cast<uint32_t>(second);
  }
  static __device__ __forceinline__ double ld_real(uint32_t a)
  {
    double v;
    asm volatile("ld.shared.f64 %0, [%1];" : "=d"(v) : "r"(a));
    return v;
  }
  static __device__ __forceinline__ double ldg_here(const double* ptr)
  {
    double v;
    asm volatile("ld.global.nc.f64 %0, [%1];" : "=d"(v) : "l"(ptr));
    return v;
  }
  template <uint32_t OFF>
  static __device__ __forceinline__ double ld_real_at(uint32_t a)
  {
    double v;
    asm volatile("ld.shared.f64 %0, [%1+%2];" : "=d"(v) : "r"(a), "n"(OFF));
    return v;
  }
  static __device__ __forceinline__ void add_if_le(uint32_t& a, double t, double x, uint32_t inc)
  {
    asm("{\n.reg .pred p;\nsetp.le.f64 p, %1, %2;\n@p add.u32 %0, %0, %3;\n}"
        : "+r"(a)
        : "d"(t), "d"(x), "r"(inc));
  }
  static __device__ __forceinline__ void st_real(uint32_t a, double v)
  {
    asm volatile("st.shared.f64 [%0], %1;" ::"r"(a), "d"(v) : "memory");
  }
  static __device__ __forceinline__ Val ld_val(uint32_t a)
  {
    Val v;
    asm volatile("ld.shared.u64 %0, [%1];" : "=l"(v) : "r"(a));
    return v;
  }
  static __device__ __forceinline__ double as_real(Val v) { return __longlong_as_double(v); }
  static __device__ __forceinline__ uint32_t low32(Val v) { return static_cast<uint32_t>(v); }
  static __device__ __forceinline__ double exp_(double x) { return exp(x); }
  static __device__ __forceinline__ double exp2_(double x) { return exp2(x); }
  static __device__ __forceinline__ double log1p_(double x) { return log1p(x); }
};

// ---------------------------------------------------------------------------------------------
// one test: does the row go to the right child?
//   numerical: x < threshold goes left; categorical: a listed category goes right;
//   a missing value (NaN) follows the node's default direction.
// ---------------------------------------------------------------------------------------------
template <typename T, bool CAT, bool NANS>
__device__ __forceinline__ bool goes_right(typename Traits<T>::Val v, uint32_t meta, T x,
                                           const ForestView& f)
{
  bool left = x < Traits<T>::as_real(v);
  if (CAT) {
    if (meta & META_CATEGORICAL) {
      // category = truncated value; negative and huge values match nothing
      const bool in_range = (x >= T(0)) && (x < T(16777216));
      const uint32_t c    = in_range ? static_cast<uint32_t>(x) : 0u;
      bool matched;
      if (f.cat_inline) {
        const uint32_t bits = Traits<T>::low32(v);
        matched             = in_range && (c < 32u) && (((bits >> (c & 31u)) & 1u) != 0u);
      } else {
        const uint32_t off     = Traits<T>::low32(v);
        const uint32_t n_words = __ldg(f.cat_pool + off);
        const uint32_t w       = c >> 5;
        matched                = false;
        if (in_range && w < n_words) {
          matched = ((__ldg(f.cat_pool + off + 1 + w) >> (c & 31u)) & 1u) != 0u;
        }
      }
      left = !matched;
    }
  }
  if (CAT || NANS) {
    if (x != x) left = (meta & META_DEFAULT_LEFT) != 0u;
  }
  return !left;
}

// ---------------------------------------------------------------------------------------------
// shared pieces of both kernels: row-tile staging, accumulation of a leaf, epilogue
// ---------------------------------------------------------------------------------------------

// Stage rows [row0, row0+R) feature-major.  A warp reads 32 consecutive features of one row
// (one 128-byte line for fp32) and scatters them to 32 different banks.  Rows past the end of the
// batch are filled with zeros.  Returns true when this thread saw a NaN.
template <typename T>
__device__ __forceinline__ bool stage_rows(const PredictParams& p, uint32_t tile, int R,
                                           int64_t row0, int warp, int lane, int n_warps)
{
  const int F             = p.f.n_features;
  const uint32_t stride_b = (R + 1) * Traits<T>::ES;
  const T* X              = static_cast<const T*>(p.X);
  bool saw_nan            = false;
  for (int rr = warp; rr < R; rr += n_warps) {
    const int64_t row = row0 + rr;
    const bool live   = row < p.n_rows;
    const T* src      = X + row * p.row_stride;
    for (int c = lane; c < F; c += 32) {
      const T v = live ? __ldg(src + c) : T(0);
      saw_nan |= (v != v);
      Traits<T>::st_real(tile + c * stride_b + rr * Traits<T>::ES, v);
    }
  }
  return saw_nan;
}

template <typename T>
__device__ __forceinline__ T postprocess_one(T s, int postproc, T alpha, T ratio_c)
{
  switch (postproc) {
    case B2FIL_POST_SIGMOID:
    case B2FIL_POST_MULTICLASS_OVA: return T(1) / (T(1) + Traits<T>::exp_(-alpha * s));
    case B2FIL_POST_EXPONENTIAL: return Traits<T>::exp_(s);
    case B2FIL_POST_LOG1PEXP: return Traits<T>::log1p_(Traits<T>::exp_(s));
    case B2FIL_POST_SIGNED_SQUARE: return (s < T(0) ? T(-1) : T(1)) * s * s;
    case B2FIL_POST_HINGE: return s > T(0) ? T(1) : T(0);
    case B2FIL_POST_EXP_STD_RATIO: return Traits<T>::exp2_(-s / ratio_c);
    default: return s;
  }
}

// Epilogue of a row tile, one thread per row: fixed-order sum over the G tree groups, average and
// base score, postprocessor, then the output the caller asked for.  `acc` is laid out
// [group][output][row]; results overwrite group 0.
template <typename T>
__device__ __forceinline__ void finish_row(const PredictParams& p, T* acc, int R, int G, int j,
                                           int64_t row)
{
  const ForestView& f = p.f;
  const int NC        = f.n_outputs;
  const T* scale      = static_cast<const T*>(f.out_scale);
  const T* bias       = static_cast<const T*>(f.out_bias);
  const T alpha       = static_cast<T>(f.sigmoid_alpha);
  const T ratio_c     = static_cast<T>(f.ratio_c);
  T mx                = T(0);
  for (int c = 0; c < NC; ++c) {
    T s = acc[c * R + j];
    for (int g = 1; g < G; ++g) s += acc[(g * NC + c) * R + j];
    s = s * __ldg(scale + c) + __ldg(bias + c);
    if (f.postproc != B2FIL_POST_SOFTMAX) s = postprocess_one(s, f.postproc, alpha, ratio_c);
    acc[c * R + j] = s;
    mx             = (c == 0 || s > mx) ? s : mx;
  }
  if (f.postproc == B2FIL_POST_SOFTMAX) {
    T z = T(0);
    for (int c = 0; c < NC; ++c) {
      const T e      = Traits<T>::exp_(acc[c * R + j] - mx);
      acc[c * R + j] = e;
      z += e;
    }
    for (int c = 0; c < NC; ++c) acc[c * R + j] = acc[c * R + j] / z;
  }
  if (row >= p.n_rows) return;
  if (p.kind == B2FIL_INFER_DEFAULT) {
    T* out = static_cast<T*>(p.out) + row * NC;
    for (int c = 0; c < NC; ++c) out[c] = acc[c * R + j];
  } else if (p.kind == B2FIL_INFER_PROBA2) {
    T* out       = static_cast<T*>(p.out) + row * 2;
    const T prob = acc[j];
    out[0]       = T(1) - prob;
    out[1]       = prob;
  } else {  // B2FIL_INFER_CLASS
    int best = 0;
    if (NC == 1) {
      best = acc[j] > static_cast<T>(p.threshold) ? 1 : 0;
    } else {
      T bv = acc[j];
      for (int c = 1; c < NC; ++c) {
        const T s = acc[c * R + j];
        if (s > bv) {  // first maximum wins
          bv   = s;
          best = c;
        }
      }
    }
    static_cast<int32_t*>(p.out)[row] = best;
  }
}

// Kernel modes.
constexpr int MODE_SCALAR  = 0;  // scalar leaves, reduced outputs
constexpr int MODE_VECTOR  = 1;  // vector leaves, reduced outputs
constexpr int MODE_PERTREE = 2;  // raw per-tree outputs
constexpr int MODE_LEAFID  = 3;  // id of the leaf reached

// Per-thread running state of the reduced modes: the sum of the class that scalar leaves are
// currently feeding, or, for vector leaves of up to kRegClasses outputs, one sum per output
// (forests with more outputs add every leaf vector to shared memory directly).
constexpr int kRegClasses = kQInlineClasses;
template <typename T>
struct Running {
  T sum;
  int cls;
  T v[kRegClasses];
};

// Consume one leaf.  `payload` is the leaf's scalar (as bits) or the index of its vector;
// `leaf_id_index` is the index of the leaf in `leaf_ids`.
template <typename T, int MODE>
__device__ __forceinline__ void take_leaf(const PredictParams& p, int tree,
                                          typename Traits<T>::Val payload, uint32_t leaf_id_index,
                                          T* acc_group, int R, int r, int64_t row, Running<T>& run)
{
  const ForestView& f = p.f;
  const int NC        = f.n_outputs;
  if (MODE == MODE_SCALAR) {
    if (NC > 1) {
      const int cls = __ldg(f.tree_class + tree);  // same for the whole warp
      if (cls != run.cls) {
        acc_group[run.cls * R + r] += run.sum;
        run.sum = T(0);
        run.cls = cls;
      }
    }
    run.sum += Traits<T>::as_real(payload);
  } else if (MODE == MODE_VECTOR) {
    const T* lv = static_cast<const T*>(f.leaf_vectors) +
                  static_cast<size_t>(Traits<T>::low32(payload)) * NC;
    if (NC <= kRegClasses) {
      // few outputs (binary and small multi-class forests of vector leaves, i.e. every
      // scikit-learn style random-forest classifier): sums stay in registers until the tile ends
#pragma unroll
      for (int c = 0; c < kRegClasses; ++c) {
        if (c < NC) run.v[c] += __ldg(lv + c);
      }
    } else {
      // four outputs at a time: the loads of a chunk are in flight together (one after the other
      // they cost a load latency per output)
      int c = 0;
      // (vectors of a multiple of four floats start on 16-byte boundaries: one load per chunk)
      const bool wide = sizeof(T) == 4 && (NC & 3) == 0;
      for (; c + 4 <= NC; c += 4) {
        T v[4], a[4];
        if (wide) {
          const float4 q = __ldg(reinterpret_cast<const float4*>(lv + c));
          v[0] = static_cast<T>(q.x);
          v[1] = static_cast<T>(q.y);
          v[2] = static_cast<T>(q.z);
          v[3] = static_cast<T>(q.w);
        } else {
#pragma unroll
          for (int u = 0; u < 4; ++u) v[u] = __ldg(lv + c + u);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) a[u] = acc_group[(c + u) * R + r];
#pragma unroll
        for (int u = 0; u < 4; ++u) acc_group[(c + u) * R + r] = a[u] + v[u];
      }
      for (; c < NC; ++c) acc_group[c * R + r] += __ldg(lv + c);
    }
  } else if (MODE == MODE_PERTREE) {
    if (row < p.n_rows) {
      const int orig = __ldg(f.tree_orig + tree);
      if (f.leaf_vector_len > 1) {
        const T* lv = static_cast<const T*>(f.leaf_vectors) +
                      static_cast<size_t>(Traits<T>::low32(payload)) * NC;
        T* out = static_cast<T*>(p.out) + (row * f.n_trees + orig) * NC;
        for (int c = 0; c < NC; ++c) out[c] = __ldg(lv + c);
      } else {
        static_cast<T*>(p.out)[row * f.n_trees + orig] = Traits<T>::as_real(payload);
      }
    }
  } else {
    if (row < p.n_rows) {
      const int orig = __ldg(f.tree_orig + tree);
      static_cast<uint32_t*>(p.out)[row * f.n_trees + orig] = __ldg(f.leaf_ids + leaf_id_index);
    }
  }
}

// Add a thread's running sums to its accumulators in shared memory (end of a row tile).
template <typename T, int MODE>
__device__ __forceinline__ void flush_running(const ForestView& f, const Running<T>& run,
                                              T* acc_group, int R, int r)
{
  if (MODE == MODE_SCALAR) acc_group[run.cls * R + r] += run.sum;
  if (MODE == MODE_VECTOR && f.n_outputs <= kRegClasses) {
#pragma unroll
    for (int c = 0; c < kRegClasses; ++c) {
      if (c < f.n_outputs) acc_group[c * R + r] += run.v[c];
    }
  }
}

__host__ __device__ inline size_t align16(size_t x) { return (x + 15) / 16 * 16; }

// Position of row r among the R uint16 entries of one feature in a rank tile.  Rows r and r + 32
// share a 32-bit word, so the 32 consecutive rows of a warp sit in 32 different banks whatever
// feature each lane reads (with the plain order two neighbouring rows share a bank and collide
// as soon as they read different features).  Tiles of 32 rows keep the plain order.
__device__ __forceinline__ uint32_t q_slot(uint32_t r, int R)
{
  return R >= 64 ? (((r & 31u) << 1) | ((r >> 5) & 1u) | ((r >> 6) << 6)) : r;
}
// The row that sits in slot s (inverse of q_slot).
__device__ __forceinline__ uint32_t q_row_of_slot(uint32_t s, int R)
{
  return R >= 64 ? (((s >> 6) << 6) | ((s & 63u) >> 1) | ((s & 1u) << 5)) : s;
}

}  // namespace
}  // namespace b2fil
