// Prediction kernels for sm_100a.
//
// Work decomposition (both storages): a CTA owns a tile of R consecutive rows, staged once in
// shared memory feature-major (`tile[f][r]`, row stride R+1 elements) so that the 32 lanes of a
// warp - 32 different rows - always read 32 different banks whatever feature each lane needs.
// Warps are organised as (R/32 row sets) x (G tree groups): every warp walks its 32 rows through
// the trees of its group, NT trees at a time for instruction-level parallelism, and keeps its
// partial sums private; a fixed-order reduction over the G groups, averaging, base score and the
// postprocessor run in the CTA's epilogue, so one launch reads every row once and writes every
// result once.
//
// DENSE storage: trees are complete and heap ordered, so a step is "load node, load feature,
// compare, index = 2*index + went_right" with no child pointer.  A producer warp streams batches
// of G*NT whole trees from global memory (L2 resident) into a ring of shared-memory stages with
// bulk asynchronous copies (cp.async.bulk, completion on an mbarrier); consumer warps release a
// stage through a second mbarrier.  CTAs are persistent (one per SM) and loop over row tiles.
//
// SPARSE storage: nodes are fetched from global memory through the read-only path; each thread
// keeps NT independent traversals in flight to cover the latency of the dependent loads.
//
// Every wait on an mbarrier is bounded: when the bound is hit the kernel sets the status word,
// stops working and returns.
#include <map>
#include <mutex>

#include "device_common.cuh"
#include "kernels_q.hpp"

namespace b2fil {
namespace {
// What the calling thread launched last (see last_launch_variant()).  Plain data: filling it costs
// a few stores per call, the text is only formatted when somebody asks.
struct LaunchRecord {
  const char* prepass = nullptr;  // kernel that ran before the traversal, or null
  const char* kernel  = nullptr;  // traversal kernel family
  const char* real    = "";       // float / double
  int mode = 0, nt = 0, depth = -1, cat = -1, fmt = -1, top = -1;
  int R = 0, G = 0, S = 0, K = 0, splits = 1;
};
thread_local LaunchRecord g_last_launch;

const char* mode_name(int mode)
{
  switch (mode) {
    case 0: return "scalar";
    case 1: return "vector";
    case 2: return "per_tree";
    default: return "leaf_id";
  }
}

// ---------------------------------------------------------------------------------------------
// bounded-wait self test
// ---------------------------------------------------------------------------------------------
__global__ void bounded_wait_selftest_kernel(int32_t* status, const uint32_t tries)
{
  __shared__ __align__(8) unsigned long long bar_word;
  const uint32_t bar = smem_addr(&bar_word);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);  // one arrival expected; nothing ever arrives
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0 && !mbar_wait_limited(bar, 0, tries)) atomicExch(status, 5);
}

// ---------------------------------------------------------------------------------------------
// DENSE kernel
// ---------------------------------------------------------------------------------------------
// Shared memory: [mbarriers 128 B][row tile][accumulators][flags 16 B][S tree stages].
template <typename T, bool CAT, int MODE, int NT>
struct DenseWalker {
  using TR = Traits<T>;

  // Walk the warp's rows through all trees of the CTA's current tile.
  template <bool NANS>
  static __device__ __forceinline__ bool walk(const PredictParams& p, int G, int S, int g, int r,
                                              int64_t row, int lane, uint32_t bars,
                                              uint32_t stages, uint32_t stage_bytes,
                                              uint32_t row_addr, uint32_t stride_b, T* acc_group,
                                              int R, RingPos& pos, Running<T>& run, int b_begin,
                                              int b_end)
  {
    const ForestView& f    = p.f;
    const int D            = f.dense_depth;
    const uint32_t tstride = static_cast<uint32_t>(f.tree_stride);
    const uint32_t width_b = (1u << D) * TR::NB;  // bytes of the node array of one tree
    const int per_batch    = G * NT;
    bool ok                = true;
    for (int b = b_begin; b < b_end; ++b) {
      const uint32_t s = pos.stage;
      if (ok) ok = mbar_wait(bars + 8u * s, pos.phase);
      if (ok) {
        const int first = b * per_batch + g * NT;
        const int n_act = min(NT, f.n_trees - first);
        if (n_act > 0) {
          uint32_t base[NT], a[NT];
#pragma unroll
          for (int k = 0; k < NT; ++k) {
            // slots past the end of the forest repeat the last live tree; results are dropped
            const int slot = g * NT + min(k, n_act - 1);
            base[k]        = stages + s * stage_bytes + slot * tstride;
            a[k]           = base[k] + TR::NB;  // heap index 1
          }
          for (int lvl = 0; lvl < D; ++lvl) {
#pragma unroll
            for (int k = 0; k < NT; ++k) {
              typename TR::Val v;
              uint32_t meta;
              TR::ld_node(a[k], v, meta);
              // flag bits 30/31 of meta leave the 32-bit product: stride_b is a multiple of 4
              const T x        = TR::ld_real(meta * stride_b + row_addr);
              const bool right = goes_right<T, CAT, NANS>(v, meta, x, f);
              // address of heap node 2i+right from the address of node i
              a[k] = 2u * a[k] - base[k] + (right ? TR::NB : 0u);
            }
          }
#pragma unroll
          for (int k = 0; k < NT; ++k) {
            if (k < n_act) {
              const uint32_t slot = (a[k] - base[k]) / TR::NB - (1u << D);
              const typename TR::Val payload = TR::ld_val(base[k] + width_b + slot * TR::ES);
              take_leaf<T, MODE>(p, first + k, payload,
                                 (static_cast<uint32_t>(first + k) << D) + slot, acc_group, R, r,
                                 row, run);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8u * (kMaxStages + s));
      pos.advance(S);
    }
    return ok;
  }
};

template <typename T, bool CAT, int MODE, int NT>
__global__ void __launch_bounds__(544, 1)
dense_kernel(const PredictParams p, const int R, const int G, const int S, const int n_splits,
             T* __restrict__ partial)
{
  using TR = Traits<T>;
  extern __shared__ __align__(128) unsigned char smem[];
  const ForestView& f = p.f;
  const int F         = f.n_features;
  const int NC        = f.n_outputs;
  const int rw        = R >> 5;
  const int n_cw      = rw * G;        // consumer warps
  const int n_ct      = n_cw * 32;     // consumer threads
  const int warp      = threadIdx.x >> 5;
  const int lane      = threadIdx.x & 31;

  const uint32_t stride_b   = (R + 1) * TR::ES;
  const size_t tile_bytes   = align16(static_cast<size_t>(F) * stride_b);
  const size_t acc_bytes    = (MODE <= MODE_VECTOR) ? align16(static_cast<size_t>(G) * NC * R * TR::ES) : 0;
  unsigned char* tile_ptr   = smem + kBarBytes;
  T* acc                    = reinterpret_cast<T*>(tile_ptr + tile_bytes);
  volatile int* flags       = reinterpret_cast<volatile int*>(tile_ptr + tile_bytes + acc_bytes);
  unsigned char* stage_ptr  = tile_ptr + tile_bytes + acc_bytes + 16;
  const uint32_t bars       = smem_addr(smem);
  const uint32_t tile       = smem_addr(tile_ptr);
  const uint32_t stages     = smem_addr(stage_ptr);
  const uint32_t tstride    = static_cast<uint32_t>(f.tree_stride);
  const int per_batch       = G * NT;
  const uint32_t stage_bytes = per_batch * tstride;
  const int n_batches       = (f.n_trees + per_batch - 1) / per_batch;
  // small batches split the forest over blockIdx.y: every CTA streams and walks only its share
  // of the tree batches and leaves raw partial sums for finish_kernel
  const int b_begin = static_cast<int>(static_cast<int64_t>(n_batches) * blockIdx.y / n_splits);
  const int b_end   = static_cast<int>(static_cast<int64_t>(n_batches) * (blockIdx.y + 1) / n_splits);
  const int64_t n_tiles     = (p.n_rows + R - 1) / R;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bars + 8u * s, 1);                    // full: the producer's expect_tx arrival
      mbar_init(bars + 8u * (kMaxStages + s), n_cw);  // empty: one arrival per consumer warp
    }
    flags[0] = 0;
    flags[1] = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == n_cw) {
    // ---- producer: one thread streams tree batches into the stage ring ----------------------
    if (lane == 0) {
      const unsigned char* src = static_cast<const unsigned char*>(f.nodes);
      RingPos pos;
      bool primed = false;  // every stage has been filled once
      for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        for (int b = b_begin; b < b_end; ++b) {
          const uint32_t s = pos.stage;
          if (primed && !mbar_wait(bars + 8u * (kMaxStages + s), pos.phase ^ 1u)) {
            atomicExch(p.status, 1);
            return;
          }
          const int first      = b * per_batch;
          const int count      = min(per_batch, f.n_trees - first);
          const uint32_t bytes = count * tstride;
          mbar_expect_tx(bars + 8u * s, bytes);
          bulk_copy_g2s(stages + s * stage_bytes, src + static_cast<size_t>(first) * tstride,
                        bytes, bars + 8u * s);
          pos.advance(S);
          if (pos.stage == 0) primed = true;
        }
      }
    }
    return;
  }

  // ---- consumers ------------------------------------------------------------------------------
  const int g           = warp / rw;
  const int r           = (warp % rw) * 32 + lane;
  T* acc_group          = acc + static_cast<size_t>(g) * NC * R;
  const uint32_t row_addr = tile + r * TR::ES;
  RingPos pos;
  bool ok               = true;
  for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const int64_t row0 = t * R;
    const bool saw_nan = stage_rows<T>(p, tile, R, row0, warp, lane, n_cw);
    if (MODE <= MODE_VECTOR) {
      for (int i = threadIdx.x; i < G * NC * R; i += n_ct) acc[i] = T(0);
    }
    if (__any_sync(0xffffffffu, saw_nan) && lane == 0) flags[0] = 1;
    consumer_sync(n_ct);
    const bool nans = flags[0] != 0;
    Running<T> run{T(0), 0, {}};
    if (ok) {
      if (CAT || nans) {
        ok = DenseWalker<T, CAT, MODE, NT>::template walk<true>(
          p, G, S, g, r, row0 + r, lane, bars, stages, stage_bytes, row_addr, stride_b, acc_group,
          R, pos, run, b_begin, b_end);
      } else {
        ok = DenseWalker<T, CAT, MODE, NT>::template walk<false>(
          p, G, S, g, r, row0 + r, lane, bars, stages, stage_bytes, row_addr, stride_b, acc_group,
          R, pos, run, b_begin, b_end);
      }
      if (!ok) atomicExch(p.status, 2);
    }
    flush_running<T, MODE>(f, run, acc_group, R, r);
    consumer_sync(n_ct);
    if (MODE <= MODE_VECTOR) {
      if (threadIdx.x < R) {
        if (n_splits == 1) {
          finish_row<T>(p, acc, R, G, threadIdx.x, row0 + threadIdx.x);
        } else if (row0 + threadIdx.x < p.n_rows) {
          // raw sums of this CTA's trees, laid out [split][output][row]
          for (int c = 0; c < NC; ++c) {
            T sum = acc[c * R + threadIdx.x];
            for (int gg = 1; gg < G; ++gg) sum += acc[(gg * NC + c) * R + threadIdx.x];
            partial[(static_cast<int64_t>(blockIdx.y) * NC + c) * p.n_rows + row0 + threadIdx.x] = sum;
          }
        }
      }
    }
    if (threadIdx.x == 0) flags[0] = 0;
    consumer_sync(n_ct);
  }
}

// Second step of a split prediction: one warp per row adds the partial sums of the splits - lane
// l takes splits l, l + 32, ..., then a shuffle tree: a fixed order, and the loads of a row are
// in flight together (one thread per row spent 6 us on 63 dependent loads for a one-row batch) -
// and lane 0 applies averaging, base score, postprocessor and the output conversion.
// `partial` is laid out [split][output][row], which is the accumulator layout finish_row expects
// with the row count as the row stride; the sums of a row replace its split-0 slots.
template <typename T>
__global__ void __launch_bounds__(256)
finish_kernel(const PredictParams p, T* __restrict__ partial, const int n_splits)
{
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane    = threadIdx.x & 31;
  if (row >= p.n_rows) return;  // whole warps
  const int NC = p.f.n_outputs;
  for (int c = 0; c < NC; ++c) {
    T sum = T(0);
    for (int g = lane; g < n_splits; g += 32)
      sum += partial[(static_cast<int64_t>(g) * NC + c) * p.n_rows + row];
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, off);
    if (lane == 0) partial[static_cast<int64_t>(c) * p.n_rows + row] = sum;
  }
  if (lane == 0) finish_row<T>(p, partial, static_cast<int>(p.n_rows), 1, static_cast<int>(row), row);
}

// The same with one thread per row, for the larger of the small batches: a handful of splits,
// thousands of rows.
template <typename T>
__global__ void __launch_bounds__(256)
finish_few_splits_kernel(const PredictParams p, T* __restrict__ partial, const int n_splits)
{
  const int64_t row = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (row >= p.n_rows) return;
  finish_row<T>(p, partial, static_cast<int>(p.n_rows), n_splits, static_cast<int>(row), row);
}

// ---------------------------------------------------------------------------------------------
// RANK QUANTISATION of rows (pre-pass of the quantised dense kernel)
// ---------------------------------------------------------------------------------------------
// Calls f(std::integral_constant<int, K>) for K = 0, 1, ...: a loop whose counter is a constant
// expression inside the body.
template <typename F, int... Ks>
__device__ __forceinline__ void for_each_constant(F&& f, std::integer_sequence<int, Ks...>)
{
  (f(std::integral_constant<int, Ks>{}), ...);
}

// One CTA owns one feature group: the group's blob (feature records, bucket tables, sorted
// thresholds, both tables interleaved across the group's features) arrives in shared memory with
// one bulk copy, then the CTA loops over row tiles.  The group size GF is a power of two that
// divides the thread count, so a thread keeps one feature for good (its record sits in registers)
// and with 32-feature groups a warp reads 128 contiguous bytes of one row per load and its 32
// table lookups never share a bank.  A thread owns NU consecutive slots of the rank tile (slot =
// q_slot(row)); it ranks them four at a time while the loads of its next tile are in flight,
// packs the ranks two per word and writes its piece of Q[tile][feature][slot] (uint16) with one
// vector store, the layout the traversal kernel pulls into shared memory with a single bulk
// copy.  Nothing is exchanged between threads, so the tile loop has no barrier.  NaN becomes
// Q_NAN_CODE and raises the tile's flag.
// Shared memory: [mbarrier 16 B][blob].

// NU = slots of a tile each thread owns (R * GF / threads, at least 1).  GFC > 0 fixes the group
// size at compile time (table strides become immediates), GFC == 0 reads it from the group.
template <typename T, int STEPS, int NU, int GFC>
__device__ __forceinline__ void quantise_tiles(const PredictParams& p, const QGroup& grp,
                                               uint16_t* __restrict__ Q,
                                               int32_t* __restrict__ tile_flags, int R,
                                               uint32_t blob_a, const QFeatRec* rec)
{
  using TR               = Traits<T>;
  constexpr int CH       = NU < 4 ? NU : 4;  // values ranked side by side
  constexpr int NCH      = NU / CH;
  const int GF           = GFC > 0 ? GFC : static_cast<int>(grp.f_end - grp.f_begin);
  const int tid          = threadIdx.x;
  const int gshift       = 31 - __clz(GF);
  const int i            = tid & (GF - 1);
  const uint32_t s0      = static_cast<uint32_t>(tid >> gshift) * NU;  // first slot of the thread
  const bool active      = s0 < static_cast<uint32_t>(R);  // false only when a tile has fewer values than threads
  const QFeatRec mine    = rec[i];
  const T scale          = static_cast<T>(mine.scale);
  const T offset         = static_cast<T>(mine.offset);
  const T nbm1           = static_cast<T>(mine.nbm1);
  const uint32_t lut_row = static_cast<uint32_t>(GF) * 2u;      // bytes between table entries
  const uint32_t thr_row = static_cast<uint32_t>(GF) * TR::ES;  // bytes between thresholds
  const int eshift       = gshift + (TR::ES == 4 ? 2 : 3);      // log2(thr_row)
  const uint32_t lut     = blob_a + mine.lut_off;
  const uint32_t thr_m1  = blob_a + mine.thr_off - thr_row;
  const bool any_cat     = __any_sync(0xffffffffu, mine.is_cat != 0);
  const int64_t tile_elems = static_cast<int64_t>(p.f.n_features) * R;  // ranks per tile
  const uint32_t q_mine  = (grp.f_begin + i) * static_cast<uint32_t>(R) + s0;  // thread's first rank in a tile
  const int64_t n_tiles  = (p.n_rows + R - 1) / R;
  // slots s0 + j, j = 0..NU-1, hold rows b + (j >> 1) + 32 * (j & 1) (NU >= 2 implies R >= 64 and
  // an even s0); element offsets inside a tile fit 32 bits (the host sizes row chunks accordingly)
  const uint32_t b       = q_row_of_slot(s0, R);
  const uint32_t e1      = static_cast<uint32_t>(p.row_stride);
  const uint32_t e32     = e1 * 32u;
  const uint32_t e_mine  = b * e1 + grp.f_begin + i;
  const T* X             = static_cast<const T*>(p.X);

  T xs[NU];
  // loads chunk c (slots s0 + c * CH ...) of tile t
  auto fetch = [&](int64_t t, int c) {
    const int64_t row0 = t * R;
    const T* tb        = X + row0 * p.row_stride;  // same for the whole CTA
    const uint32_t cb  = e_mine + static_cast<uint32_t>(c * (CH / 2)) * e1;
    if (row0 + R <= p.n_rows) {
#pragma unroll
      for (int u = 0; u < CH; ++u)
        xs[c * CH + u] = active ? TR::ldg_here(tb + (cb + (u >> 1) * e1 + (u & 1) * e32)) : T(0);
    } else {
#pragma unroll
      for (int u = 0; u < CH; ++u) {
        const int64_t row = row0 + b + c * (CH / 2) + (u >> 1) + 32 * (u & 1);
        xs[c * CH + u] =
          (active && row < p.n_rows) ? TR::ldg_here(tb + (cb + (u >> 1) * e1 + (u & 1) * e32)) : T(0);
      }
    }
  };
  if (blockIdx.x < n_tiles) {
#pragma unroll
    for (int c = 0; c < NCH; ++c) fetch(blockIdx.x, c);
  }
  for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    uint32_t packed[NU > 1 ? NU / 2 : 1];
    bool saw_nan = false;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      T cur[CH];
#pragma unroll
      for (int u = 0; u < CH; ++u) cur[u] = xs[c * CH + u];
      // the same chunk of the CTA's next tile is requested right away, so a whole tile of loads
      // per thread stays in flight (an additional L2 prefetch further ahead measured slower)
      if (t + gridDim.x < n_tiles) fetch(t + gridDim.x, c);
      // rank of the CH values, step by step across all of them so that the dependent
      // shared-memory lookups of different values overlap.  A NaN walks the same code (bucket 0,
      // every comparison false) and is replaced by Q_NAN_CODE at the end; so does a categorical
      // value (its feature has empty tables), replaced by its category.
      uint32_t a[CH];  // address of the threshold below the current window
#pragma unroll
      for (int u = 0; u < CH; ++u) {
        // same expression as q_bucket_host: fma, clamp (NaN becomes 0), truncate
        T v = fma(cur[u], scale, offset);
        v   = fmax(v, T(0));
        v   = fmin(v, nbm1);
        a[u] = (lds_u16(lut + static_cast<uint32_t>(v) * lut_row) << eshift) + thr_m1;
      }
      if (STEPS > 0 && GFC > 0) {
        // group size and step count known: the probe offsets are immediates of the loads
        for_each_constant(
          [&](auto kc) {
            constexpr int k        = (STEPS > 0 ? STEPS : 1) - 1 - decltype(kc)::value;
            constexpr uint32_t S_B = (static_cast<uint32_t>(GFC > 0 ? GFC : 1) * TR::ES) << k;
            T thr[CH];
#pragma unroll
            for (int u = 0; u < CH; ++u) thr[u] = TR::template ld_real_at<S_B>(a[u]);
#pragma unroll
            for (int u = 0; u < CH; ++u) TR::add_if_le(a[u], thr[u], cur[u], S_B);
          },
          std::make_integer_sequence<int, (STEPS > 0 ? STEPS : 0)>{});
      } else if (STEPS >= 0) {
#pragma unroll
        for (int k = STEPS - 1; k >= 0; --k) {
          const uint32_t s_b = thr_row << k;
          T thr[CH];
#pragma unroll
          for (int u = 0; u < CH; ++u) thr[u] = TR::ld_real(a[u] + s_b);
#pragma unroll
          for (int u = 0; u < CH; ++u) TR::add_if_le(a[u], thr[u], cur[u], s_b);
        }
      } else {  // very full buckets: the number of halvings is only known at run time
        for (int k = static_cast<int>(grp.steps) - 1; k >= 0; --k) {
          const uint32_t s_b = thr_row << k;
#pragma unroll
          for (int u = 0; u < CH; ++u) TR::add_if_le(a[u], TR::ld_real(a[u] + s_b), cur[u], s_b);
        }
      }
      uint32_t code[CH];
#pragma unroll
      for (int u = 0; u < CH; ++u) code[u] = (a[u] - thr_m1) >> eshift;
      if (any_cat) {
        // groups with categorical features only (the warp-wide barrier keeps this a real branch
        // instead of conversions and selects that every group would execute): the code of a
        // categorical value is the category itself (truncated value); negative and huge values
        // match no listed category
        __syncwarp();
#pragma unroll
        for (int u = 0; u < CH; ++u) {
          const bool in_range = (cur[u] >= T(0)) && (cur[u] < T(Q_NO_CATEGORY));
          if (mine.is_cat) code[u] = in_range ? static_cast<uint32_t>(cur[u]) : Q_NO_CATEGORY;
        }
      }
#pragma unroll
      for (int u = 0; u < CH; ++u) {
        const bool is_nan = cur[u] != cur[u];
        saw_nan |= is_nan;
        const uint32_t cd = is_nan ? Q_NAN_CODE : code[u];
        const int j       = c * CH + u;
        if (NU == 1) {
          packed[0] = cd;
        } else if (j & 1) {
          packed[j >> 1] |= cd << 16;
        } else {
          packed[j >> 1] = cd;
        }
      }
    }
    // Q[tile][feature][slot]: the thread's NU consecutive slots of its feature in one store
    if (active) {
      uint16_t* dst = Q + t * tile_elems + q_mine;
      if (NU == 8) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[NU > 2 ? 1 : 0],
                                                    packed[NU > 4 ? 2 : 0], packed[NU > 6 ? 3 : 0]);
      } else if (NU == 4) {
        *reinterpret_cast<uint2*>(dst) = make_uint2(packed[0], packed[NU > 2 ? 1 : 0]);
      } else if (NU == 2) {
        *reinterpret_cast<uint32_t*>(dst) = packed[0];
      } else {
        *dst = static_cast<uint16_t>(packed[0]);
      }
    }
    if (__any_sync(0xffffffffu, saw_nan) && (tid & 31) == 0) atomicOr(tile_flags + t, 1);
  }
}

template <typename T, int STEPS>
__device__ __forceinline__ void quantise_rows(const PredictParams& p, const QGroup& grp,
                                              uint16_t* __restrict__ Q,
                                              int32_t* __restrict__ tile_flags, int R,
                                              uint32_t blob_a, const QFeatRec* rec)
{
  const int GF         = static_cast<int>(grp.f_end - grp.f_begin);
  const int per_thread = (R * GF) / static_cast<int>(blockDim.x);
  // full-width groups on large tiles, the shape of big batches, get the group size baked in
  if (GF == 32 && STEPS >= 2 && per_thread == 8) {
    quantise_tiles<T, STEPS, 8, 32>(p, grp, Q, tile_flags, R, blob_a, rec);
    return;
  }
  switch (per_thread) {
    case 8: quantise_tiles<T, STEPS, 8, 0>(p, grp, Q, tile_flags, R, blob_a, rec); break;
    case 4: quantise_tiles<T, STEPS, 4, 0>(p, grp, Q, tile_flags, R, blob_a, rec); break;
    case 2: quantise_tiles<T, STEPS, 2, 0>(p, grp, Q, tile_flags, R, blob_a, rec); break;
    default: quantise_tiles<T, STEPS, 1, 0>(p, grp, Q, tile_flags, R, blob_a, rec); break;
  }
}

template <typename T>
__global__ void __launch_bounds__(1024, 1)
quantise_kernel(const PredictParams p, uint16_t* __restrict__ Q, int32_t* __restrict__ tile_flags,
                const int R)
{
  extern __shared__ __align__(128) unsigned char smem[];
  const ForestView& f   = p.f;
  const QGroup grp      = f.q_groups[blockIdx.y];
  const uint32_t bar    = smem_addr(smem);
  unsigned char* blob   = smem + 16;
  const uint32_t blob_a = smem_addr(blob);
  const QFeatRec* rec   = reinterpret_cast<const QFeatRec*>(blob);

  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
    mbar_expect_tx(bar, grp.blob_bytes);
    bulk_copy_g2s(blob_a, f.q_blob + grp.blob_off, grp.blob_bytes, bar);
  }
  __syncthreads();
  if (!mbar_wait(bar, 0)) {
    if (threadIdx.x == 0) atomicExch(p.status, 4);
    return;
  }
  // the number of halvings is fixed per group: pick the unrolled body once
  switch (grp.steps) {
    case 0: quantise_rows<T, 0>(p, grp, Q, tile_flags, R, blob_a, rec); break;
    case 1: quantise_rows<T, 1>(p, grp, Q, tile_flags, R, blob_a, rec); break;
    case 2: quantise_rows<T, 2>(p, grp, Q, tile_flags, R, blob_a, rec); break;
    case 3: quantise_rows<T, 3>(p, grp, Q, tile_flags, R, blob_a, rec); break;
    case 4: quantise_rows<T, 4>(p, grp, Q, tile_flags, R, blob_a, rec); break;
    case 5: quantise_rows<T, 5>(p, grp, Q, tile_flags, R, blob_a, rec); break;
    default: quantise_rows<T, -1>(p, grp, Q, tile_flags, R, blob_a, rec); break;
  }
}

// ---------------------------------------------------------------------------------------------
// SPARSE kernel
// ---------------------------------------------------------------------------------------------
template <int FMT>
struct SparseFmt;
template <>
struct SparseFmt<FMT_SPARSE_8> {
  using T = float;
  struct Node {
    uint32_t value, meta, offset;
  };
  static __device__ __forceinline__ Node load(const void* nodes, uint32_t i, int feat_bits)
  {
    const uint2 raw = __ldg(static_cast<const uint2*>(nodes) + i);
    Node n;
    n.value  = raw.x;
    n.meta   = raw.y;
    n.offset = (raw.y & META_LOW29) >> feat_bits;
    return n;
  }
  static __device__ __forceinline__ uint32_t feature(const Node& n, int feat_bits)
  {
    return n.meta & ((1u << feat_bits) - 1u);
  }
};
template <>
struct SparseFmt<FMT_SPARSE_16F> {
  using T = float;
  struct Node {
    uint32_t value, meta, offset;
  };
  static __device__ __forceinline__ Node load(const void* nodes, uint32_t i, int)
  {
    const uint4 raw = __ldg(static_cast<const uint4*>(nodes) + i);
    return Node{raw.x, raw.y, raw.z};
  }
  static __device__ __forceinline__ uint32_t feature(const Node& n, int)
  {
    return n.meta & META_LOW29;
  }
};
template <>
struct SparseFmt<FMT_SPARSE_16D> {
  using T = double;
  struct Node {
    uint64_t value;
    uint32_t meta, offset;
  };
  static __device__ __forceinline__ Node load(const void* nodes, uint32_t i, int)
  {
    const uint4 raw = __ldg(static_cast<const uint4*>(nodes) + i);
    return Node{static_cast<uint64_t>(raw.x) | (static_cast<uint64_t>(raw.y) << 32), raw.z, raw.w};
  }
  static __device__ __forceinline__ uint32_t feature(const Node& n, int)
  {
    return n.meta & META_LOW29;
  }
};

// Shared memory: [row tile (when rows_in_smem)][accumulators].
template <int FMT, int MODE, int NT>
__global__ void __launch_bounds__(1024, 1)
sparse_kernel(const PredictParams p, const int R, const int G, const int rows_in_smem)
{
  using SF = SparseFmt<FMT>;
  using T  = typename SF::T;
  using TR = Traits<T>;
  extern __shared__ __align__(128) unsigned char smem[];
  const ForestView& f = p.f;
  const int F         = f.n_features;
  const int NC        = f.n_outputs;
  const int rw        = R >> 5;
  const int n_warps   = rw * G;
  const int warp      = threadIdx.x >> 5;
  const int lane      = threadIdx.x & 31;
  const int g         = warp / rw;
  const int r         = (warp % rw) * 32 + lane;
  const bool dfs      = f.layout == B2FIL_LAYOUT_DEPTH_FIRST;
  const int fb        = f.feat_bits;

  const uint32_t stride_b = (R + 1) * TR::ES;
  const size_t tile_bytes = rows_in_smem ? align16(static_cast<size_t>(F) * stride_b) : 0;
  T* acc                  = reinterpret_cast<T*>(smem + tile_bytes);
  T* acc_group            = acc + static_cast<size_t>(g) * NC * R;
  const uint32_t tile     = smem_addr(smem);
  const uint32_t row_addr = tile + r * TR::ES;
  const int64_t n_tiles   = (p.n_rows + R - 1) / R;
  const int per_batch     = G * NT;
  const T* X              = static_cast<const T*>(p.X);

  for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const int64_t row0 = t * R;
    const int64_t row  = row0 + r;
    if (rows_in_smem) stage_rows<T>(p, tile, R, row0, warp, lane, n_warps);
    if (MODE <= MODE_VECTOR) {
      for (int i = threadIdx.x; i < G * NC * R; i += n_warps * 32) acc[i] = T(0);
    }
    __syncthreads();
    // rows past the end of the batch read row 0 of the tile's global memory when not staged
    const T* xrow = X + (row < p.n_rows ? row : row0) * p.row_stride;
    Running<T> run{T(0), 0, {}};
    for (int first = g * NT; first < f.n_trees; first += per_batch) {
      const int n_act = min(NT, f.n_trees - first);
      uint32_t idx[NT];
      typename SF::Node node[NT];
#pragma unroll
      for (int k = 0; k < NT; ++k) idx[k] = __ldg(f.roots + first + min(k, n_act - 1));
      // max_depth + 1 nodes lie on the longest path: the loop cannot run away on a bad forest.
      // Every step first issues the node fetches of all NT walks (a walk that has reached its
      // leaf fetches the leaf again, a cache hit), then advances them without branches, so a
      // thread really has NT independent fetches in flight; the warp leaves the loop together.
      for (int step = 0; step <= f.max_depth; ++step) {
#pragma unroll
        for (int k = 0; k < NT; ++k) node[k] = SF::load(f.nodes, idx[k], fb);
        bool walking = false;
#pragma unroll
        for (int k = 0; k < NT; ++k) {
          const bool leaf     = (node[k].meta & META_LEAF) != 0;
          const uint32_t feat = leaf ? 0u : SF::feature(node[k], fb);
          const T x = rows_in_smem ? TR::ld_real(feat * stride_b + row_addr) : __ldg(xrow + feat);
          typename TR::Val v  = node[k].value;
          const bool right    = f.has_categorical
                                  ? goes_right<T, true, true>(v, node[k].meta, x, f)
                                  : goes_right<T, false, true>(v, node[k].meta, x, f);
          // depth-first: left child follows its parent, `offset` reaches the right child;
          // otherwise the children are adjacent and `offset` reaches the left one
          const uint32_t hop =
            dfs ? (right ? node[k].offset : 1u) : (node[k].offset + (right ? 1u : 0u));
          idx[k] += leaf ? 0u : hop;
          walking |= !leaf;
        }
        if (!__any_sync(0xffffffffu, walking)) break;
      }
#pragma unroll
      for (int k = 0; k < NT; ++k) {
        if (k < n_act && (node[k].meta & META_LEAF) != 0) {
          take_leaf<T, MODE>(p, first + k, node[k].value, idx[k], acc_group, R, r, row, run);
        }
      }
    }
    flush_running<T, MODE>(f, run, acc_group, R, r);
    __syncthreads();
    if (MODE <= MODE_VECTOR) {
      if (threadIdx.x < R) finish_row<T>(p, acc, R, G, threadIdx.x, row0 + threadIdx.x);
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// host side: launch shapes and dispatch
// ---------------------------------------------------------------------------------------------
size_t dense_tree_stride(int depth, int precision)
{
  const size_t nb = precision == B2FIL_F32 ? 8 : 16;
  const size_t lb = precision == B2FIL_F32 ? 4 : 8;
  return align16((size_t(1) << depth) * (nb + lb));
}

size_t dense_smem(int depth, int precision, int F, int NC, bool reduce, int R, int G, int NT, int S)
{
  const size_t es = precision == B2FIL_F32 ? 4 : 8;
  size_t b        = kBarBytes;
  b += align16(static_cast<size_t>(F) * (R + 1) * es);
  if (reduce) b += align16(static_cast<size_t>(G) * NC * R * es);
  b += 16;
  b += static_cast<size_t>(S) * G * NT * dense_tree_stride(depth, precision);
  return b;
}

// Raise a kernel's dynamic shared-memory limit to `bytes`.  The limit is a per-device attribute
// of the kernel: it is set once per (device, kernel) and only raised afterwards, so the steady
// state of a serving loop pays a table lookup instead of a driver call.
template <typename K>
int set_smem(K kernel, size_t bytes, std::string& err)
{
  return set_smem_bytes(reinterpret_cast<const void*>(kernel), bytes, err);
}

template <typename T, bool CAT, int MODE>
int launch_dense_mode(const PredictParams& p, const DenseCfg& c, dim3 grid, int n_splits,
                      void* partial, cudaStream_t stream, std::string& err)
{
  int rc;
  T* part = static_cast<T*>(partial);
  if (c.trees_in_flight == 2) {
    auto k = dense_kernel<T, CAT, MODE, 2>;
    if ((rc = set_smem(k, c.smem_bytes, err)) != B2FIL_OK) return rc;
    k<<<grid, c.threads, c.smem_bytes, stream>>>(p, c.rows_per_tile, c.tree_groups, c.stages,
                                                 n_splits, part);
  } else {
    auto k = dense_kernel<T, CAT, MODE, 1>;
    if ((rc = set_smem(k, c.smem_bytes, err)) != B2FIL_OK) return rc;
    k<<<grid, c.threads, c.smem_bytes, stream>>>(p, c.rows_per_tile, c.tree_groups, c.stages,
                                                 n_splits, part);
  }
  if (n_splits > 1 && MODE <= MODE_VECTOR) {
    launch_finish_rows(p, part, n_splits, sizeof(T) == 8, stream);
  }
  return B2FIL_OK;
}

template <typename T, bool CAT>
int launch_dense_cat(const PredictParams& p, int mode, const DenseCfg& c, dim3 grid, int n_splits,
                     void* partial, cudaStream_t stream, std::string& err)
{
  switch (mode) {
    case MODE_SCALAR:
      return launch_dense_mode<T, CAT, MODE_SCALAR>(p, c, grid, n_splits, partial, stream, err);
    case MODE_VECTOR:
      return launch_dense_mode<T, CAT, MODE_VECTOR>(p, c, grid, n_splits, partial, stream, err);
    case MODE_PERTREE:
      return launch_dense_mode<T, CAT, MODE_PERTREE>(p, c, grid, n_splits, partial, stream, err);
    default:
      return launch_dense_mode<T, CAT, MODE_LEAFID>(p, c, grid, n_splits, partial, stream, err);
  }
}

template <int FMT>
int launch_sparse_fmt(const PredictParams& p, int mode, int R, int G, int rows_in_smem, int grid,
                      size_t smem, cudaStream_t stream, std::string& err)
{
  constexpr int NT = 4;
  const int threads = (R / 32) * G * 32;
  int rc;
#define B2FIL_SPARSE_CASE(M)                                                       \
  {                                                                                \
    auto k = sparse_kernel<FMT, M, NT>;                                            \
    if ((rc = set_smem(k, smem, err)) != B2FIL_OK) return rc;                      \
    k<<<grid, threads, smem, stream>>>(p, R, G, rows_in_smem);                     \
  }
  switch (mode) {
    case MODE_SCALAR: B2FIL_SPARSE_CASE(MODE_SCALAR) break;
    case MODE_VECTOR: B2FIL_SPARSE_CASE(MODE_VECTOR) break;
    case MODE_PERTREE: B2FIL_SPARSE_CASE(MODE_PERTREE) break;
    default: B2FIL_SPARSE_CASE(MODE_LEAFID) break;
  }
#undef B2FIL_SPARSE_CASE
  return B2FIL_OK;
}

size_t dense_q_smem(size_t qstride, int precision, int F, int NC, bool reduce, int R, int G, int NT,
                    int S, int K)
{
  const size_t es = precision == B2FIL_F32 ? 4 : 8;
  size_t b        = kBarBytes;
  b += static_cast<size_t>(F) * R * 2;
  if (reduce) b += align16(static_cast<size_t>(G) * NC * R * es);
  b += 16;
  b += static_cast<size_t>(S) * G * NT * K * qstride;
  return b;
}

// Bytes of a tree's test nodes when kernels exist that keep only those in the stages
// (dense_q_leafg_kernel: fp32 scalar leaves, no categorical tests, depth 9 or 10), else 0.
size_t q_node_only_stride(const ForestView& f, int mode)
{
  const bool ok = f.format == FMT_DENSE_F && mode == MODE_SCALAR && !f.q_has_cat &&
                  (f.dense_depth == 9 || f.dense_depth == 10);
  return ok ? (size_t(4) << f.dense_depth) : 0;
}

// Most trees a warp of the quantised kernel may walk side by side: the kernels that exist.
int q_max_trees_in_flight(const ForestView& f, int mode)
{
  if (f.q_has_cat) return 4;
  const bool specialised = f.format == FMT_DENSE_F && (mode == MODE_SCALAR || mode == MODE_VECTOR) &&
                           f.dense_depth >= 4 && f.dense_depth <= 10;
  return specialised ? 6 : 4;
}

// Launch shape of the quantised dense kernel: the largest row tile that fits, then as many warps
// as fit (31 consumer warps at most), then as many trees in flight per warp as there is a kernel
// for, then the deepest tree ring that still fits.
// `node_stride` > 0 says that kernels exist which keep only a tree's test nodes (that many bytes)
// in the stages and fetch leaf payloads from global memory; the shape with them is taken when it
// puts at least a third more walks in flight.
bool dense_q_config(size_t qstride, int max_nt, int precision, int F, int NC, bool reduce,
                    int64_t n_rows, int chunk_size, int sm_count, DenseCfg& cfg,
                    int depth_hint = 0, size_t node_stride = 0)
{
  int want = 256;
  if (chunk_size > 0) {
    want = std::min(256, std::max(32, 32 * chunk_size));
  } else {
    while (want > 32 && n_rows < static_cast<int64_t>(want) * sm_count) want /= 2;
  }
  // tuning aid "R,G,NT,S,K": from the environment (read once per process) or, taking
  // precedence, from the knobs q_R, q_G, q_NT, q_S, q_K of b2fil_set_tuning
  static const struct ForcedShape {
    bool set = false;
    int R = 0, G = 0, NT = 0, S = 0, K = 0;
    ForcedShape()
    {
      const char* e = getenv("B2FIL_Q_SHAPE");
      set = e && sscanf(e, "%d,%d,%d,%d,%d", &R, &G, &NT, &S, &K) == 5;
    }
  } from_env;
  ForcedShape forced = from_env;
  if (const int R = tuning_value("q_R", 0); R > 0) {
    forced.set = true;
    forced.R   = R;
    forced.G   = tuning_value("q_G", 1);
    forced.NT  = tuning_value("q_NT", 1);
    forced.S   = tuning_value("q_S", 2);
    forced.K   = tuning_value("q_K", 1);
  }
  if (forced.set) {
    const int R = forced.R, G = forced.G, NT = forced.NT, S = forced.S, K = forced.K;
    if (R >= 32 && R % 32 == 0 &&
        R <= 256 && (R & (R - 1)) == 0 && G >= 1 && (R / 32) * G <= 31 &&
        (NT == 1 || NT == 2 || NT == 4 || (NT == 6 && (R / 32) * G <= 24) ||
         (NT == 3 && max_nt == 6 && depth_hint >= 9)) && S >= 2 &&
        S <= kMaxStages && K >= 1 && NT <= max_nt) {
      const bool leafg = node_stride > 0 && tuning_value("q_leafg", 0) == 1 && NT >= 2 && NT <= 4;
      const size_t b = dense_q_smem(leafg ? node_stride : qstride, precision, F, NC, reduce, R, G, NT, S, K);
      if (b <= kMaxSmemBytes) {
        cfg = DenseCfg{R, G, NT, S, b, ((R / 32) * G + 1) * 32, K, leafg ? 1 : 0};
        return true;
      }
    }
  }
  const int leafg_knob = tuning_value("q_leafg", -1);  // -1 automatic, 0 never, 1 whenever possible
  for (int R = want; R >= 32; R /= 2) {
    const int rw = R / 32;
    // Among the (tree groups, trees in flight) pairs that fit with a two-stage ring, take the one
    // with the most walks in flight per CTA (row warps x groups x trees): that is what hides the
    // latency of a step, and shapes that shared memory keeps small are bound by exactly it
    // (measured on 2000 depth-10 trees over 512 features, where only 12 trees fit: 3 groups x 2
    // trees 7.2e7 rows/s, 5 groups x 1 tree 6.3e7).  Ties go to more warps.
    int best_g = 0, best_nt = 0;
    // a CTA holds at most 32 warps and one of them is the producer
    for (int G = std::min(8, 31 / rw); G >= 1; --G) {
      for (int NT = max_nt; NT >= 1; NT = NT == 6 ? 4 : NT / 2) {
        // the six-tree kernels are built for at most 24 consumer warps (80 registers a thread)
        if (NT > 4 && rw * G > 24) continue;
        if (dense_q_smem(qstride, precision, F, NC, reduce, R, G, NT, 2, 1) > kMaxSmemBytes) continue;
        if (G * NT > best_g * best_nt) {
          best_g  = G;
          best_nt = NT;
        }
        break;  // smaller NT with the same G only has fewer walks
      }
    }
    size_t stride = qstride;
    int leafg     = 0;
    if (node_stride > 0 && leafg_knob != 0) {
      // the same search with node-only trees (kernels for two to four trees in flight)
      int lg = 0, lnt = 0;
      for (int G = std::min(8, 31 / rw); G >= 1; --G) {
        for (int NT = 4; NT >= 2; --NT) {
          if (dense_q_smem(node_stride, precision, F, NC, reduce, R, G, NT, 2, 1) > kMaxSmemBytes) continue;
          if (G * NT > lg * lnt) {
            lg  = G;
            lnt = NT;
          }
          break;
        }
      }
      if (lg > 0 && (leafg_knob == 1 || lg * lnt * 3 >= best_g * best_nt * 4)) {
        best_g  = lg;
        best_nt = lnt;
        stride  = node_stride;
        leafg   = 1;
      }
    }
    if (best_g == 0) continue;
    // a stage holds K sub-batches so that a warp waits and signals once per K * NT trees.
    // Two stages already hide the bulk copies (measured: S = 2 and S = 3 run alike).
    for (int K = 2; K >= 1; K /= 2) {
      for (int S = 3; S >= 2; --S) {
        const size_t b = dense_q_smem(stride, precision, F, NC, reduce, R, best_g, best_nt, S, K);
        if (b <= kMaxSmemBytes) {
          cfg = DenseCfg{R, best_g, best_nt, S, b, (rw * best_g + 1) * 32, K, leafg};
          return true;
        }
      }
    }
  }
  return false;
}

// Launch shapes with at most this many walks in flight per CTA take the child-pair walk.
constexpr int kPairWalkLimit = 0;  // 0: never automatically (set from measurements)

// Pick the kernel family for a launch of the quantised traversal; the families are instantiated
// in the kernels_q_*.cu translation units.
int launch_dense_q_kernel(const QLaunch& L, int mode, bool f64, std::string& err)
{
  const ForestView& f = L.p.f;
  LaunchRecord& rec   = g_last_launch;
  rec                 = LaunchRecord{};
  rec.prepass         = "quantise_kernel";
  rec.kernel          = "dense_q_kernel";
  rec.real            = f64 ? "double" : "float";
  rec.mode            = mode;
  rec.nt              = L.c.trees_in_flight;
  rec.depth           = 0;  // read at run time unless a specialised body is picked below
  rec.cat             = f.q_has_cat ? 1 : 0;
  rec.R               = L.c.rows_per_tile;
  rec.G               = L.c.tree_groups;
  rec.S               = L.c.stages;
  rec.K               = L.c.sub_batches;
  if (f.q_has_cat) {
    // kernels_q_cat.cu: fp32 scalar leaves of depth 4..8 with four trees in flight are specialised
    if (!f64 && mode == MODE_SCALAR && L.c.trees_in_flight == 4 && f.dense_depth >= 4 &&
        f.dense_depth <= 8)
      rec.depth = f.dense_depth;
    return launch_q_cat(L, mode, f64, err);
  }
  // Few walks in flight (shapes that shared memory keeps small): the latency of a step is the
  // limit, and the walk that fetches both children ahead of the test halves it.
  const int walks  = (L.c.rows_per_tile / 32) * L.c.tree_groups * L.c.trees_in_flight;
  const int pair   = tuning_value("q_pair", -1);
  const bool can_pair = !f64 && mode == MODE_SCALAR && L.c.trees_in_flight <= 4 && f.dense_depth >= 1;
  if (can_pair && (pair == 1 || (pair < 0 && walks <= kPairWalkLimit))) {
    rec.kernel = "dense_q_pair_kernel";
    return launch_q_pair(L, err);
  }
  if (L.c.leaves_global) {
    rec.kernel = "dense_q_leafg_kernel";
    rec.depth  = f.dense_depth;
    return launch_q_leafg(L, err);
  }
  if (!f64 && mode == MODE_VECTOR && f.dense_depth >= 4 && f.dense_depth <= 10 &&
      (L.c.trees_in_flight == 6 || L.c.trees_in_flight == 4)) {
    rec.depth = f.dense_depth;
    return launch_q_vec(L, err);
  }
  const bool specialised = !f64 && mode == MODE_SCALAR && f.dense_depth >= 4 && f.dense_depth <= 10;
  if (specialised && L.c.trees_in_flight == 6) {
    // the common boosted-tree shapes: depth-specialised bodies with six trees in flight
    // (q_max_trees_in_flight offers six only for them)
    rec.depth = f.dense_depth;
    if (L.p.q_top != nullptr && f.n_trees <= kQTopTrees) {
      rec.kernel = "dense_q_top_kernel";
      return launch_q_top6(L, err);
    }
    return launch_q_plain6(L, err);
  }
  if (specialised && L.c.trees_in_flight == 4) {
    rec.depth = f.dense_depth;
    return launch_q_plain4(L, err);
  }
  if (specialised && f.dense_depth >= 9 && (L.c.trees_in_flight == 2 || L.c.trees_in_flight == 3)) {
    rec.depth = f.dense_depth;
    return launch_q_plain23(L, err);
  }
  return launch_q_generic(L, mode, f64, err);
}

// CTAs per feature group of the rank pre-pass.  Every CTA holds the tables of one group, so the
// grid is (CTAs per group) x (groups) and the SMs take it in waves of one CTA each.  With g
// groups on s SMs, s / g CTAs per group fill one wave but leave s mod g SMs idle (64 groups on
// 148 SMs: 20 idle); more, shorter CTAs per group waste less: the count that minimises
// waves / (CTAs per group) is taken, among up to 48 or one wave's worth (a CTA loads its group's
// tables once, about 200 KB from L2).
int quantise_ctas_per_group(int n_groups, int sm_count, int64_t n_tiles)
{
  int best = 1;
  double best_cost = 1e30;
  const int most = std::max(48, sm_count / std::max(1, n_groups));
  for (int gx = 1; gx <= most; ++gx) {
    const int waves   = (gx * n_groups + sm_count - 1) / sm_count;
    const double cost = static_cast<double>(waves) / gx;
    if (cost < best_cost * 0.99) {  // ties and near ties: fewer CTAs
      best_cost = cost;
      best      = gx;
    }
  }
  return static_cast<int>(std::min<int64_t>(n_tiles, best));
}

// Rank-quantised prediction: rows are processed in chunks of whole waves of tiles; for each
// chunk the pre-pass writes the ranks into stream-ordered scratch and the traversal kernel reads
// them back.
int launch_dense_q(const PredictParams& p, int mode, int chunk_size, int sm_count,
                   cudaStream_t stream, cudaMemPool_t pool, std::string& err, int64_t* launches)
{
  const ForestView& f = p.f;
  const int precision = f.format == FMT_DENSE_F ? B2FIL_F32 : B2FIL_F64;
  const bool reduce   = mode <= MODE_VECTOR;
  DenseCfg c;
  if (!dense_q_config(static_cast<size_t>(f.q_tree_stride), q_max_trees_in_flight(f, mode), precision,
                      f.n_features, f.n_outputs, reduce, p.n_rows, chunk_size, sm_count, c,
                      f.dense_depth, q_node_only_stride(f, mode))) {
    err = "no quantised launch shape fits shared memory";
    return B2FIL_ERR_UNSUPPORTED;
  }
  const int R            = c.rows_per_tile;
  const size_t es        = precision == B2FIL_F32 ? 4 : 8;
  const size_t tile_b    = static_cast<size_t>(f.n_features) * R * 2;
  const int64_t wave     = static_cast<int64_t>(R) * sm_count;
  // measured on the 1000-tree depth-8 forest: 64 MB chunks (rank image resident in L2) 2.51e8
  // rows/s, 512 MB chunks 2.62e8: fewer, longer launches beat L2 residency because HBM has
  // plenty of headroom on this path
  // (B2FIL_Q_CHUNK_MB, a tuning aid, overrides the size; the environment is read once)
  static const size_t target = [] {
    size_t t = size_t(512) << 20;
    if (const char* e = getenv("B2FIL_Q_CHUNK_MB")) {
      const long mb = atol(e);
      if (mb >= 1 && mb <= 16384) t = static_cast<size_t>(mb) << 20;
    }
    return t;
  }();
  const int64_t waves    = std::max<int64_t>(1, static_cast<int64_t>(target / (tile_b * sm_count)));
  const int64_t chunk    = std::min<int64_t>(wave * waves, (p.n_rows + R - 1) / R * R);
  const int64_t ch_tiles = (chunk + R - 1) / R;
  const size_t q_bytes   = static_cast<size_t>(ch_tiles) * tile_b;
  const size_t fl_bytes  = (static_cast<size_t>(ch_tiles) * 4 + 255) / 256 * 256;
  unsigned char* scratch = nullptr;
  cudaError_t e = cudaMallocFromPoolAsync(reinterpret_cast<void**>(&scratch), q_bytes + fl_bytes,
                                          pool, stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    err = std::string("scratch allocation for quantised rows failed: ") + cudaGetErrorString(e);
    return e == cudaErrorMemoryAllocation ? B2FIL_ERR_NO_MEMORY : B2FIL_ERR_CUDA;
  }
  uint16_t* Q    = reinterpret_cast<uint16_t*>(scratch);
  int32_t* flags = reinterpret_cast<int32_t*>(scratch + q_bytes);
  // shared memory of the pre-pass: mbarrier and the largest group blob
  const size_t q_smem = 16 + static_cast<size_t>(f.q_max_blob_bytes);
  int rc = B2FIL_OK;
  const size_t out_row_b =
    (p.kind == B2FIL_INFER_LEAF_ID ? size_t(4) * f.n_trees
     : p.kind == B2FIL_INFER_CLASS ? size_t(4)
     : p.kind == B2FIL_INFER_PROBA2 ? 2 * es
     : p.kind == B2FIL_INFER_PER_TREE
       ? es * f.n_trees * (f.leaf_vector_len > 1 ? f.n_outputs : 1)
       : es * f.n_outputs);
  for (int64_t r0 = 0; r0 < p.n_rows && rc == B2FIL_OK; r0 += chunk) {
    PredictParams pc = p;
    pc.n_rows        = std::min<int64_t>(chunk, p.n_rows - r0);
    pc.X             = static_cast<const unsigned char*>(p.X) + static_cast<size_t>(r0) * p.row_stride * es;
    pc.out           = static_cast<unsigned char*>(p.out) + static_cast<size_t>(r0) * out_row_b;
    const int64_t n_tiles = (pc.n_rows + R - 1) / R;
    e = cudaMemsetAsync(flags, 0, static_cast<size_t>(n_tiles) * 4, stream);
    if (e != cudaSuccess) {
      err = std::string("cudaMemsetAsync: ") + cudaGetErrorString(e);
      rc  = B2FIL_ERR_CUDA;
      break;
    }
    const int gx = quantise_ctas_per_group(f.q_n_groups, sm_count, n_tiles);
    const dim3 qgrid(gx, f.q_n_groups);
    const dim3 qblock(1024);
    if (precision == B2FIL_F32) {
      auto k = quantise_kernel<float>;
      if ((rc = set_smem(k, q_smem, err)) != B2FIL_OK) break;
      k<<<qgrid, qblock, q_smem, stream>>>(pc, Q, flags, R);
    } else {
      auto k = quantise_kernel<double>;
      if ((rc = set_smem(k, q_smem, err)) != B2FIL_OK) break;
      k<<<qgrid, qblock, q_smem, stream>>>(pc, Q, flags, R);
    }
    const int grid = static_cast<int>(std::min<int64_t>(n_tiles, sm_count));
    rc = launch_dense_q_kernel(QLaunch{pc, Q, flags, c, grid, stream}, mode,
                               precision != B2FIL_F32, err);
    if (launches) *launches += 2;
  }
  cudaFreeAsync(scratch, stream);
  return rc;
}

// ---------------------------------------------------------------------------------------------
// prediction on rank-quantised rows with a fixed, preallocated scratch array
// ---------------------------------------------------------------------------------------------
// The rank image of a batch normally lives in stream-ordered scratch taken from a memory pool.
// This array replaces it for callers that must not allocate while they predict.  It is part of
// the library image: every GPU that loads the library holds it until the process exits.
constexpr size_t kFixedScratchBytes = B2FIL_FIXED_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_fixed_scratch[kFixedScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_fixed_mu;
void* g_fixed_ptr[kMaxDevices] = {};

// Device address of g_fixed_scratch on the current device (`device` is its ordinal).  In host
// code the array's name is only a handle for the runtime, not an address a kernel can use, so the
// address is asked for once per device and cached.
int fixed_scratch_address(int device, void** out, std::string& err)
{
  if (device < 0 || device >= kMaxDevices) {
    err = "device ordinal beyond the fixed-scratch table";
    return B2FIL_ERR_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_fixed_mu);
  if (!g_fixed_ptr[device]) {
    void* ptr           = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_fixed_scratch);
    if (e != cudaSuccess || !ptr) {
      err = std::string("cudaGetSymbolAddress(fixed scratch): ") + cudaGetErrorString(e);
      return B2FIL_ERR_CUDA;
    }
    g_fixed_ptr[device] = ptr;
  }
  *out = g_fixed_ptr[device];
  return B2FIL_OK;
}

int pick_rows_per_tile(int64_t n_rows, int chunk_size, int sm_count)
{
  if (chunk_size > 0) return std::min(128, std::max(32, 32 * chunk_size));
  // keep every SM busy before growing the tile
  if (n_rows >= static_cast<int64_t>(128) * sm_count) return 128;
  if (n_rows >= static_cast<int64_t>(64) * sm_count) return 64;
  return 32;
}

std::mutex g_smem_mu;
std::map<std::pair<int, const void*>, size_t> g_smem_set;
std::mutex g_tuning_mu;
std::map<std::string, int> g_tuning;
}  // namespace

namespace {
template <typename T>
void finish_rows(const PredictParams& p, T* part, int n_splits, cudaStream_t stream)
{
  if (n_splits > 4) {
    const int blocks = static_cast<int>((p.n_rows + 7) / 8);  // a warp per row
    finish_kernel<T><<<blocks, 256, 0, stream>>>(p, part, n_splits);
  } else {
    const int blocks = static_cast<int>((p.n_rows + 255) / 256);
    finish_few_splits_kernel<T><<<blocks, 256, 0, stream>>>(p, part, n_splits);
  }
}
}  // namespace

void launch_finish_rows(const PredictParams& p, void* partial, int n_splits, bool f64,
                        cudaStream_t stream)
{
  if (f64) {
    finish_rows<double>(p, static_cast<double*>(partial), n_splits, stream);
  } else {
    finish_rows<float>(p, static_cast<float*>(partial), n_splits, stream);
  }
}

int tuning_value(const char* key, int fallback)
{
  std::lock_guard<std::mutex> lock(g_tuning_mu);
  if (g_tuning.empty()) return fallback;
  const auto it = g_tuning.find(key);
  return it == g_tuning.end() ? fallback : it->second;
}
void set_tuning_value(const char* key, int value)
{
  std::lock_guard<std::mutex> lock(g_tuning_mu);
  g_tuning[key] = value;
}

int set_smem_bytes(const void* kernel, size_t bytes, std::string& err)
{
  int device = 0;
  cudaGetDevice(&device);
  const auto key = std::make_pair(device, kernel);
  {
    std::lock_guard<std::mutex> lock(g_smem_mu);
    const auto it = g_smem_set.find(key);
    if (it != g_smem_set.end() && it->second >= bytes) return B2FIL_OK;
  }
  const cudaError_t e = cudaFuncSetAttribute(
    kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
  if (e != cudaSuccess) {
    err = std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e);
    return B2FIL_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_smem_mu);
  size_t& have = g_smem_set[key];
  have         = std::max(have, bytes);
  return B2FIL_OK;
}

bool dense_config(int depth, int precision, int n_features, int n_outputs, bool reduce_kind,
                  int64_t n_rows, int chunk_size, int sm_count, DenseCfg& cfg)
{
  int want = pick_rows_per_tile(n_rows, chunk_size, sm_count);
  // small batches get their parallelism from splitting the forest across CTAs, not from many
  // small row tiles: every tile has to stream the trees it walks, so fewer, larger tiles win
  if (chunk_size <= 0 && n_rows <= static_cast<int64_t>(64) * sm_count)
    want = n_rows <= 32 ? 32 : (n_rows <= 64 ? 64 : 128);
  for (int R = want; R >= 32; R /= 2) {
    const int rw = R / 32;
    for (int G = 16 / rw; G >= 1; G /= 2) {
      for (int NT = 2; NT >= 1; --NT) {
        for (int S = 3; S >= 2; --S) {
          const size_t b =
            dense_smem(depth, precision, n_features, n_outputs, reduce_kind, R, G, NT, S);
          if (b <= kMaxSmemBytes) {
            cfg = DenseCfg{R, G, NT, S, b, (rw * G + 1) * 32, 1, 0};
            return true;
          }
        }
      }
    }
  }
  return false;
}

int dense_ok(int depth, int precision, int n_features, int n_outputs)
{
  // usable when at least 64 rows and two tree groups fit next to a two-stage ring
  if (dense_smem(depth, precision, n_features, n_outputs, true, 64, 2, 1, 2) <= kMaxSmemBytes) return 1;
  // else the traversal over rank-quantised rows alone, if a 32-row tile of ranks and two stages
  // of one tree fit (a tree counted at its largest: 8-byte test nodes, four inline outputs)
  const size_t es      = precision == B2FIL_F32 ? 4 : 8;
  const size_t qstride = (size_t(8) + 4 * es) << depth;
  if (dense_q_smem(qstride, precision, n_features, n_outputs, true, 32, 1, 1, 2, 1) <= kMaxSmemBytes &&
      n_features < (1 << 14))
    return 2;
  return 0;
}

int launch_predict(const PredictParams& p, int chunk_size, int sm_count, cudaStream_t stream,
                   cudaMemPool_t pool, std::string& err, int64_t* launches)
{
  const ForestView& f = p.f;
  if (p.n_rows == 0) return B2FIL_OK;
  int mode;
  switch (p.kind) {
    case B2FIL_INFER_DEFAULT:
    case B2FIL_INFER_CLASS: mode = f.leaf_vector_len > 1 ? MODE_VECTOR : MODE_SCALAR; break;
    case B2FIL_INFER_PROBA2:
      if (f.n_outputs != 1) {
        err = "B2FIL_INFER_PROBA2 needs a forest with one output";
        return B2FIL_ERR_INVALID_ARG;
      }
      mode = MODE_SCALAR;
      break;
    case B2FIL_INFER_PER_TREE: mode = MODE_PERTREE; break;
    case B2FIL_INFER_LEAF_ID: mode = MODE_LEAFID; break;
    default: err = "unknown infer_kind"; return B2FIL_ERR_INVALID_ARG;
  }
  const bool reduce = mode <= MODE_VECTOR;
  int rc            = B2FIL_OK;
  // the pre-pass indexes a row tile with 32-bit element offsets
  // (small batches skip the pre-pass: with fewer 128-row tiles than half the SMs the forest is
  // split across CTAs of the plain dense kernel instead, which is what bounds their latency)
  // (forests whose row tile only fits as ranks - a thousand features and more - have no other
  // dense kernel and take this path at every batch size)
  const bool dense_fmt = f.format == FMT_DENSE_F || f.format == FMT_DENSE_D;
  const bool ranks_only =
    dense_fmt && dense_ok(f.dense_depth, f.format == FMT_DENSE_F ? B2FIL_F32 : B2FIL_F64,
                          f.n_features, f.n_outputs) != 1;
  if (dense_fmt && f.q_enabled && p.row_stride < (int64_t(1) << 22) && pool != nullptr &&
      (chunk_size > 0 || ranks_only || (p.n_rows + 127) / 128 * 2 > sm_count)) {
    rc = launch_dense_q(p, mode, chunk_size, sm_count, stream, pool, err, launches);
    if (rc != B2FIL_OK) return rc;
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
      err = std::string("kernel launch: ") + cudaGetErrorString(e);
      return B2FIL_ERR_CUDA;
    }
    return B2FIL_OK;
  }
  if (f.format == FMT_DENSE_F || f.format == FMT_DENSE_D) {
    const int precision = f.format == FMT_DENSE_F ? B2FIL_F32 : B2FIL_F64;
    DenseCfg c;
    if (!dense_config(f.dense_depth, precision, f.n_features, f.n_outputs, reduce, p.n_rows,
                      chunk_size, sm_count, c)) {
      err = "no dense launch shape fits shared memory";
      return B2FIL_ERR_UNSUPPORTED;
    }
    const int64_t n_tiles = (p.n_rows + c.rows_per_tile - 1) / c.rows_per_tile;
    const int gx          = static_cast<int>(std::min<int64_t>(n_tiles, sm_count));
    // batches with fewer row tiles than SMs split the forest across CTAs (blockIdx.y): a CTA then
    // streams only its share of the trees; reduced outputs take a tiny second kernel
    const int per_batch = c.tree_groups * c.trees_in_flight;
    const int n_batches = (f.n_trees + per_batch - 1) / per_batch;
    int n_splits        = 1;
    if (n_tiles * 2 <= sm_count && (pool != nullptr || !reduce)) {  // no pool: never allocate
      // one wave of CTAs: tiles x splits fills the SMs once
      n_splits = static_cast<int>(std::min<int64_t>(n_batches, sm_count / n_tiles));
      n_splits = std::max(1, n_splits);
    }
    void* partial = nullptr;
    if (n_splits > 1 && reduce) {
      const size_t es    = precision == B2FIL_F32 ? 4 : 8;
      const size_t bytes = static_cast<size_t>(n_splits) * f.n_outputs * p.n_rows * es;
      const cudaError_t e = cudaMallocFromPoolAsync(&partial, bytes, pool, stream);
      if (e != cudaSuccess) {
        cudaGetLastError();
        err = std::string("scratch allocation for split prediction failed: ") + cudaGetErrorString(e);
        return e == cudaErrorMemoryAllocation ? B2FIL_ERR_NO_MEMORY : B2FIL_ERR_CUDA;
      }
    }
    const dim3 grid(gx, n_splits);
    {
      LaunchRecord& rec = g_last_launch;
      rec               = LaunchRecord{};
      rec.kernel        = "dense_kernel";
      rec.real          = precision == B2FIL_F32 ? "float" : "double";
      rec.mode          = mode;
      rec.nt            = c.trees_in_flight == 2 ? 2 : 1;
      rec.cat           = f.has_categorical ? 1 : 0;
      rec.R             = c.rows_per_tile;
      rec.G             = c.tree_groups;
      rec.S             = c.stages;
      rec.splits        = n_splits;
    }
    if (precision == B2FIL_F32) {
      rc = f.has_categorical
             ? launch_dense_cat<float, true>(p, mode, c, grid, n_splits, partial, stream, err)
             : launch_dense_cat<float, false>(p, mode, c, grid, n_splits, partial, stream, err);
    } else {
      rc = f.has_categorical
             ? launch_dense_cat<double, true>(p, mode, c, grid, n_splits, partial, stream, err)
             : launch_dense_cat<double, false>(p, mode, c, grid, n_splits, partial, stream, err);
    }
    if (partial) cudaFreeAsync(partial, stream);
    if (launches && n_splits > 1 && reduce) ++*launches;
  } else if (CompactCfg cc; compact_config(f, reduce, pick_rows_per_tile(p.n_rows, chunk_size, sm_count),
                                          p.n_rows, sm_count,
                                          chunk_size <= 0 && (pool != nullptr || !reduce), cc)) {
    // deep / ragged forests with a compact image: heaps of the top levels through shared memory,
    // 8-byte internal nodes below
    LaunchRecord& rec = g_last_launch;
    rec               = LaunchRecord{};
    rec.kernel        = "sparse_compact_kernel";
    rec.real          = f.format == FMT_SPARSE_16D ? "double" : "float";
    rec.mode          = mode;
    rec.nt            = kCompactTreesInFlight;
    rec.cat           = f.has_categorical ? 1 : 0;
    rec.top           = f.c_top_levels;
    rec.R             = cc.rows_per_tile;
    rec.G             = cc.tree_groups;
    rec.S             = cc.stages;
    rec.splits        = cc.splits;
    rc = launch_sparse_compact(p, mode, cc, stream, pool, err, launches);
  } else {
    const size_t es = f.format == FMT_SPARSE_16D ? 8 : 4;
    int R           = pick_rows_per_tile(p.n_rows, chunk_size, sm_count);
    int G           = std::min(8, 32 / (R / 32));
    G               = std::max(1, std::min(G, (f.n_trees + 3) / 4));
    // two CTAs per SM when the tile is small enough, else one; rows stay in global memory when
    // even a 32-row tile does not fit
    size_t acc_b = 0, tile_b = 0;
    int rows_in_smem = 1;
    for (;;) {
      acc_b  = reduce ? align16(static_cast<size_t>(G) * f.n_outputs * R * es) : 0;
      tile_b = align16(static_cast<size_t>(f.n_features) * (R + 1) * es);
      if (acc_b + tile_b <= kMaxSmemBytes) break;
      if (R > 32) {
        R /= 2;
        continue;
      }
      rows_in_smem = 0;
      tile_b       = 0;
      if (acc_b > kMaxSmemBytes) {
        if (G > 1) {
          G /= 2;
          continue;
        }
        err = "too many outputs for the accumulators to fit shared memory";
        return B2FIL_ERR_UNSUPPORTED;
      }
      break;
    }
    const size_t smem     = acc_b + tile_b;
    const int64_t n_tiles = (p.n_rows + R - 1) / R;
    const int grid        = static_cast<int>(std::min<int64_t>(n_tiles, int64_t(sm_count) * 8));
    {
      LaunchRecord& rec = g_last_launch;
      rec               = LaunchRecord{};
      rec.kernel        = "sparse_kernel";
      rec.real          = f.format == FMT_SPARSE_16D ? "double" : "float";
      rec.mode          = mode;
      rec.nt            = 4;
      rec.fmt           = f.format;
      rec.R             = R;
      rec.G             = G;
    }
    switch (f.format) {
      case FMT_SPARSE_8:
        rc = launch_sparse_fmt<FMT_SPARSE_8>(p, mode, R, G, rows_in_smem, grid, smem, stream, err);
        break;
      case FMT_SPARSE_16F:
        rc = launch_sparse_fmt<FMT_SPARSE_16F>(p, mode, R, G, rows_in_smem, grid, smem, stream, err);
        break;
      default:
        rc = launch_sparse_fmt<FMT_SPARSE_16D>(p, mode, R, G, rows_in_smem, grid, smem, stream, err);
        break;
    }
  }
  if (rc != B2FIL_OK) return rc;
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    err = std::string("kernel launch: ") + cudaGetErrorString(e);
    return B2FIL_ERR_CUDA;
  }
  if (launches) ++*launches;
  return B2FIL_OK;
}


int launch_predict_fixed_scratch(const PredictParams& p, int chunk_size, int sm_count, int device,
                                 cudaStream_t stream, std::string& err, int64_t* launches)
{
  const ForestView& f = p.f;
  if (p.n_rows == 0) return B2FIL_OK;
  const bool quantised = (f.format == FMT_DENSE_F || f.format == FMT_DENSE_D) && f.q_enabled &&
                         p.row_stride < (int64_t(1) << 22);
  // forests that predict without scratch take the ordinary path, which allocates nothing for them
  if (!quantised) return launch_predict(p, chunk_size, sm_count, stream, nullptr, err, launches);
  int mode;
  switch (p.kind) {
    case B2FIL_INFER_DEFAULT:
    case B2FIL_INFER_CLASS: mode = f.leaf_vector_len > 1 ? MODE_VECTOR : MODE_SCALAR; break;
    case B2FIL_INFER_PROBA2:
      if (f.n_outputs != 1) {
        err = "B2FIL_INFER_PROBA2 needs a forest with one output";
        return B2FIL_ERR_INVALID_ARG;
      }
      mode = MODE_SCALAR;
      break;
    case B2FIL_INFER_PER_TREE: mode = MODE_PERTREE; break;
    case B2FIL_INFER_LEAF_ID: mode = MODE_LEAFID; break;
    default: err = "unknown infer_kind"; return B2FIL_ERR_INVALID_ARG;
  }
  const int precision = f.format == FMT_DENSE_F ? B2FIL_F32 : B2FIL_F64;
  DenseCfg c;
  if (!dense_q_config(static_cast<size_t>(f.q_tree_stride), q_max_trees_in_flight(f, mode), precision,
                      f.n_features, f.n_outputs, mode <= MODE_VECTOR, p.n_rows, chunk_size,
                      sm_count, c, f.dense_depth, q_node_only_stride(f, mode))) {
    err = "no quantised launch shape fits shared memory";
    return B2FIL_ERR_UNSUPPORTED;
  }
  const int R           = c.rows_per_tile;
  const size_t tile_b   = static_cast<size_t>(f.n_features) * R * 2;
  const int64_t n_tiles = (p.n_rows + R - 1) / R;
  const size_t q_bytes  = static_cast<size_t>(n_tiles) * tile_b;
  const size_t fl_bytes = (static_cast<size_t>(n_tiles) * 4 + 255) / 256 * 256;
  if (q_bytes + fl_bytes > kFixedScratchBytes) {
    const size_t per_row = static_cast<size_t>(f.n_features) * 2 + 1;
    err = "batch too large for the fixed scratch array: " + std::to_string(p.n_rows) +
          " rows of " + std::to_string(f.n_features) + " features need " +
          std::to_string(q_bytes + fl_bytes) + " bytes, the array holds " +
          std::to_string(kFixedScratchBytes) + " (about " +
          std::to_string(kFixedScratchBytes / per_row / 256 * 256) + " rows per call)";
    return B2FIL_ERR_TOO_LARGE;
  }
  void* base = nullptr;
  int rc     = fixed_scratch_address(device, &base, err);
  if (rc != B2FIL_OK) return rc;
  uint16_t* Q    = reinterpret_cast<uint16_t*>(base);
  int32_t* flags = reinterpret_cast<int32_t*>(static_cast<unsigned char*>(base) + q_bytes);
  // the array keeps what the previous call left in it: the NaN flags of the tiles are
  // accumulated with atomicOr and must start at zero (the ranks themselves are fully rewritten)
  cudaError_t e = cudaMemsetAsync(flags, 0, static_cast<size_t>(n_tiles) * 4, stream);
  if (e != cudaSuccess) {
    err = std::string("cudaMemsetAsync: ") + cudaGetErrorString(e);
    return B2FIL_ERR_CUDA;
  }
  const size_t q_smem = 16 + static_cast<size_t>(f.q_max_blob_bytes);
  const int gx = quantise_ctas_per_group(f.q_n_groups, sm_count, n_tiles);
  const dim3 qgrid(gx, f.q_n_groups);
  const dim3 qblock(1024);
  if (precision == B2FIL_F32) {
    auto k = quantise_kernel<float>;
    if ((rc = set_smem(k, q_smem, err)) != B2FIL_OK) return rc;
    k<<<qgrid, qblock, q_smem, stream>>>(p, Q, flags, R);
  } else {
    auto k = quantise_kernel<double>;
    if ((rc = set_smem(k, q_smem, err)) != B2FIL_OK) return rc;
    k<<<qgrid, qblock, q_smem, stream>>>(p, Q, flags, R);
  }
  const int grid = static_cast<int>(std::min<int64_t>(n_tiles, sm_count));
  rc = launch_dense_q_kernel(QLaunch{p, Q, flags, c, grid, stream}, mode, precision != B2FIL_F32,
                             err);
  if (rc != B2FIL_OK) return rc;
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    err = std::string("kernel launch: ") + cudaGetErrorString(e);
    return B2FIL_ERR_CUDA;
  }
  if (launches) *launches += 2;
  return B2FIL_OK;
}

std::string last_launch_variant()
{
  const LaunchRecord& r = g_last_launch;
  if (!r.kernel) return std::string();
  std::string s;
  if (r.prepass) s += std::string(r.prepass) + "<" + r.real + "> + ";
  s += std::string(r.kernel) + "<" + r.real;
  if (r.fmt >= 0) {
    s += r.fmt == FMT_SPARSE_8 ? ",node8" : (r.fmt == FMT_SPARSE_16F ? ",node16f" : ",node16d");
  }
  s += std::string(",") + mode_name(r.mode) + ",NT=" + std::to_string(r.nt);
  if (r.depth >= 0) s += ",DEPTH=" + (r.depth ? std::to_string(r.depth) : std::string("runtime"));
  if (r.cat >= 0) s += r.cat ? ",CAT" : "";
  if (r.top >= 0) s += ",TOP=" + std::to_string(r.top);
  s += "> R=" + std::to_string(r.R) + " G=" + std::to_string(r.G);
  if (r.S) s += " S=" + std::to_string(r.S);
  if (r.K) s += " K=" + std::to_string(r.K);
  if (r.splits > 1) s += " forest_splits=" + std::to_string(r.splits) + " + finish_kernel";
  return s;
}

int launch_bounded_wait_selftest(int32_t* status, uint32_t tries, cudaStream_t stream,
                                 std::string& err)
{
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(status, tries);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    err = std::string("kernel launch: ") + cudaGetErrorString(e);
    return B2FIL_ERR_CUDA;
  }
  return B2FIL_OK;
}

}  // namespace b2fil
