// Kernel for sparse forests that carry the compact image (forest.hpp): deep, ragged trees whose
// prediction is a chain of dependent node fetches.
//
// A CTA owns a tile of R rows staged feature-major in shared memory, like the other kernels, and
// its warps form (R/32 row sets) x (G tree groups); a warp walks its 32 rows through NT trees at
// a time.  Every walk has two parts:
//   1. the top T levels of the tree are a complete heap that a producer warp streams through a
//      ring of shared-memory stages (bulk copies from the L2-resident heap array; one stage =
//      the heaps of G * NT trees): T steps without a global fetch, then one exit {k, L} that names
//      the internal node to continue at and the leaves before it, or the leaf reached;
//   2. below the heap the walk follows the compact nodes in global memory: 8-byte internal
//      nodes, first child adjacent, (k, L) bookkeeping for the leaf number, nodes fetched as
//      aligned 16-byte pairs so that a step from an even node to its first child needs no fetch.
//      A step is straight-line code: the NT tests, then per walk compact_step, which moves
//      (k, L) and ends in the predicated fetch for the next step; only a test that the float
//      compare leaves open (missing value, fp64 tie) takes a branch.
// A stage is released as soon as the warp has left the heaps, before it starts on part 2, so the
// next batch of heaps arrives while the warps wait for their node fetches.
// The row tile holds floats also for fp64 forests: every value is rounded DOWN to float when the
// tile is staged.  With lo = the largest float <= threshold (what an fp64 forest's 8-byte node
// stores) and xl = the largest float <= x:  xl < lo proves x < threshold, xl > lo proves
// x > threshold, and only xl == lo leaves the answer open; then, and only then (once in 2^24
// visits on continuous data), the walk reads the row's double from global memory and the exact
// threshold from a side array.  So fp64 forests run on 4-byte tiles and float compares and still
// decide every test exactly.  (fp32 forests: xl = x, lo = threshold, only a missing value is open.)
// Categories survive the rounding too: integers below 2^24 are floats, so trunc(xl) = trunc(x).
// Small batches split the tree batches of a row tile over CTAs (blockIdx.y) and leave raw sums
// for finish_kernel, like the dense kernel does.
#include "device_common.cuh"
#include "kernels_q.hpp"

namespace b2fil {
namespace {

constexpr int kCompactThreads    = 800;   // 24 consumer warps + 1 producer warp (72 registers)
constexpr int kCompactThreadsBig = 1024;  // 31 consumer warps + 1 producer warp (64 registers)

__device__ __forceinline__ void lds_node(uint32_t a, uint32_t& value, uint32_t& meta)
{
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(value), "=r"(meta) : "r"(a));
}

// One aligned 16-byte fetch = nodes 2m and 2m + 1, issued only where `wanted`; the registers keep
// their contents otherwise.  A predicated instruction rather than a branch: the walks of a warp
// want their fetches at different steps, and a branch per fetch costs more issue slots than the
// fetch.  L2-only (.cg): the fetches of a warp go to 32 unrelated lines and nothing is reused, so
// the L1 should only track the misses in flight (measured 4 to 8 % faster than the read-only
// path; L2 eviction hints measured slower).
__device__ __forceinline__ void ld_compact_pair_if(bool wanted, const void* ptr, uint32_t& x,
                                                   uint32_t& y, uint32_t& z, uint32_t& w)
{
  asm volatile(
    "{\n\t"
    ".reg .pred want;\n\t"
    "setp.ne.u32 want, %5, 0;\n\t"
    "@want ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];\n\t"
    "}"
    : "+r"(x), "+r"(y), "+r"(z), "+r"(w)
    : "l"(ptr), "r"(static_cast<uint32_t>(wanted)));
}

// A test is the float compare xl < lo, where xl is the row's value rounded down to float and lo
// the node's float (fp64 forests: the largest float <= threshold).  It is OPEN when that compare
// does not settle it: the value is missing, or, in an fp64 forest, xl == lo (lo <= x < next float:
// only the doubles know).  One compare instruction (equal-or-unordered) finds both.
template <typename T>
__device__ __forceinline__ bool test_is_open(float xl, float lo)
{
  if constexpr (sizeof(T) == 8) return !(xl < lo || xl > lo);
  return xl != xl;
}

// Exact form of an fp64 test that the floats left open.  `k` is the internal node whose exact
// threshold settles it (C_NO_NODE: none, heap padding: the row goes right).
__device__ __noinline__ bool compact_exact_left(const double* row_values, const double* exact,
                                                uint32_t k, uint32_t feat)
{
  if (k == C_NO_NODE) return false;
  // rows past the end of the batch (no values) were staged as zeros
  const double x = row_values != nullptr ? __ldg(row_values + feat) : 0.0;
  return x < __ldg(exact + k);
}

// Settle an open test off the common path and rewrite (xl, lo) so that the plain compare
// xl < lo gives the answer.
template <typename T, typename ExactIndex>
__device__ __forceinline__ void settle_open_test(float& xl, float& lo, uint32_t meta, uint32_t feat,
                                                 const double* row_values, const double* exact,
                                                 ExactIndex exact_index)
{
  if (!test_is_open<T>(xl, lo)) return;
  bool left = false;  // fp32 forests: xl == lo is x == threshold, which goes right
  if (xl != xl) {
    left = (meta & META_DEFAULT_LEFT) != 0u;
  } else if constexpr (sizeof(T) == 8) {
    left = compact_exact_left(row_values, exact, exact_index(), feat);
  }
  lo = 0.f;
  xl = left ? -1.f : 1.f;
}

// A categorical test, also rewritten into (xl, lo).
__device__ __forceinline__ void settle_categorical_test(float& xl, float& lo, uint32_t value,
                                                        uint32_t meta, const ForestView& f)
{
  const bool right = goes_right<float, true, true>(value, meta, xl, f);
  lo               = 0.f;
  xl               = right ? 1.f : -1.f;
}

// One step of a walk below the heap, after its test operands (xl, lo) are known.  State: k = the
// node the walk is on (bit 31 set once it has reached its leaf), L = leaves before the walk's
// position, {x, y, z, w} = the aligned pair of nodes that holds node k.  The step takes the
// branch, moves (k, L), and fetches the pair of the new node when that is a different pair: a
// first child reached from an even node is the neighbour already held.  Predicate logic all the
// way, no branch; written in PTX because the C++ form of the same step compiled to 2.5 times the
// instructions (flags kept as integers and re-tested), and issue slots are what the walk is
// short of.
__device__ __forceinline__ void compact_step(uint32_t& k, uint32_t& L, uint32_t& x, uint32_t& y,
                                             uint32_t& z, uint32_t& w, float xl, float lo,
                                             uint32_t meta, int off_shift, const void* nodes)
{
  asm volatile(
    "{\n\t"
    ".reg .pred lt, sw, second, leaf, live, ls, go, want;\n\t"
    ".reg .u32 t, off, hop, kn;\n\t"
    ".reg .u64 a;\n\t"
    "setp.lt.f32 lt, %6, %7;\n\t"
    "and.b32 t, %8, 0x08000000;\n\t"  // CMETA_SWAPPED
    "setp.ne.u32 sw, t, 0;\n\t"
    "xor.pred second, lt, sw;\n\t"
    "not.pred second, second;\n\t"    // second child = (left == swapped)
    "shl.b32 off, %8, 5;\n\t"
    "shr.u32 off, off, %9;\n\t"
    "selp.u32 t, 0x10000000, 0x20000000, second;\n\t"  // CMETA_SECOND_LEAF, CMETA_FIRST_LEAF
    "and.b32 t, t, %8;\n\t"
    "setp.ne.u32 leaf, t, 0;\n\t"
    "setp.ge.s32 live, %0, 0;\n\t"
    "and.pred ls, live, second;\n\t"
    "@ls add.u32 %1, %1, off;\n\t"    // the second child skips the leaves of the first
    "selp.u32 hop, off, 1, second;\n\t"
    "and.pred go, live, !leaf;\n\t"
    "add.u32 kn, %0, hop;\n\t"
    "xor.b32 t, kn, %0;\n\t"
    "setp.gt.u32 want, t, 1;\n\t"     // another pair
    "and.pred want, want, go;\n\t"
    "@!go or.b32 %0, %0, 0x80000000;\n\t"
    "@go mov.u32 %0, kn;\n\t"
    "and.b32 t, kn, 0x7ffffffe;\n\t"
    "mad.wide.u32 a, t, 8, %10;\n\t"
    "@want ld.global.cg.v4.u32 {%2, %3, %4, %5}, [a];\n\t"
    "}"
    : "+r"(k), "+r"(L), "+r"(x), "+r"(y), "+r"(z), "+r"(w)
    : "f"(xl), "f"(lo), "r"(meta), "r"(off_shift), "l"(nodes));
}
static_assert(CMETA_SWAPPED == 0x08000000u && CMETA_SECOND_LEAF == 0x10000000u &&
                CMETA_FIRST_LEAF == 0x20000000u && C_EXIT_LEAF == 0x80000000u,
              "compact_step spells these constants out");

// Stage rows [row0, row0 + R) feature-major as floats (fp64 inputs rounded down).  A warp reads 32
// consecutive features of one row and scatters them to 32 different banks.  Rows past the end of
// the batch become zeros.
template <typename T>
__device__ __forceinline__ void stage_rows_as_float(const PredictParams& p, uint32_t tile, int R,
                                                    int64_t row0, int warp, int lane, int n_warps)
{
  const int F             = p.f.n_features;
  const uint32_t stride_b = (R + 1) * 4u;
  const T* X              = static_cast<const T*>(p.X);
  for (int rr = warp; rr < R; rr += n_warps) {
    const int64_t row = row0 + rr;
    const bool live   = row < p.n_rows;
    const T* src      = X + row * p.row_stride;
    for (int c = lane; c < F; c += 32) {
      float v = 0.f;
      if (live) {
        const T raw = __ldg(src + c);
        if constexpr (sizeof(T) == 8) {
          v = __double2float_rd(raw);
        } else {
          v = raw;
        }
      }
      Traits<float>::st_real(tile + c * stride_b + rr * 4u, v);
    }
  }
}

// Shared memory: [mbarriers 256 B][row tile][accumulators][16 B][S stages of G * NT heaps].
template <typename T, bool CAT, int MODE, int NT, int MAXT>
__global__ void __launch_bounds__(MAXT, 1)
sparse_compact_kernel(const PredictParams p, const int R, const int G, const int S,
                      const int n_splits, T* __restrict__ partial)
{
  using TR  = Traits<T>;
  using Val = typename TR::Val;
  extern __shared__ __align__(128) unsigned char smem[];
  const ForestView& f = p.f;
  const int F         = f.n_features;
  const int NC        = f.n_outputs;
  const int rw        = R >> 5;
  const int n_cw      = rw * G;
  const int n_ct      = n_cw * 32;
  const int warp      = threadIdx.x >> 5;
  const int lane      = threadIdx.x & 31;
  const int TL        = f.c_top_levels;
  const uint32_t heap_n     = 1u << TL;
  const uint32_t top_stride = static_cast<uint32_t>(f.c_top_stride);
  const int fb              = f.c_feat_bits;
  const uint32_t feat_mask  = (1u << fb) - 1u;

  const uint32_t stride_b    = (R + 1) * 4u;  // the tile holds floats whatever the forest precision
  const size_t tile_bytes    = align16(static_cast<size_t>(F) * stride_b);
  const size_t acc_bytes     = (MODE <= MODE_VECTOR) ? align16(static_cast<size_t>(G) * NC * R * TR::ES) : 0;
  unsigned char* tile_ptr    = smem + kBarBytes;
  T* acc                     = reinterpret_cast<T*>(tile_ptr + tile_bytes);
  unsigned char* stage_ptr   = tile_ptr + tile_bytes + acc_bytes + 16;
  const uint32_t bars        = smem_addr(smem);
  const uint32_t tile        = smem_addr(tile_ptr);
  const uint32_t stages      = smem_addr(stage_ptr);
  const int per_batch        = G * NT;
  const uint32_t stage_bytes = per_batch * top_stride;
  const int n_batches        = (f.n_trees + per_batch - 1) / per_batch;
  // small batches: blockIdx.y splits the tree batches over CTAs (n_splits = gridDim.y); a CTA
  // then streams and walks only its share and leaves raw sums for finish_kernel
  const int b_begin = static_cast<int>(static_cast<int64_t>(n_batches) * blockIdx.y / n_splits);
  const int b_end   = static_cast<int>(static_cast<int64_t>(n_batches) * (blockIdx.y + 1) / n_splits);
  const int64_t n_tiles      = (p.n_rows + R - 1) / R;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bars + 8u * s, 1);                    // full: the producer's expect_tx arrival
      mbar_init(bars + 8u * (kMaxStages + s), n_cw);  // empty: one arrival per consumer warp
    }
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == n_cw) {
    // ---- producer: one thread streams the heaps of tree batches into the stage ring ------------
    if (lane == 0) {
      const unsigned char* src = f.c_top;
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
          const uint32_t bytes = count * top_stride;
          mbar_expect_tx(bars + 8u * s, bytes);
          bulk_copy_g2s(stages + s * stage_bytes, src + static_cast<size_t>(first) * top_stride,
                        bytes, bars + 8u * s);
          pos.advance(S);
          if (pos.stage == 0) primed = true;
        }
      }
    }
    return;
  }
  if (warp > n_cw) return;

  // ---- consumers --------------------------------------------------------------------------------
  const int g             = warp / rw;
  const int r             = (warp % rw) * 32 + lane;
  T* acc_group            = acc + static_cast<size_t>(g) * NC * R;
  const uint32_t row_addr = tile + r * 4u;
  const CompactNode* __restrict__ nodes = f.c_nodes;
  RingPos pos;
  bool ok = true;
  for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const int64_t row0 = t * R;
    const int64_t row  = row0 + r;
    stage_rows_as_float<T>(p, tile, R, row0, warp, lane, n_cw);
    if (MODE <= MODE_VECTOR) {
      for (int i = threadIdx.x; i < G * NC * R; i += n_ct) acc[i] = T(0);
    }
    consumer_sync(n_ct);
    {
      // ask the L2 for the rows of this CTA's next tile, so that staging them does not wait on HBM
      const int64_t next0 = row0 + static_cast<int64_t>(gridDim.x) * R;
      const int row_bytes = F * static_cast<int>(sizeof(T));
      const int lines     = (row_bytes + 127) >> 7;
      for (int i = threadIdx.x; i < R * lines; i += n_ct) {
        const int64_t nrow = next0 + i / lines;
        if (nrow < p.n_rows) {
          const char* at = reinterpret_cast<const char*>(static_cast<const T*>(p.X) + nrow * p.row_stride) +
                           min((i % lines) << 7, row_bytes - 1);
          asm volatile("prefetch.global.L2 [%0];" ::"l"(at));
        }
      }
    }
    Running<T> run{T(0), 0, {}};
    // the row's doubles, for the tests that the float tile leaves open
    auto row_values = [&]() -> const double* {
      return row < p.n_rows ? static_cast<const double*>(p.X) + row * p.row_stride : nullptr;
    };
    for (int b = b_begin; b < b_end; ++b) {
      const uint32_t s = pos.stage;
      if (ok) ok = mbar_wait(bars + 8u * s, pos.phase);
      const int first = b * per_batch + g * NT;
      const int n_act = ok ? min(NT, f.n_trees - first) : 0;
      uint32_t k[NT], L[NT];  // bit 31 of k: the walk has reached its leaf, L is its number
      if (n_act > 0) {
        // part 1: the heaps in shared memory
        uint32_t base[NT], h[NT];
#pragma unroll
        for (int kk = 0; kk < NT; ++kk) {
          // slots past the end of the forest repeat the last live tree; results are dropped
          base[kk] = stages + s * stage_bytes +
                     static_cast<uint32_t>(g * NT + min(kk, n_act - 1)) * top_stride;
          h[kk] = 1u;
        }
        for (int lvl = 0; lvl < TL; ++lvl) {
          uint32_t value[NT], meta[NT];
          float xl[NT], lo[NT];
          bool any_open = false;
#pragma unroll
          for (int kk = 0; kk < NT; ++kk) lds_node(base[kk] + h[kk] * 8u, value[kk], meta[kk]);
#pragma unroll
          for (int kk = 0; kk < NT; ++kk) {
            xl[kk] = Traits<float>::ld_real((meta[kk] & CMETA_LOW27) * stride_b + row_addr);
            lo[kk] = __uint_as_float(value[kk]);
            if (CAT && (meta[kk] & META_CATEGORICAL))
              settle_categorical_test(xl[kk], lo[kk], value[kk], meta[kk], f);
            any_open |= test_is_open<T>(xl[kk], lo[kk]);
          }
          if (any_open) {
#pragma unroll
            for (int kk = 0; kk < NT; ++kk) {
              settle_open_test<T>(xl[kk], lo[kk], meta[kk], meta[kk] & CMETA_LOW27, row_values(),
                                  f.c_exact, [&]() {
                                    const size_t tree = static_cast<size_t>(first + min(kk, n_act - 1));
                                    return __ldg(f.c_top_src + tree * heap_n + h[kk]);
                                  });
            }
          }
#pragma unroll
          for (int kk = 0; kk < NT; ++kk) h[kk] = 2u * h[kk] + (xl[kk] < lo[kk] ? 0u : 1u);
        }
#pragma unroll
        for (int kk = 0; kk < NT; ++kk) {
          // the exits follow the 2^T node slots: exit e sits at 8 * (2^T + e) = 8 * h
          uint32_t ek, eL;
          lds_node(base[kk] + h[kk] * 8u, ek, eL);
          const bool done = (ek & C_EXIT_LEAF) != 0u;
          k[kk]           = ek;                              // an exit that is a leaf carries bit 31
          L[kk]           = done ? (ek & ~C_EXIT_LEAF) : eL;  // the leaf itself, or leaves before k
        }
      }
      // the heaps of this batch are no longer needed: let the producer refill the stage
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8u * (kMaxStages + s));
      pos.advance(S);
      if (n_act > 0) {
        // part 2: compact nodes in global memory
        // Nodes come in aligned pairs {2m, 2m + 1} and a walk holds the pair of its node.  The
        // first child of node k is node k + 1, so a walk that sits on an even node and goes to its
        // first child already holds the next node and skips the fetch: lanes that skip touch no
        // cache line.  A step is straight-line code: the operands of the NT tests, one rarely
        // taken branch for tests that the floats leave open, then NT times compact_step, which
        // ends in the (predicated) fetch for the next step.
        uint32_t pair[NT][4];
        const uint2* node_ptr = reinterpret_cast<const uint2*>(nodes);
#pragma unroll
        for (int kk = 0; kk < NT; ++kk) {
          // a walk that ended in the heap keeps a node that no value ties with
          pair[kk][0] = pair[kk][2] = 0x00800001u;
          pair[kk][1] = pair[kk][3] = 0u;
          ld_compact_pair_if(static_cast<int32_t>(k[kk]) >= 0, node_ptr + (k[kk] & 0x7ffffffeu),
                             pair[kk][0], pair[kk][1], pair[kk][2], pair[kk][3]);
        }
        const int off_shift = 5 + fb;  // the offset sits between the five flag bits and the feature
        for (int step = 0; step < f.c_bottom_steps; ++step) {
          uint32_t value[NT], meta[NT];
          float xl[NT], lo[NT];
          bool any_open = false;
#pragma unroll
          for (int kk = 0; kk < NT; ++kk) {
            const bool odd = (k[kk] & 1u) != 0u;
            value[kk]      = odd ? pair[kk][2] : pair[kk][0];
            meta[kk]       = odd ? pair[kk][3] : pair[kk][1];
            xl[kk]         = Traits<float>::ld_real((meta[kk] & feat_mask) * stride_b + row_addr);
            lo[kk]         = __uint_as_float(value[kk]);
            if (CAT && (meta[kk] & META_CATEGORICAL))
              settle_categorical_test(xl[kk], lo[kk], value[kk], meta[kk], f);
            any_open |= test_is_open<T>(xl[kk], lo[kk]);
          }
          if (any_open) {
#pragma unroll
            for (int kk = 0; kk < NT; ++kk) {
              // (a finished walk repeats its last test: nothing to settle)
              if (static_cast<int32_t>(k[kk]) >= 0)
                settle_open_test<T>(xl[kk], lo[kk], meta[kk], meta[kk] & feat_mask, row_values(),
                                    f.c_exact, [&]() { return k[kk]; });
            }
          }
#pragma unroll
          for (int kk = 0; kk < NT; ++kk)
            compact_step(k[kk], L[kk], pair[kk][0], pair[kk][1], pair[kk][2], pair[kk][3], xl[kk],
                         lo[kk], meta[kk], off_shift, node_ptr);
          uint32_t all = k[0];
#pragma unroll
          for (int kk = 1; kk < NT; ++kk) all &= k[kk];
          if (!__any_sync(0xffffffffu, static_cast<int32_t>(all) >= 0)) break;
        }
        // the leaves: payload (or id) from the leaf arrays
        if (MODE == MODE_LEAFID) {
          uint32_t id[NT];
#pragma unroll
          for (int kk = 0; kk < NT; ++kk)
            id[kk] = __ldg(f.c_leaf_ids + L[kk]);
          // four live trees that are also the caller's trees o, o + 1, o + 2, o + 3 with o a
          // multiple of four: the row's four ids are contiguous and leave as one 16-byte store
          // (scalar 4-byte stores at a stride of a whole output row cost a sector request each)
          int orig[NT];
#pragma unroll
          for (int kk = 0; kk < NT; ++kk) orig[kk] = __ldg(f.tree_orig + first + min(kk, n_act - 1));
          bool wide = NT == 4 && n_act == NT && (orig[0] & 3) == 0 && (f.n_trees & 3) == 0 &&
                      (reinterpret_cast<uintptr_t>(p.out) & 15u) == 0;
#pragma unroll
          for (int kk = 1; kk < NT; ++kk) wide = wide && orig[kk] == orig[0] + kk;
          if (wide) {
            if (row < p.n_rows) {
              uint32_t* dst = static_cast<uint32_t*>(p.out) + row * f.n_trees + orig[0];
              *reinterpret_cast<uint4*>(dst) =
                make_uint4(id[0], id[NT > 1 ? 1 : 0], id[NT > 2 ? 2 : 0], id[NT > 3 ? 3 : 0]);
            }
          } else {
#pragma unroll
            for (int kk = 0; kk < NT; ++kk) {
              if (kk < n_act && row < p.n_rows)
                static_cast<uint32_t*>(p.out)[row * f.n_trees + orig[kk]] = id[kk];
            }
          }
        } else {
          Val pay[NT];
#pragma unroll
          for (int kk = 0; kk < NT; ++kk) {
            pay[kk] = __ldg(static_cast<const Val*>(f.c_leaf_payload) + L[kk]);
          }
          bool wide = false;
          int first_orig = 0;
          if (MODE == MODE_PERTREE) {
            // per-tree scalar outputs: the same 16-byte stores as for leaf ids
            first_orig = __ldg(f.tree_orig + first);
            wide = NT == 4 && n_act == NT && f.leaf_vector_len <= 1 && (first_orig & 3) == 0 &&
                   (f.n_trees & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15u) == 0;
#pragma unroll
            for (int kk = 1; kk < NT; ++kk)
              wide = wide && __ldg(f.tree_orig + first + min(kk, n_act - 1)) == first_orig + kk;
          }
          if (MODE == MODE_PERTREE && wide) {
            if (row < p.n_rows) {
              Val* dst = static_cast<Val*>(p.out) + row * f.n_trees + first_orig;
              if constexpr (sizeof(Val) == 4) {
                *reinterpret_cast<uint4*>(dst) = make_uint4(pay[0], pay[NT > 1 ? 1 : 0],
                                                            pay[NT > 2 ? 2 : 0], pay[NT > 3 ? 3 : 0]);
              } else {
                *reinterpret_cast<ulonglong2*>(dst)     = make_ulonglong2(pay[0], pay[NT > 1 ? 1 : 0]);
                *reinterpret_cast<ulonglong2*>(dst + 2) = make_ulonglong2(pay[NT > 2 ? 2 : 0],
                                                                          pay[NT > 3 ? 3 : 0]);
              }
            }
          } else {
#pragma unroll
            for (int kk = 0; kk < NT; ++kk) {
              if (kk < n_act) take_leaf<T, MODE>(p, first + kk, pay[kk], 0u, acc_group, R, r, row, run);
            }
          }
        }
      }
    }
    if (!ok) atomicExch(p.status, 2);
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
    consumer_sync(n_ct);
  }
}

size_t compact_smem(const ForestView& f, size_t es, bool reduce, int R, int G, int NT, int S)
{
  size_t b = kBarBytes;
  b += align16(static_cast<size_t>(f.n_features) * (R + 1) * 4);  // the row tile holds floats
  if (reduce) b += align16(static_cast<size_t>(G) * f.n_outputs * R * es);
  b += 16;
  b += static_cast<size_t>(S) * G * NT * static_cast<size_t>(f.c_top_stride);
  return b;
}

template <typename T, bool CAT, int MODE>
int launch_mode(const PredictParams& p, const CompactCfg& c, void* partial, cudaStream_t stream,
                std::string& err)
{
  const dim3 grid(c.grid, c.splits);
  T* part = static_cast<T*>(partial);
  if (c.threads > kCompactThreads) {
    auto k       = sparse_compact_kernel<T, CAT, MODE, kCompactTreesInFlight, kCompactThreadsBig>;
    const int rc = set_smem_bytes(reinterpret_cast<const void*>(k), c.smem_bytes, err);
    if (rc != B2FIL_OK) return rc;
    k<<<grid, c.threads, c.smem_bytes, stream>>>(p, c.rows_per_tile, c.tree_groups, c.stages,
                                                 c.splits, part);
    return B2FIL_OK;
  }
  auto k       = sparse_compact_kernel<T, CAT, MODE, kCompactTreesInFlight, kCompactThreads>;
  const int rc = set_smem_bytes(reinterpret_cast<const void*>(k), c.smem_bytes, err);
  if (rc != B2FIL_OK) return rc;
  k<<<grid, c.threads, c.smem_bytes, stream>>>(p, c.rows_per_tile, c.tree_groups, c.stages,
                                               c.splits, part);
  return B2FIL_OK;
}

template <typename T, bool CAT>
int launch_cat(const PredictParams& p, int mode, const CompactCfg& c, void* partial,
               cudaStream_t stream, std::string& err)
{
  switch (mode) {
    case MODE_SCALAR: return launch_mode<T, CAT, MODE_SCALAR>(p, c, partial, stream, err);
    case MODE_VECTOR: return launch_mode<T, CAT, MODE_VECTOR>(p, c, partial, stream, err);
    case MODE_PERTREE: return launch_mode<T, CAT, MODE_PERTREE>(p, c, partial, stream, err);
    default: return launch_mode<T, CAT, MODE_LEAFID>(p, c, partial, stream, err);
  }
}

}  // namespace

bool compact_config(const ForestView& f, bool reduce, int rows_per_tile, int64_t n_rows,
                    int sm_count, bool may_split, CompactCfg& cfg)
{
  if (!f.c_enabled) return false;
  const size_t es = f.format == FMT_SPARSE_16D ? 8 : 4;
  // Small batches (fewer row tiles than half the SMs): one CTA per tile would walk the whole
  // forest batch after batch, which is what bounds their latency.  The tree batches are split
  // over CTAs instead (tiles x splits fills the SMs once) with few tree groups per CTA, so that
  // there are enough batches to split.
  const int64_t small_tiles = (n_rows + 31) / 32;
  if (may_split && small_tiles * 2 <= sm_count && tuning_value("compact_R", 0) == 0) {
    const int want_splits = static_cast<int>(sm_count / small_tiles);
    const int n_quads     = (f.n_trees + kCompactTreesInFlight - 1) / kCompactTreesInFlight;
    int G                 = std::max(1, std::min(31, (n_quads + want_splits - 1) / want_splits));
    for (; G >= 1; --G) {
      const size_t b = compact_smem(f, es, reduce, 32, G, kCompactTreesInFlight, 1);
      if (b > kMaxSmemBytes) continue;
      const int per_batch = G * kCompactTreesInFlight;
      const int n_batches = (f.n_trees + per_batch - 1) / per_batch;
      const int splits    = std::max(1, std::min(n_batches, want_splits));
      cfg = CompactCfg{32, G, 1, b, (G + 1) * 32, static_cast<int>(small_tiles), splits};
      return true;
    }
  }
  if (const int R = tuning_value("compact_R", 0), G = tuning_value("compact_G", 0),
      S = tuning_value("compact_S", 0);
      R >= 32 && (R & (R - 1)) == 0 && R <= 128 && G >= 1 && (R / 32) * G <= 31 && S >= 1 &&
      S <= kMaxStages) {  // tuning aid: forced shape
    const size_t b = compact_smem(f, es, reduce, R, G, kCompactTreesInFlight, S);
    if (b <= kMaxSmemBytes) {
      const int64_t n_tiles = (n_rows + R - 1) / R;
      cfg = CompactCfg{R, G, S, b, ((R / 32) * G + 1) * 32,
                       static_cast<int>(std::min<int64_t>(n_tiles, sm_count)), 1};
      return true;
    }
  }
  // Shared memory left unused becomes L1, which is what keeps the node fetches in flight: shapes
  // that stay under 160 KiB are preferred (measured: the same kernel runs twice as fast at
  // 110 KiB as at 216 KiB).  Within a limit: as many warps as fit (up to 31 consumer warps; above
  // 24 the 1024-thread build with 64 registers runs), then a second stage.
  for (const size_t limit : {size_t(160) * 1024, kMaxSmemBytes}) {
    for (int R = rows_per_tile; R >= 32; R /= 2) {
      const int rw = R / 32;
      for (int G = std::min(31 / rw, std::max(1, (f.n_trees + kCompactTreesInFlight - 1) /
                                                    kCompactTreesInFlight));
           G >= 1; --G) {
        for (int S = 2; S >= 1; --S) {
          const size_t b = compact_smem(f, es, reduce, R, G, kCompactTreesInFlight, S);
          if (b <= limit) {
            const int64_t n_tiles = (n_rows + R - 1) / R;
            cfg = CompactCfg{R, G, S, b, (rw * G + 1) * 32,
                             static_cast<int>(std::min<int64_t>(n_tiles, sm_count)), 1};
            return true;
          }
        }
      }
    }
  }
  return false;
}

int launch_sparse_compact(const PredictParams& p, int mode, const CompactCfg& c,
                          cudaStream_t stream, cudaMemPool_t pool, std::string& err,
                          int64_t* launches)
{
  const ForestView& f = p.f;
  const bool f64      = f.format == FMT_SPARSE_16D;
  void* partial       = nullptr;
  if (c.splits > 1 && mode <= MODE_VECTOR) {
    const size_t bytes  = static_cast<size_t>(c.splits) * f.n_outputs * p.n_rows * (f64 ? 8 : 4);
    const cudaError_t e = cudaMallocFromPoolAsync(&partial, bytes, pool, stream);
    if (e != cudaSuccess) {
      cudaGetLastError();
      err = std::string("scratch allocation for split prediction failed: ") + cudaGetErrorString(e);
      return e == cudaErrorMemoryAllocation ? B2FIL_ERR_NO_MEMORY : B2FIL_ERR_CUDA;
    }
  }
  int rc;
  if (f64) {
    rc = f.has_categorical ? launch_cat<double, true>(p, mode, c, partial, stream, err)
                           : launch_cat<double, false>(p, mode, c, partial, stream, err);
  } else {
    rc = f.has_categorical ? launch_cat<float, true>(p, mode, c, partial, stream, err)
                           : launch_cat<float, false>(p, mode, c, partial, stream, err);
  }
  if (partial) {
    if (rc == B2FIL_OK) {
      launch_finish_rows(p, partial, c.splits, f64, stream);
      if (launches) ++*launches;
    }
    cudaFreeAsync(partial, stream);
  }
  return rc;
}

}  // namespace b2fil
