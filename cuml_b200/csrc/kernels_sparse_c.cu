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
//      Every step first issues the fetches of all NT walks, then advances them.
// A stage is released as soon as the warp has left the heaps, before it starts on part 2, so the
// next batch of heaps arrives while the warps wait for their node fetches.
// The row tile holds floats also for fp64 forests: every value is rounded DOWN to float when the
// tile is staged.  With lo = the largest float <= threshold (what an fp64 forest's 8-byte node
// stores) and xl = the largest float <= x:  xl < lo proves x < threshold, xl > lo proves
// x > threshold, and only xl == lo leaves the answer open; then, and only then (once in 2^24
// visits on continuous data), the walk reads the row's double from global memory and the exact
// threshold from a side array.  So fp64 forests run on 4-byte tiles and float compares and still
// decide every test exactly.  (fp32 forests: xl = x, lo = threshold, nothing is ever open.)
// Categories survive the rounding too: integers below 2^24 are floats, so trunc(xl) = trunc(x).
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

// How the walk below the heap fetches its nodes from global memory.  The fetches of a warp go to
// 32 unrelated cache lines and nothing is reused, so what matters is how many of them the SM can
// keep in flight; the L1 allocation policy of the load decides that.
enum NodeLoad : int { kLoadNc = 0, kLoadCg = 1, kLoadNoAllocate = 2, kLoadCgKeep = 3 };

// L2 cache policies: the node array is read over and over and should stay (evict last); rows and
// leaf payloads are read once (evict first).
__device__ __forceinline__ uint64_t l2_policy_evict_last()
{
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first()
{
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint2 ld_compact_node(const uint2* ptr, int kind, uint64_t keep)
{
  uint2 v;
  if (kind == kLoadCgKeep) {
    asm volatile("ld.global.cg.L2::cache_hint.v2.u32 {%0, %1}, [%2], %3;"
                 : "=r"(v.x), "=r"(v.y)
                 : "l"(ptr), "l"(keep));
  } else if (kind == kLoadCg) {
    asm volatile("ld.global.cg.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(ptr));
  } else if (kind == kLoadNoAllocate) {
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];"
                 : "=r"(v.x), "=r"(v.y)
                 : "l"(ptr));
  } else {
    asm volatile("ld.global.nc.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(ptr));
  }
  return v;
}
// One aligned 16-byte load = nodes 2m and 2m + 1.
__device__ __forceinline__ uint4 ld_compact_pair(const uint4* ptr, int kind, uint64_t keep)
{
  uint4 v;
  if (kind == kLoadCgKeep) {
    asm volatile("ld.global.cg.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(ptr), "l"(keep));
  } else if (kind == kLoadCg) {
    asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(ptr));
  } else if (kind == kLoadNoAllocate) {
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(ptr));
  } else {
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(ptr));
  }
  return v;
}

// Does the row go right at a compact node?  `xl` is the row's value rounded down to float;
// `exact_index()` yields the internal node whose exact threshold settles an fp64 test that the
// float bound leaves open (C_NO_NODE: none, heap padding).
template <typename T, bool CAT, typename ExactIndex>
__device__ __forceinline__ bool compact_goes_right(uint32_t value, uint32_t meta, float xl,
                                                   uint32_t feat, int64_t row,
                                                   const PredictParams& p, ExactIndex exact_index)
{
  const ForestView& f = p.f;
  if (CAT && (meta & META_CATEGORICAL)) return goes_right<float, true, true>(value, meta, xl, f);
  const float lo = __uint_as_float(value);  // fp64 forests: largest float <= threshold
  bool left      = xl < lo;
  if constexpr (sizeof(T) == 8) {
    if (xl == lo) {
      // lo <= x < next float: only the doubles know
      const uint32_t k = exact_index();
      if (k != C_NO_NODE) {
        const double x = row < p.n_rows
                           ? __ldg(static_cast<const double*>(p.X) + row * p.row_stride + feat)
                           : 0.0;  // rows past the end of the batch were staged as zeros
        left = x < __ldg(f.c_exact + k);
      }
    }
  }
  if (xl != xl) left = (meta & META_DEFAULT_LEFT) != 0u;
  return !left;
}

// Stage rows [row0, row0 + R) feature-major as floats (fp64 inputs rounded down).  A warp reads 32
// consecutive features of one row and scatters them to 32 different banks.  Rows past the end of
// the batch become zeros.
template <typename T>
__device__ __forceinline__ T ld_once(const T* ptr, uint64_t once)
{
  T v;
  if constexpr (sizeof(T) == 8) {
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.b64 %0, [%1], %2;"
                 : "=l"(reinterpret_cast<uint64_t&>(v))
                 : "l"(ptr), "l"(once));
  } else {
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.b32 %0, [%1], %2;"
                 : "=r"(reinterpret_cast<uint32_t&>(v))
                 : "l"(ptr), "l"(once));
  }
  return v;
}

template <typename T>
__device__ __forceinline__ void stage_rows_as_float(const PredictParams& p, uint32_t tile, int R,
                                                    int64_t row0, int warp, int lane, int n_warps,
                                                    bool hint, uint64_t once)
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
        const T raw = hint ? ld_once(src + c, once) : __ldg(src + c);
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
                      const int node_load)
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
        for (int b = 0; b < n_batches; ++b) {
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
  const uint64_t keep  = l2_policy_evict_last();
  const uint64_t once  = l2_policy_evict_first();
  RingPos pos;
  bool ok = true;
  for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const int64_t row0 = t * R;
    const int64_t row  = row0 + r;
    stage_rows_as_float<T>(p, tile, R, row0, warp, lane, n_cw, node_load == kLoadCgKeep, once);
    if (MODE <= MODE_VECTOR) {
      for (int i = threadIdx.x; i < G * NC * R; i += n_ct) acc[i] = T(0);
    }
    consumer_sync(n_ct);
    Running<T> run{T(0), 0, {}};
    for (int b = 0; b < n_batches; ++b) {
      const uint32_t s = pos.stage;
      if (ok) ok = mbar_wait(bars + 8u * s, pos.phase);
      const int first = b * per_batch + g * NT;
      const int n_act = ok ? min(NT, f.n_trees - first) : 0;
      uint32_t k[NT], L[NT];
      bool live[NT];
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
#pragma unroll
          for (int kk = 0; kk < NT; ++kk) lds_node(base[kk] + h[kk] * 8u, value[kk], meta[kk]);
#pragma unroll
          for (int kk = 0; kk < NT; ++kk) {
            const uint32_t feat = meta[kk] & CMETA_LOW27;
            const float xl      = Traits<float>::ld_real(feat * stride_b + row_addr);
            const bool right    = compact_goes_right<T, CAT>(value[kk], meta[kk], xl, feat, row, p, [&]() {
              const size_t tree = static_cast<size_t>(first + min(kk, n_act - 1));
              return __ldg(f.c_top_src + tree * heap_n + h[kk]);
            });
            h[kk] = 2u * h[kk] + (right ? 1u : 0u);
          }
        }
#pragma unroll
        for (int kk = 0; kk < NT; ++kk) {
          // the exits follow the 2^T node slots: exit e sits at 8 * (2^T + e) = 8 * h
          uint32_t ek, eL;
          lds_node(base[kk] + h[kk] * 8u, ek, eL);
          live[kk] = (ek & C_EXIT_LEAF) == 0u;
          k[kk]    = live[kk] ? ek : 0u;  // a finished walk keeps fetching node 0: harmless
          L[kk]    = live[kk] ? eL : (ek & ~C_EXIT_LEAF);  // leaves before k, or the leaf itself
        }
      }
      // the heaps of this batch are no longer needed: let the producer refill the stage
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8u * (kMaxStages + s));
      pos.advance(S);
      if (n_act > 0) {
        // part 2: compact nodes in global memory
        // Nodes come in aligned pairs {2m, 2m + 1}.  The first child of node k is node k + 1, so
        // a walk that sits on an even node and goes to its first child already holds the next
        // node and skips the fetch: lanes that skip touch no cache line, and the L1's line
        // look-ups are what bounds this loop.  A walk on an even node loads the pair (16 bytes),
        // a walk on an odd node only its own node (8 bytes): no selects afterwards.
        uint32_t cv[NT], cm[NT], nv[NT], nm[NT];  // current node, and its neighbour when k is even
        bool need[NT];
#pragma unroll
        for (int kk = 0; kk < NT; ++kk) {
          need[kk] = live[kk];
          cv[kk] = cm[kk] = nv[kk] = nm[kk] = 0u;
        }
        const uint2* node_ptr = reinterpret_cast<const uint2*>(nodes);
        const int off_shift   = 5 + fb;  // the offset sits between the five flag bits and the feature
        for (int step = 0; step < f.c_bottom_steps; ++step) {
#pragma unroll
          for (int kk = 0; kk < NT; ++kk) {
            if (need[kk]) {
              if (k[kk] & 1u) {
                const uint2 one = ld_compact_node(node_ptr + k[kk], node_load, keep);
                cv[kk]          = one.x;
                cm[kk]          = one.y;
              } else {
                const uint4 two = ld_compact_pair(reinterpret_cast<const uint4*>(node_ptr + k[kk]), node_load, keep);
                cv[kk]          = two.x;
                cm[kk]          = two.y;
                nv[kk]          = two.z;
                nm[kk]          = two.w;
              }
            }
          }
          bool walking = false;
#pragma unroll
          for (int kk = 0; kk < NT; ++kk) {
            const uint32_t meta = cm[kk];
            const uint32_t feat = meta & feat_mask;
            const float xl      = Traits<float>::ld_real(feat * stride_b + row_addr);
            const uint32_t kx   = k[kk];
            const bool right    = compact_goes_right<T, CAT>(cv[kk], meta, xl, feat, row, p,
                                                             [&]() { return kx; });
            const bool second   = right != ((meta & CMETA_SWAPPED) != 0u);
            const uint32_t off  = (meta << 5) >> off_shift;
            const bool at_leaf  = (meta & (second ? CMETA_SECOND_LEAF : CMETA_FIRST_LEAF)) != 0u;
            if (live[kk]) {
              const uint32_t hop = second ? off : 0u;
              L[kk] += hop;
              live[kk] = !at_leaf;
              if (live[kk]) {
                // a first child reached from an even node is the neighbour already held
                const bool reuse = !second && (kx & 1u) == 0u;
                k[kk]            = kx + (second ? off : 1u);
                need[kk]         = !reuse;
                if (reuse) {
                  cv[kk] = nv[kk];
                  cm[kk] = nm[kk];
                }
              } else {
                need[kk] = false;
              }
            }
            walking |= live[kk];
          }
          if (!__any_sync(0xffffffffu, walking)) break;
        }
        // the leaves: payload (or id) from the leaf arrays
        if (MODE == MODE_LEAFID) {
          uint32_t id[NT];
#pragma unroll
          for (int kk = 0; kk < NT; ++kk)
            id[kk] = node_load == kLoadCgKeep ? ld_once(f.c_leaf_ids + L[kk], once) : __ldg(f.c_leaf_ids + L[kk]);
#pragma unroll
          for (int kk = 0; kk < NT; ++kk) {
            if (kk < n_act && row < p.n_rows) {
              const int orig = __ldg(f.tree_orig + first + kk);
              static_cast<uint32_t*>(p.out)[row * f.n_trees + orig] = id[kk];
            }
          }
        } else {
          Val pay[NT];
#pragma unroll
          for (int kk = 0; kk < NT; ++kk) {
            const Val* lp = static_cast<const Val*>(f.c_leaf_payload) + L[kk];
            pay[kk]       = node_load == kLoadCgKeep ? ld_once(lp, once) : __ldg(lp);
          }
#pragma unroll
          for (int kk = 0; kk < NT; ++kk) {
            if (kk < n_act) take_leaf<T, MODE>(p, first + kk, pay[kk], 0u, acc_group, R, r, row, run);
          }
        }
      }
    }
    if (!ok) atomicExch(p.status, 2);
    flush_running<T, MODE>(f, run, acc_group, R, r);
    consumer_sync(n_ct);
    if (MODE <= MODE_VECTOR) {
      if (threadIdx.x < R) finish_row<T>(p, acc, R, G, threadIdx.x, row0 + threadIdx.x);
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
int launch_mode(const PredictParams& p, const CompactCfg& c, cudaStream_t stream, std::string& err)
{
  if (c.threads > kCompactThreads) {
    auto k       = sparse_compact_kernel<T, CAT, MODE, kCompactTreesInFlight, kCompactThreadsBig>;
    const int rc = set_smem_bytes(reinterpret_cast<const void*>(k), c.smem_bytes, err);
    if (rc != B2FIL_OK) return rc;
    k<<<c.grid, c.threads, c.smem_bytes, stream>>>(p, c.rows_per_tile, c.tree_groups, c.stages,
                                                   c.node_load);
    return B2FIL_OK;
  }
  auto k       = sparse_compact_kernel<T, CAT, MODE, kCompactTreesInFlight, kCompactThreads>;
  const int rc = set_smem_bytes(reinterpret_cast<const void*>(k), c.smem_bytes, err);
  if (rc != B2FIL_OK) return rc;
  k<<<c.grid, c.threads, c.smem_bytes, stream>>>(p, c.rows_per_tile, c.tree_groups, c.stages,
                                                 c.node_load);
  return B2FIL_OK;
}

template <typename T, bool CAT>
int launch_cat(const PredictParams& p, int mode, const CompactCfg& c, cudaStream_t stream,
               std::string& err)
{
  switch (mode) {
    case MODE_SCALAR: return launch_mode<T, CAT, MODE_SCALAR>(p, c, stream, err);
    case MODE_VECTOR: return launch_mode<T, CAT, MODE_VECTOR>(p, c, stream, err);
    case MODE_PERTREE: return launch_mode<T, CAT, MODE_PERTREE>(p, c, stream, err);
    default: return launch_mode<T, CAT, MODE_LEAFID>(p, c, stream, err);
  }
}

}  // namespace

bool compact_config(const ForestView& f, bool reduce, int rows_per_tile, int64_t n_rows,
                    int sm_count, CompactCfg& cfg)
{
  if (!f.c_enabled) return false;
  const size_t es = f.format == FMT_SPARSE_16D ? 8 : 4;
  // L2-only loads measured 4 to 8 % faster than the read-only path: the lines are never reused
  const int load  = tuning_value("compact_load", kLoadCg);
  if (const int R = tuning_value("compact_R", 0), G = tuning_value("compact_G", 0),
      S = tuning_value("compact_S", 0);
      R >= 32 && (R & (R - 1)) == 0 && R <= 128 && G >= 1 && (R / 32) * G <= 31 && S >= 1 &&
      S <= kMaxStages) {  // tuning aid: forced shape
    const size_t b = compact_smem(f, es, reduce, R, G, kCompactTreesInFlight, S);
    if (b <= kMaxSmemBytes) {
      const int64_t n_tiles = (n_rows + R - 1) / R;
      cfg = CompactCfg{R, G, S, b, ((R / 32) * G + 1) * 32,
                       static_cast<int>(std::min<int64_t>(n_tiles, sm_count)), load};
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
                             static_cast<int>(std::min<int64_t>(n_tiles, sm_count)), load};
            return true;
          }
        }
      }
    }
  }
  return false;
}

int launch_sparse_compact(const PredictParams& p, int mode, const CompactCfg& c,
                          cudaStream_t stream, std::string& err)
{
  const ForestView& f = p.f;
  if (f.format == FMT_SPARSE_16D) {
    return f.has_categorical ? launch_cat<double, true>(p, mode, c, stream, err)
                             : launch_cat<double, false>(p, mode, c, stream, err);
  }
  return f.has_categorical ? launch_cat<float, true>(p, mode, c, stream, err)
                           : launch_cat<float, false>(p, mode, c, stream, err);
}

}  // namespace b2fil
