// Kernel for sparse forests that carry the compact image (forest.hpp): deep, ragged trees whose
// prediction is a chain of dependent node fetches.
//
// A CTA owns a tile of R rows staged feature-major in shared memory, like the other kernels, and
// its warps form (R/32 row sets) x (G tree groups); a warp walks its 32 rows through NT trees at
// a time.  Every walk has two parts:
//   1. the top T levels of the tree are a complete heap that a producer warp streams through a
//      ring of shared-memory stages (bulk copies from the L2-resident heap array; one stage =
//      the heaps of G * NT trees): T steps without a global fetch, then one exit word that names
//      the internal node to continue at, or the leaf reached;
//   2. below the heap the walk follows the compact nodes in global memory: 8-byte internal
//      nodes, left child adjacent, (k, L) bookkeeping for the leaf number.  Every step first
//      issues the node fetches of all NT walks, then advances them without branches.
// A stage is released as soon as the warp has left the heaps, before it starts on part 2, so the
// next batch of heaps arrives while the warps wait for their node fetches.
// fp64 forests test against the float bound stored in the 8-byte node and read the exact
// threshold only when that bound cannot decide (x rounded down to float equals the bound).
#include "device_common.cuh"
#include "kernels_q.hpp"

namespace b2fil {
namespace {

constexpr int kCompactThreads = 800;  // 24 consumer warps + 1 producer warp at most

__device__ __forceinline__ void lds_node(uint32_t a, uint32_t& value, uint32_t& meta)
{
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(value), "=r"(meta) : "r"(a));
}

// How the walk below the heap fetches its nodes from global memory.  The fetches of a warp go to
// 32 unrelated cache lines and nothing is reused, so what matters is how many of them the SM can
// keep in flight; the L1 allocation policy of the load decides that.
enum NodeLoad : int { kLoadNc = 0, kLoadCg = 1, kLoadNoAllocate = 2 };
__device__ __forceinline__ uint2 ld_compact_node(const uint2* ptr, int kind)
{
  uint2 v;
  if (kind == kLoadCg) {
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

// Does the row go right at a compact node?  `exact_index()` yields the internal node whose exact
// threshold settles an fp64 test that the float bound leaves open (C_NO_NODE: none, heap padding).
template <typename T, bool CAT, typename ExactIndex>
__device__ __forceinline__ bool compact_goes_right(uint32_t value, uint32_t meta, T x,
                                                   const ForestView& f, ExactIndex exact_index)
{
  if constexpr (sizeof(T) == 4) {
    return goes_right<float, CAT, true>(value, meta, x, f);
  } else {
    if (CAT && (meta & META_CATEGORICAL))
      return goes_right<double, true, true>(static_cast<uint64_t>(value), meta, x, f);
    const float lo = __uint_as_float(value);  // largest float <= threshold
    bool left      = x < static_cast<double>(lo);
    if (!left && __double2float_rd(x) == lo) {
      // lo <= x < next float: only the exact threshold knows
      const uint32_t k = exact_index();
      if (k != C_NO_NODE) left = x < __ldg(f.c_exact + k);
    }
    if (x != x) left = (meta & META_DEFAULT_LEFT) != 0u;
    return !left;
  }
}

// Shared memory: [mbarriers 256 B][row tile][accumulators][16 B][S stages of G * NT heaps].
template <typename T, bool CAT, int MODE, int NT>
__global__ void __launch_bounds__(kCompactThreads, 1)
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

  const uint32_t stride_b    = (R + 1) * TR::ES;
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
  const uint32_t row_addr = tile + r * TR::ES;
  const CompactNode* __restrict__ nodes = f.c_nodes;
  RingPos pos;
  bool ok = true;
  for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const int64_t row0 = t * R;
    const int64_t row  = row0 + r;
    stage_rows<T>(p, tile, R, row0, warp, lane, n_cw);
    if (MODE <= MODE_VECTOR) {
      for (int i = threadIdx.x; i < G * NC * R; i += n_ct) acc[i] = T(0);
    }
    consumer_sync(n_ct);
    Running<T> run{T(0), 0};
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
            const T x = TR::ld_real((meta[kk] & CMETA_LOW28) * stride_b + row_addr);
            const bool right = compact_goes_right<T, CAT>(value[kk], meta[kk], x, f, [&]() {
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
        for (int step = 0; step < f.c_bottom_steps; ++step) {
          uint2 node[NT];
#pragma unroll
          for (int kk = 0; kk < NT; ++kk)
            node[kk] = ld_compact_node(reinterpret_cast<const uint2*>(nodes) + k[kk], node_load);
          bool walking = false;
#pragma unroll
          for (int kk = 0; kk < NT; ++kk) {
            const uint32_t value = node[kk].x, meta = node[kk].y;
            const T x = TR::ld_real((meta & feat_mask) * stride_b + row_addr);
            const uint32_t kx = k[kk];
            const bool right  = compact_goes_right<T, CAT>(value, meta, x, f, [&]() { return kx; });
            const uint32_t off = (meta & CMETA_LOW28) >> fb;
            const bool at_leaf = (meta & (right ? CMETA_RIGHT_LEAF : CMETA_LEFT_LEAF)) != 0u;
            if (live[kk]) {
              L[kk] += right ? off : 0u;
              if (!at_leaf) k[kk] += right ? off : 1u;
              live[kk] = !at_leaf;
            }
            walking |= live[kk];
          }
          if (!__any_sync(0xffffffffu, walking)) break;
        }
        // the leaves: payload (or id) from the leaf arrays
        if (MODE == MODE_LEAFID) {
          uint32_t id[NT];
#pragma unroll
          for (int kk = 0; kk < NT; ++kk) id[kk] = __ldg(f.c_leaf_ids + L[kk]);
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
          for (int kk = 0; kk < NT; ++kk) pay[kk] = __ldg(static_cast<const Val*>(f.c_leaf_payload) + L[kk]);
#pragma unroll
          for (int kk = 0; kk < NT; ++kk) {
            if (kk < n_act) take_leaf<T, MODE>(p, first + kk, pay[kk], 0u, acc_group, R, r, row, run);
          }
        }
      }
    }
    if (!ok) atomicExch(p.status, 2);
    if (MODE == MODE_SCALAR) acc_group[run.cls * R + r] += run.sum;
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
  b += align16(static_cast<size_t>(f.n_features) * (R + 1) * es);
  if (reduce) b += align16(static_cast<size_t>(G) * f.n_outputs * R * es);
  b += 16;
  b += static_cast<size_t>(S) * G * NT * static_cast<size_t>(f.c_top_stride);
  return b;
}

template <typename T, bool CAT, int MODE>
int launch_mode(const PredictParams& p, const CompactCfg& c, cudaStream_t stream, std::string& err)
{
  auto k       = sparse_compact_kernel<T, CAT, MODE, kCompactTreesInFlight>;
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
      R >= 32 && (R & (R - 1)) == 0 && R <= 128 && G >= 1 && (R / 32) * G <= 24 && S >= 1 &&
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
  // that stay under 150 KiB are preferred (measured: the same kernel runs twice as fast at
  // 110 KiB as at 216 KiB).  Within a limit: as many warps as fit, then a second stage.
  for (const size_t limit : {size_t(150) * 1024, kMaxSmemBytes}) {
    for (int R = rows_per_tile; R >= 32; R /= 2) {
      const int rw = R / 32;
      for (int G = std::min(24 / rw, std::max(1, (f.n_trees + kCompactTreesInFlight - 1) /
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
