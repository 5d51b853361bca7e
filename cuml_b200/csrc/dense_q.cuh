// Traversal kernels over rank-quantised rows (templates) and the helper that launches one
// instantiation.  Included by the kernels_q_*.cu translation units, each of which instantiates
// one family of these kernels, so that the families compile in parallel.
#pragma once

#include "device_common.cuh"
#include "kernels_q.hpp"

namespace b2fil {
namespace {

// ---------------------------------------------------------------------------------------------
// DENSE kernel on rank-quantised rows
// ---------------------------------------------------------------------------------------------
// Shared memory: [mbarriers 128 B][row tile F x R uint16][accumulators][flags 16 B][S tree stages].
// The row tile arrives with one bulk copy per tile (the pre-pass already stored it feature-major);
// tree batches stream through the stage ring exactly as in dense_kernel.  A node is 4 bytes
// (rank j << 17 | default-right << 16 | feature << 2 | categorical) and a test is one signed
// subtraction.
constexpr int kBarTileFull  = 2 * kMaxStages;      // mbarrier slots after the stage ring
constexpr int kBarTileEmpty = 2 * kMaxStages + 1;

// node - (q << 17) in one multiply-add: the sign of (j - rank) lands in bit 31.
__device__ __forceinline__ uint32_t rank_diff(uint32_t node, uint32_t q)
{
  static_assert(Q_RANK_SHIFT == 17, "the multiplier below is -(1 << Q_RANK_SHIFT)");
  uint32_t d;
  asm("mad.lo.u32 %0, %1, 0xFFFE0000, %2;" : "=r"(d) : "r"(q), "r"(node));
  return d;
}

// The three top nodes (heap words 1..3) of every tree, passed to the kernel by value: kernel
// parameters live in the constant bank, so the first two levels of every walk read their nodes
// through the constant cache and spend no shared-memory bandwidth, the resource that bounds the
// traversal (a warp reads the same tree in all lanes, so each lookup is one constant access).
struct QTop {
  uint32_t w[3 * kQTopTrees];
};

__device__ __forceinline__ uint2 lds_u32x2(uint32_t a)
{
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}

// DEPTH > 0 fixes the tree depth at compile time (the level loop is fully unrolled); DEPTH == 0
// reads it from the forest.  TOPC: the first two levels take their nodes from `top`.
// PAIR: the walk for launch shapes that shared memory keeps small (few warps, few trees in
// flight), where the latency of one step, not the shared-memory pipe, is the limit: both children
// of the current node (heap words 2i and 2i + 1, one aligned 8-byte load) are requested together
// with the row's rank, before the test is decided, so the next node is already there when the
// test is known; a step costs one shared-memory latency instead of two, and one more wavefront.
// LEAFG: the stages hold only the test nodes of the trees and a walk fetches its leaf payload from
// the forest image in global memory (L2).  Deep trees are half payloads (4 KB of 8 KB at depth
// 10); where shared memory next to the row tile holds only a dozen whole trees, leaving the
// payloads out doubles the walks in flight, which is what such shapes are bound by.  The payload
// fetch of a sub-batch is consumed one sub-batch later, behind the next walk.
template <typename T, int MODE, int NT, int DEPTH, bool CAT, bool TOPC, bool PAIR = false,
          bool LEAFG = false>
struct DenseQWalker {
  using TR = Traits<T>;
  // Walk the warp's 32 rows through all trees.  A stage of the ring holds K sub-batches of G * NT
  // trees; the warp waits once per stage and walks its NT trees of every sub-batch.
  template <bool NANS>
  static __device__ __forceinline__ bool walk(const PredictParams& p, int G, int S, int K, int g,
                                              int r, int64_t row, int lane, uint32_t bars,
                                              uint32_t stages, uint32_t stage_bytes,
                                              uint32_t row_addr, uint32_t stride_b, T* acc_group,
                                              int R, RingPos& pos, Running<T>& run,
                                              const QTop* top)
  {
    static_assert(!TOPC || (DEPTH >= 2 && !CAT), "top nodes need two plain levels");
    static_assert(!PAIR || (!CAT && !TOPC && MODE == MODE_SCALAR && sizeof(T) == 4),
                  "the child-pair walk exists for fp32 scalar leaves without categorical tests");
    static_assert(!LEAFG || (!CAT && !PAIR && MODE == MODE_SCALAR && sizeof(T) == 4),
                  "payloads outside the stages exist for fp32 scalar leaves without categorical tests");
    const ForestView& f    = p.f;
    const int D            = DEPTH > 0 ? DEPTH : f.dense_depth;
    constexpr uint32_t QNB = CAT ? 8u : 4u;  // bytes per test node: {node, category set} or node
    const uint32_t width_b = (1u << D) * QNB;
    // bytes between two trees of a stage
    const uint32_t tstride = LEAFG ? width_b : static_cast<uint32_t>(f.q_tree_stride);
    // bytes per leaf payload: the element size, except where vector leaves sit in the tree block
    const uint32_t lbytes  = MODE == MODE_SCALAR ? TR::ES : static_cast<uint32_t>(f.q_leaf_bytes);
    const bool inline_vec  = MODE != MODE_SCALAR && lbytes > TR::ES;
    const uint32_t fstride = stride_b >> Q_FEATURE_SHIFT;  // R / 2 <= 128: fits a byte
    const int per_sub      = G * NT;
    const int per_batch    = per_sub * K;
    const int n_batches    = (f.n_trees + per_batch - 1) / per_batch;
    const uint32_t mine    = static_cast<uint32_t>(g * NT) * tstride;  // this warp's trees in a sub-batch
    const uint32_t sub_b   = static_cast<uint32_t>(per_sub) * tstride;
    bool ok                = true;

    // LEAFG: payloads requested by the previous sub-batch, not yet added
    uint32_t pend[NT] = {};
    int pend_first = 0, pend_n = 0;
    auto take_pending = [&]() {
#pragma unroll
      for (int k = 0; k < NT; ++k) {
        if (k < pend_n) take_leaf<T, MODE>(p, pend_first + k, pend[k], 0u, acc_group, R, r, row, run);
      }
      pend_n = 0;
    };
    // One sub-batch: NT trees side by side.  FULL means all NT slots hold live trees, which lets
    // the compiler drop every per-slot guard.
    auto sub_batch = [&](auto full_tag, uint32_t base0, int first, int n_act) {
      constexpr bool FULL = decltype(full_tag)::value;
      uint32_t base[NT], idx[NT], a[NT];
#pragma unroll
      for (int k = 0; k < NT; ++k) {
        // slots past the end of the forest repeat the last live tree; results are dropped
        base[k] = base0 + static_cast<uint32_t>(FULL ? k : min(k, n_act - 1)) * tstride;
        idx[k]  = 1u;  // heap index of the root
        a[k]    = base[k] + QNB;
      }
      // the NT walks are independent: all node loads are issued first, then all rank loads,
      // so that their shared-memory latencies overlap inside one warp.
      // test(): the rows' ranks against NT nodes; the sign bit of d[k] is the step to the right.
      auto test = [&](const uint32_t(&node)[NT], const uint32_t(&bits)[CAT ? NT : 1], uint32_t(&d)[NT]) {
        uint32_t q[NT];
#pragma unroll
        for (int k = 0; k < NT; ++k)
          // the low half of a node is feature * 4: one dot-product instruction (low half x byte 0
          // of fstride, high half x byte 1 = 0) turns it into the address of the row's rank of
          // that feature
          q[k] = lds_u16(__dp2a_lo(node[k], fstride, row_addr));
#pragma unroll
        for (int k = 0; k < NT; ++k) {
          // rank j in the high half: x < T[j] <=> rank(x) <= j, so right <=> j - rank < 0
          d[k] = rank_diff(node[k], q[k]);
          if (CAT) {
            // the code of a categorical value is its category and the node's set (fetched with
            // the node; numerical nodes hold an empty one) is stored bit-reversed: the clamped
            // funnel shift by the code moves the category's bit to the sign position and yields 0
            // for every code of 32 and above (no category, NaN).  A categorical node carries the
            // largest rank (its comparison never says "right"), so the two answers are simply
            // ORed and the walk has no data-dependent branch.
            d[k] |= __funnelshift_lc(0u, bits[k], q[k]);
          }
          if (NANS) {
            // the missing-goes-right flag sits 15 bits below the sign.  (Both forms compute the
            // same; each kernel family keeps the one it was measured fastest with: the two walks
            // of a kernel share its register allocation.)
            if (CAT) {
              if (q[k] == Q_NAN_CODE) d[k] = node[k] << 15;
            } else {
              if (q[k] == Q_NAN_CODE) d[k] = (node[k] & Q_DEFAULT_RIGHT) ? 0x80000000u : 0u;
            }
          }
        }
      };
      auto level = [&]() {
        uint32_t node[NT], d[NT], bits[CAT ? NT : 1];
#pragma unroll
        for (int k = 0; k < NT; ++k) {
          if (CAT) {
            const uint2 both = lds_u32x2(a[k]);
            node[k]          = both.x;
            bits[k]          = both.y;
          } else {
            node[k] = lds_u32(a[k]);
          }
        }
        test(node, bits, d);
#pragma unroll
        for (int k = 0; k < NT; ++k) {
          // heap index 2i + right in one funnel shift: (i << 1) | (d >> 31)
          idx[k] = __funnelshift_l(d[k], idx[k], 1);
          a[k]   = idx[k] * QNB + base[k];
        }
      };
      const uint32_t no_bits[1] = {0u};  // walks without categorical tests
      if constexpr (PAIR) {
        uint32_t node[NT], d[NT];
#pragma unroll
        for (int k = 0; k < NT; ++k) node[k] = lds_u32(a[k]);  // the root
#pragma unroll 2
        for (int lvl = 0; lvl < D; ++lvl) {
          // children of node i are heap words 2i and 2i + 1; below the last level these are the
          // two leaf payloads (4-byte payloads continue the heap)
          uint2 pair[NT];
#pragma unroll
          for (int k = 0; k < NT; ++k) pair[k] = lds_u32x2(base[k] + idx[k] * 8u);
          test(node, reinterpret_cast<const uint32_t(&)[CAT ? NT : 1]>(no_bits), d);
#pragma unroll
          for (int k = 0; k < NT; ++k) {
            idx[k]  = __funnelshift_l(d[k], idx[k], 1);
            node[k] = static_cast<int32_t>(d[k]) < 0 ? pair[k].y : pair[k].x;
          }
        }
#pragma unroll
        for (int k = 0; k < NT; ++k) {
          if (FULL || k < n_act)
            take_leaf<T, MODE>(p, first + k, node[k], 0u, acc_group, R, r, row, run);
        }
        return;
      }
      if (TOPC) {
        // root and children from the constant bank: the same words in every lane
        uint32_t n1[NT], n2[NT], n3[NT], node[NT], d[NT];
#pragma unroll
        for (int k = 0; k < NT; ++k) {
          const int t = 3 * (first + (FULL ? k : min(k, n_act - 1)));
          n1[k]       = top->w[t];
          n2[k]       = top->w[t + 1];
          n3[k]       = top->w[t + 2];
        }
        test(n1, reinterpret_cast<const uint32_t(&)[CAT ? NT : 1]>(no_bits), d);
#pragma unroll
        for (int k = 0; k < NT; ++k) {
          node[k] = static_cast<int32_t>(d[k]) < 0 ? n3[k] : n2[k];
          idx[k]  = __funnelshift_l(d[k], 1u, 1);
        }
        test(node, reinterpret_cast<const uint32_t(&)[CAT ? NT : 1]>(no_bits), d);
#pragma unroll
        for (int k = 0; k < NT; ++k) {
          idx[k] = __funnelshift_l(d[k], idx[k], 1);
          a[k]   = idx[k] * 4u + base[k];
        }
      }
      if (DEPTH > 0) {
#pragma unroll
        for (int lvl = TOPC ? 2 : 0; lvl < DEPTH; ++lvl) level();
      } else {
#pragma unroll 4
        for (int lvl = 0; lvl < D; ++lvl) level();
      }
      if constexpr (LEAFG) {
        // add the payloads that the previous sub-batch requested (they arrived during this
        // walk), then request this sub-batch's; nothing touches them until the next one is done
        take_pending();
        const unsigned char* image = static_cast<const unsigned char*>(f.q_nodes) + width_b;
#pragma unroll
        for (int k = 0; k < NT; ++k) {
          const uint32_t slot = idx[k] - (1u << D);
          const int tree      = first + (FULL ? k : min(k, n_act - 1));
          pend[k] = __ldg(reinterpret_cast<const uint32_t*>(
            image + static_cast<size_t>(tree) * static_cast<size_t>(f.q_tree_stride) + slot * 4u));
        }
        pend_first = first;
        pend_n     = FULL ? NT : n_act;
        return;
      }
      // scalar leaves of a multi-class forest: trees are stored class by class, so when the
      // first and the last tree of the sub-batch feed the class of the running sum, all do
      bool same_class = false;
      if (MODE == MODE_SCALAR && CAT) {
        same_class = f.n_outputs == 1 ||
                     (__ldg(f.tree_class + first) == run.cls &&
                      __ldg(f.tree_class + first + n_act - 1) == run.cls);
      }
      if (MODE >= MODE_PERTREE) {
        // One output per (row, tree).  The payload slot holds what is reported: the leaf value,
        // or the leaf id when the CTA streams the image made for that (MODE_LEAFID).  With four
        // live trees that are also the caller's trees first..first+3, a row's four outputs are
        // contiguous and leave as 16-byte stores: scalar 4-byte stores at a stride of a whole
        // output row cost one sector request each and bound these predictions otherwise.
        typename TR::Val val[NT];
        uint32_t leaf_at[NT];
#pragma unroll
        for (int k = 0; k < NT; ++k) {
          const uint32_t slot = idx[k] - (1u << D);
          leaf_at[k]          = base[k] + width_b + slot * lbytes;
          val[k]              = TR::ld_val(leaf_at[k]);
        }
        const bool scalar_out = MODE == MODE_LEAFID || f.leaf_vector_len <= 1;
        const bool wide = FULL && NT == 4 && scalar_out && f.q_trees_in_order != 0 &&
                          (f.n_trees & 3) == 0 &&
                          (reinterpret_cast<uintptr_t>(p.out) & 15u) == 0;
        if (wide) {
          if (row < p.n_rows) {
            if (MODE == MODE_LEAFID || TR::ES == 4) {
              uint32_t* dst = static_cast<uint32_t*>(p.out) + row * f.n_trees + first;
              *reinterpret_cast<uint4*>(dst) =
                make_uint4(TR::low32(val[0]), TR::low32(val[NT > 1 ? 1 : 0]),
                           TR::low32(val[NT > 2 ? 2 : 0]), TR::low32(val[NT > 3 ? 3 : 0]));
            } else {
              uint64_t* dst = static_cast<uint64_t*>(p.out) + row * f.n_trees + first;
              *reinterpret_cast<ulonglong2*>(dst) =
                make_ulonglong2(val[0], val[NT > 1 ? 1 : 0]);
              *reinterpret_cast<ulonglong2*>(dst + 2) =
                make_ulonglong2(val[NT > 2 ? 2 : 0], val[NT > 3 ? 3 : 0]);
            }
          }
        } else {
#pragma unroll
          for (int k = 0; k < NT; ++k) {
            if (FULL || k < n_act) {
              if (MODE == MODE_LEAFID) {
                if (row < p.n_rows) {
                  const int orig = __ldg(f.tree_orig + first + k);
                  static_cast<uint32_t*>(p.out)[row * f.n_trees + orig] = TR::low32(val[k]);
                }
              } else if (inline_vec) {
                // per-tree outputs of vector leaves that sit in the tree block
                if (row < p.n_rows) {
                  const int orig = __ldg(f.tree_orig + first + k);
                  T* out = static_cast<T*>(p.out) + (row * f.n_trees + orig) * f.n_outputs;
                  for (int c = 0; c < f.n_outputs; ++c) out[c] = TR::ld_real(leaf_at[k] + c * TR::ES);
                }
              } else {
                take_leaf<T, MODE>(p, first + k, val[k], 0u, acc_group, R, r, row, run);
              }
            }
          }
        }
      } else {
#pragma unroll
        for (int k = 0; k < NT; ++k) {
          if (FULL || k < n_act) {
            // the leaf payloads follow the 2^D node words: for 4-byte payloads the heap
            // address of leaf slot j is exactly the address the walk ended on
            const uint32_t slot   = idx[k] - (1u << D);
            const uint32_t leaf_a = (MODE == MODE_SCALAR && TR::ES == 4 && !CAT)
                                      ? a[k]
                                      : base[k] + width_b + slot * lbytes;
            if (MODE == MODE_VECTOR && inline_vec) {
              // the leaf's vector sits in the tree block: one sum per output, in registers
#pragma unroll
              for (int c = 0; c < kRegClasses; ++c) {
                if (c < f.n_outputs) run.v[c] += TR::ld_real(leaf_a + c * TR::ES);
              }
              continue;
            }
            const typename TR::Val payload = TR::ld_val(leaf_a);
            if (MODE == MODE_SCALAR && CAT && same_class) {
              run.sum += TR::as_real(payload);
            } else {
              take_leaf<T, MODE>(p, first + k, payload, 0u, acc_group, R, r, row, run);
            }
          }
        }
      }
    };

    for (int b = 0; b < n_batches; ++b) {
      const uint32_t s = pos.stage;
      if (ok) ok = mbar_wait(bars + 8u * s, pos.phase);
      if (ok) {
        uint32_t base0 = stages + s * stage_bytes + mine;
        int first      = b * per_batch + g * NT;  // first tree of this warp inside the stage
        for (int kk = 0; kk < K; ++kk, base0 += sub_b, first += per_sub) {
          const int n_act = f.n_trees - first;
          if (n_act >= NT) {
            sub_batch(std::true_type{}, base0, first, NT);
          } else if (n_act > 0) {
            sub_batch(std::false_type{}, base0, first, n_act);
          } else {
            break;
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8u * (kMaxStages + s));
      pos.advance(S);
    }
    if constexpr (LEAFG) take_pending();
    return ok;
  }
};

template <typename T, int MODE, int NT, int DEPTH, bool CAT, bool TOPC, bool PAIR = false,
          bool LEAFG = false>
__device__ __forceinline__ void dense_q_body(const PredictParams& p, const uint16_t* __restrict__ Q,
                                             const int32_t* __restrict__ tile_flags, const int R,
                                             const int G, const int S, const int K,
                                             const QTop* top)
{
  using TR = Traits<T>;
  extern __shared__ __align__(128) unsigned char smem[];
  const ForestView& f = p.f;
  const int F         = f.n_features;
  const int NC        = f.n_outputs;
  const int rw        = R >> 5;
  const int n_cw      = rw * G;
  const int n_ct      = n_cw * 32;
  const int warp      = threadIdx.x >> 5;
  const int lane      = threadIdx.x & 31;

  const uint32_t stride_b    = R * 2u;  // bytes between features in the tile
  const uint32_t tile_bytes  = static_cast<uint32_t>(F) * stride_b;  // multiple of 64
  const size_t acc_bytes     = (MODE <= MODE_VECTOR) ? align16(static_cast<size_t>(G) * NC * R * TR::ES) : 0;
  unsigned char* tile_ptr    = smem + kBarBytes;
  T* acc                     = reinterpret_cast<T*>(tile_ptr + tile_bytes);
  unsigned char* stage_ptr   = tile_ptr + tile_bytes + acc_bytes + 16;
  const uint32_t bars        = smem_addr(smem);
  const uint32_t tile        = smem_addr(tile_ptr);
  const uint32_t stages      = smem_addr(stage_ptr);
  const uint32_t gstride     = static_cast<uint32_t>(f.q_tree_stride);  // trees in the forest image
  // trees in a stage: whole, or (LEAFG) only their 2^depth test nodes
  const uint32_t tstride     = LEAFG ? (4u << (DEPTH > 0 ? DEPTH : f.dense_depth)) : gstride;
  const int per_batch        = G * NT * K;
  const uint32_t stage_bytes = per_batch * tstride;
  const int n_batches        = (f.n_trees + per_batch - 1) / per_batch;
  const int64_t n_tiles      = (p.n_rows + R - 1) / R;
  const uint32_t bar_tfull   = bars + 8u * kBarTileFull;
  const uint32_t bar_tempty  = bars + 8u * kBarTileEmpty;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bars + 8u * s, 1);
      mbar_init(bars + 8u * (kMaxStages + s), n_cw);
    }
    mbar_init(bar_tfull, 1);
    mbar_init(bar_tempty, n_cw);
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == n_cw) {
    // ---- producer: row tile, then the tree batches of that tile ------------------------------
    if (lane == 0) {
      // predictions that report leaves stream the image whose payload slots hold the leaf ids
      const unsigned char* src  = static_cast<const unsigned char*>(
        MODE == MODE_LEAFID ? f.q_nodes_ids : f.q_nodes);
      const unsigned char* qsrc = reinterpret_cast<const unsigned char*>(Q);
      RingPos pos;
      bool primed               = false;  // every stage has been filled once
      uint32_t n_done           = 0;
      for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x, ++n_done) {
        // the tile buffer is free once every consumer warp has left the previous tile's trees
        if (n_done > 0 && !mbar_wait(bar_tempty, (n_done - 1) & 1u)) {
          atomicExch(p.status, 3);
          return;
        }
        mbar_expect_tx(bar_tfull, tile_bytes);
        bulk_copy_g2s(tile, qsrc + static_cast<size_t>(t) * tile_bytes, tile_bytes, bar_tfull);
        for (int b = 0; b < n_batches; ++b) {
          const uint32_t s = pos.stage;
          if (primed && !mbar_wait(bars + 8u * (kMaxStages + s), pos.phase ^ 1u)) {
            atomicExch(p.status, 1);
            return;
          }
          const int first      = b * per_batch;
          const int count      = min(per_batch, f.n_trees - first);
          const uint32_t bytes = count * tstride;
          mbar_expect_tx(bars + 8u * s, bytes);
          if (LEAFG) {
            // one copy per tree: the node half of its block
            for (int i = 0; i < count; ++i)
              bulk_copy_g2s(stages + s * stage_bytes + i * tstride,
                            src + static_cast<size_t>(first + i) * gstride, tstride, bars + 8u * s);
          } else {
            bulk_copy_g2s(stages + s * stage_bytes, src + static_cast<size_t>(first) * gstride,
                          bytes, bars + 8u * s);
          }
          pos.advance(S);
          if (pos.stage == 0) primed = true;
        }
      }
    }
    return;
  }

  // ---- consumers ------------------------------------------------------------------------------
  const int g             = warp / rw;
  const int r             = (warp % rw) * 32 + lane;
  T* acc_group            = acc + static_cast<size_t>(g) * NC * R;
  const uint32_t row_addr = tile + q_slot(r, R) * 2u;
  RingPos pos;
  uint32_t n_done         = 0;
  bool ok                 = true;
  for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x, ++n_done) {
    const int64_t row0 = t * R;
    if (MODE <= MODE_VECTOR) {
      for (int i = threadIdx.x; i < G * NC * R; i += n_ct) acc[i] = T(0);
    }
    const bool nans = __ldg(tile_flags + t) != 0;
    consumer_sync(n_ct);
    if (ok) ok = mbar_wait(bar_tfull, n_done & 1u);
    Running<T> run{T(0), 0, {}};
    if (ok) {
      if (nans) {
        ok = DenseQWalker<T, MODE, NT, DEPTH, CAT, TOPC, PAIR, LEAFG>::template walk<true>(
          p, G, S, K, g, r, row0 + r, lane, bars, stages, stage_bytes, row_addr, stride_b,
          acc_group, R, pos, run, top);
      } else {
        ok = DenseQWalker<T, MODE, NT, DEPTH, CAT, TOPC, PAIR, LEAFG>::template walk<false>(
          p, G, S, K, g, r, row0 + r, lane, bars, stages, stage_bytes, row_addr, stride_b,
          acc_group, R, pos, run, top);
      }
      if (!ok) atomicExch(p.status, 2);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_tempty);
    flush_running<T, MODE>(f, run, acc_group, R, r);
    consumer_sync(n_ct);
    if (MODE <= MODE_VECTOR) {
      if (threadIdx.x < R) finish_row<T>(p, acc, R, G, threadIdx.x, row0 + threadIdx.x);
    }
    consumer_sync(n_ct);
  }
}


template <typename T, int MODE, int NT, int DEPTH, bool CAT>
__global__ void __launch_bounds__(NT > 4 ? 800 : 1024, 1)
dense_q_kernel(const PredictParams p, const uint16_t* __restrict__ Q,
               const int32_t* __restrict__ tile_flags, const int R, const int G, const int S,
               const int K)
{
  dense_q_body<T, MODE, NT, DEPTH, CAT, false>(p, Q, tile_flags, R, G, S, K, nullptr);
}

// Same kernel with the child-pair walk (see DenseQWalker).
template <int NT>
__global__ void __launch_bounds__(1024, 1)
dense_q_pair_kernel(const PredictParams p, const uint16_t* __restrict__ Q,
                    const int32_t* __restrict__ tile_flags, const int R, const int G, const int S,
                    const int K)
{
  dense_q_body<float, MODE_SCALAR, NT, 0, false, false, true>(p, Q, tile_flags, R, G, S, K, nullptr);
}

// Same kernel with the leaf payloads left in global memory (see DenseQWalker).
template <int NT, int DEPTH>
__global__ void __launch_bounds__(1024, 1)
dense_q_leafg_kernel(const PredictParams p, const uint16_t* __restrict__ Q,
                     const int32_t* __restrict__ tile_flags, const int R, const int G, const int S,
                     const int K)
{
  dense_q_body<float, MODE_SCALAR, NT, DEPTH, false, false, false, true>(p, Q, tile_flags, R, G, S,
                                                                         K, nullptr);
}

// Same kernel with the top nodes of every tree in the parameter block.
template <typename T, int MODE, int NT, int DEPTH>
__global__ void __launch_bounds__(NT > 4 ? 800 : 1024, 1)
dense_q_top_kernel(const __grid_constant__ PredictParams p, const uint16_t* __restrict__ Q,
                   const int32_t* __restrict__ tile_flags, const int R, const int G, const int S,
                   const int K, const __grid_constant__ QTop top)
{
  dense_q_body<T, MODE, NT, DEPTH, false, true>(p, Q, tile_flags, R, G, S, K, &top);
}

// Launch one instantiation of dense_q_kernel.
template <typename T, int MODE, int NT, int DEPTH, bool CAT>
int launch_q(const QLaunch& L, std::string& err)
{
  auto k = dense_q_kernel<T, MODE, NT, DEPTH, CAT>;
  const int rc = set_smem_bytes(reinterpret_cast<const void*>(k), L.c.smem_bytes, err);
  if (rc != B2FIL_OK) return rc;
  k<<<L.grid, L.c.threads, L.c.smem_bytes, L.stream>>>(L.p, L.Q, L.flags, L.c.rows_per_tile,
                                                       L.c.tree_groups, L.c.stages,
                                                       L.c.sub_batches);
  return B2FIL_OK;
}

// One case per output mode of the generic-depth kernels.
template <typename T, int NT, bool CAT>
int launch_q_modes(const QLaunch& L, int mode, std::string& err)
{
  switch (mode) {
    case MODE_SCALAR: return launch_q<T, MODE_SCALAR, NT, 0, CAT>(L, err);
    case MODE_VECTOR: return launch_q<T, MODE_VECTOR, NT, 0, CAT>(L, err);
    case MODE_PERTREE: return launch_q<T, MODE_PERTREE, NT, 0, CAT>(L, err);
    default: return launch_q<T, MODE_LEAFID, NT, 0, CAT>(L, err);
  }
}

}  // namespace
}  // namespace b2fil
