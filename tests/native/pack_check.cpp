// Test-only host walker over a PACKED forest (the arrays the kernels read), used by the CPU test
// suite to check the packer without a GPU: it links cuml_b200/csrc/pack.cpp directly, packs a
// description and follows the packed nodes with the same index arithmetic as the kernels
// (heap addressing for dense storage, child offsets and bit fields for sparse storage).
// It is not part of libb2fil.so.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <string>
#include <vector>

#include "../../cuml_b200/csrc/forest.hpp"

using namespace b2fil;

namespace {
int always_dense(int depth, int, int, int) { return depth <= 16 ? 1 : 0; }
std::string g_err;

template <typename T, typename V>
bool goes_right(V value, uint32_t meta, T x, const PackedForest& pf)
{
  T thr;
  std::memcpy(&thr, &value, sizeof(T));
  bool left = x < thr;
  if (meta & META_CATEGORICAL) {
    const bool in_range = (x >= T(0)) && (x < T(16777216));
    const uint32_t c    = in_range ? static_cast<uint32_t>(x) : 0u;
    const uint32_t low  = static_cast<uint32_t>(value);
    bool matched        = false;
    if (pf.view.cat_inline) {
      matched = in_range && c < 32u && ((low >> (c & 31u)) & 1u);
    } else {
      const uint32_t n_words = pf.cat_pool[low];
      const uint32_t w       = c >> 5;
      if (in_range && w < n_words) matched = (pf.cat_pool[low + 1 + w] >> (c & 31u)) & 1u;
    }
    left = !matched;
  }
  if (x != x) left = (meta & META_DEFAULT_LEFT) != 0;
  return !left;
}

template <typename T>
void walk(const PackedForest& pf, const T* X, int64_t n_rows, int64_t stride, uint32_t* ids,
          double* payload)
{
  const ForestView& v = pf.view;
  using V             = typename std::conditional<sizeof(T) == 4, uint32_t, uint64_t>::type;
  for (int64_t r = 0; r < n_rows; ++r) {
    const T* row = X + r * stride;
    for (int p = 0; p < v.n_trees; ++p) {
      const int orig = pf.tree_orig[p];
      uint32_t id;
      V pay;
      if (v.format == FMT_DENSE_F || v.format == FMT_DENSE_D) {
        const size_t nb  = sizeof(T) == 4 ? 8 : 16;
        const int D      = v.dense_depth;
        const uint8_t* t = pf.nodes.data() + static_cast<size_t>(v.tree_stride) * p;
        uint32_t i       = 1;
        for (int l = 0; l < D; ++l) {
          V value;
          uint32_t meta;
          std::memcpy(&value, t + i * nb, sizeof(V));
          std::memcpy(&meta, t + i * nb + sizeof(V), 4);
          const uint32_t feat = meta & 0x3FFFFFFFu;
          i = 2 * i + (goes_right<T, V>(value, meta, row[feat], pf) ? 1 : 0);
        }
        const uint32_t slot = i - (1u << D);
        std::memcpy(&pay, t + (size_t(1) << D) * nb + slot * sizeof(T), sizeof(V));
        id = pf.leaf_ids[(static_cast<size_t>(p) << D) + slot];
      } else {
        uint32_t idx = pf.roots[p];
        for (;;) {
          V value;
          uint32_t meta, offset, feat;
          if (v.format == FMT_SPARSE_8) {
            SparseNode8 n;
            std::memcpy(&n, pf.nodes.data() + size_t(idx) * 8, 8);
            value  = n.value;
            meta   = n.meta;
            offset = (n.meta & META_LOW29) >> v.feat_bits;
            feat   = n.meta & ((1u << v.feat_bits) - 1u);
          } else if (v.format == FMT_SPARSE_16F) {
            SparseNode16F n;
            std::memcpy(&n, pf.nodes.data() + size_t(idx) * 16, 16);
            value  = n.value;
            meta   = n.meta;
            offset = n.offset;
            feat   = n.meta & META_LOW29;
          } else {
            SparseNode16D n;
            std::memcpy(&n, pf.nodes.data() + size_t(idx) * 16, 16);
            value  = static_cast<V>(n.value);
            meta   = n.meta;
            offset = n.offset;
            feat   = n.meta & META_LOW29;
          }
          if (meta & META_LEAF) {
            pay = value;
            id  = pf.leaf_ids[idx];
            break;
          }
          const bool right = goes_right<T, V>(value, meta, row[feat], pf);
          idx += (v.layout == B2FIL_LAYOUT_DEPTH_FIRST) ? (right ? offset : 1u)
                                                         : (offset + (right ? 1u : 0u));
        }
      }
      ids[r * v.n_trees + orig] = id;
      if (v.leaf_vector_len > 1) {
        payload[r * v.n_trees + orig] = static_cast<double>(static_cast<uint32_t>(pay));
      } else {
        T val;
        std::memcpy(&val, &pay, sizeof(T));
        payload[r * v.n_trees + orig] = static_cast<double>(val);
      }
    }
  }
}
// Walk the rank-quantised copy of a dense forest the way quantise_kernel + dense_q_kernel do:
// rank through the bucket table, then one signed subtraction per test.  Returns the number of
// (row, tree) pairs whose leaf differs from `ids`.
template <typename T>
int64_t walk_quantised(const PackedForest& pf, const T* X, int64_t n_rows, int64_t stride,
                       const uint32_t* ids)
{
  const ForestView& v = pf.view;
  const int D         = v.dense_depth;
  const int F         = v.n_features;
  std::vector<uint16_t> q(F);
  int64_t bad = 0;
  for (int64_t r = 0; r < n_rows; ++r) {
    const T* row = X + r * stride;
    for (const QGroup& g : pf.q_groups) {
      const uint8_t* blob = pf.q_blob.data() + g.blob_off;
      for (uint32_t f = g.f_begin; f < g.f_end; ++f) {
        QFeatRec rec;
        std::memcpy(&rec, blob + (f - g.f_begin) * sizeof(QFeatRec), sizeof(rec));
        const T x = row[f];
        if (x != x) {
          q[f] = Q_NAN_CODE;
          continue;
        }
        if (rec.is_cat) {  // the code of a categorical value is its category
          const bool in_range = (x >= T(0)) && (x < T(Q_NO_CATEGORY));
          q[f] = in_range ? static_cast<uint16_t>(static_cast<uint32_t>(x)) : Q_NO_CATEGORY;
          continue;
        }
        const uint32_t b = q_bucket_host<T>(x, static_cast<T>(rec.scale),
                                            static_cast<T>(rec.offset), rec.nbm1 + 1);
        // both tables are interleaved across the group's GF features
        const size_t GF = g.f_end - g.f_begin;
        uint16_t lo16;
        std::memcpy(&lo16, blob + rec.lut_off + b * GF * 2, 2);
        uint32_t pos = lo16;
        for (uint32_t s2 = (1u << g.steps) >> 1; s2 >= 1; s2 >>= 1) {
          T thr;
          std::memcpy(&thr, blob + rec.thr_off + (pos + s2 - 1) * GF * sizeof(T), sizeof(T));
          if (thr <= x) pos += s2;
        }
        q[f] = static_cast<uint16_t>(pos);
      }
    }
    for (int p = 0; p < v.n_trees; ++p) {
      const uint8_t* t = pf.q_nodes.data() + static_cast<size_t>(v.q_tree_stride) * p;
      const size_t qnb = pf.view.q_has_cat ? 8 : 4;  // {node, category set} or node alone
      uint32_t i       = 1;
      for (int l = 0; l < D; ++l) {
        uint32_t node;
        std::memcpy(&node, t + i * qnb, 4);
        const uint32_t qq = q[(node & Q_FEATURE_FIELD) >> Q_FEATURE_SHIFT];
        bool right = static_cast<int32_t>(node - (qq << Q_RANK_SHIFT)) < 0;
        if (pf.view.q_has_cat) {
          // the kernel's arithmetic: OR of the rank comparison (never "right" on a categorical
          // node) and the bit-reversed category set shifted left by the code (0 from 32 up)
          uint32_t bits;
          std::memcpy(&bits, t + i * qnb + 4, 4);
          const uint32_t shifted = qq < 32u ? bits << qq : 0u;
          right = right || (shifted >> 31) != 0u;
          // numerical nodes hold empty sets (a categorical node carries the largest rank)
          if ((node >> Q_RANK_SHIFT) != Q_MAX_RANK_FIELD && bits != 0u) ++bad;
        }
        if (qq == Q_NAN_CODE) right = (node & Q_DEFAULT_RIGHT) != 0u;
        i = 2 * i + (right ? 1 : 0);
      }
      const uint32_t slot = i - (1u << D);
      const uint32_t id   = pf.leaf_ids[(static_cast<size_t>(p) << D) + slot];
      if (id != ids[r * v.n_trees + pf.tree_orig[p]]) ++bad;
      // the image that reports leaves holds the same id in the payload slot
      const size_t lbytes = static_cast<size_t>(v.q_leaf_bytes);
      uint32_t id2;
      std::memcpy(&id2, pf.q_nodes_ids.data() + static_cast<size_t>(v.q_tree_stride) * p +
                          (size_t(1) << D) * qnb + slot * lbytes, 4);
      if (id2 != id) ++bad;
      if (lbytes > sizeof(T)) {
        // vector leaves stored in the tree block: the same values as the forest's vector table
        const uint8_t* dense_leaf = pf.nodes.data() + static_cast<size_t>(v.tree_stride) * p +
                                    (size_t(1) << D) * (sizeof(T) == 4 ? 8 : 16) + slot * sizeof(T);
        uint32_t vi;
        std::memcpy(&vi, dense_leaf, 4);
        if (std::memcmp(t + (size_t(1) << D) * qnb + slot * lbytes,
                        pf.leaf_vectors.data() + static_cast<size_t>(vi) * v.n_outputs * sizeof(T),
                        lbytes) != 0)
          ++bad;
      }
    }
  }
  return bad;
}
// Walk the compact image of a sparse forest the way the fast sparse kernel does: T steps through
// the tree's heap, leave through an exit, then (k, L) steps over the 8-byte internal nodes; fp64
// tests look the exact threshold up only when the float bound leaves the answer open.  Returns
// the number of (row, tree) pairs whose leaf id or payload differs from the primary walk, and
// counts the exact look-ups in *n_exact.
template <typename T>
int64_t walk_compact(const PackedForest& pf, const T* X, int64_t n_rows, int64_t stride,
                     const uint32_t* ids, const double* payload, int64_t* n_exact)
{
  const ForestView& v = pf.view;
  using V             = typename std::conditional<sizeof(T) == 4, uint32_t, uint64_t>::type;
  const int TL        = v.c_top_levels;
  const size_t heap_n = size_t(1) << TL;
  const int fb        = v.c_feat_bits;
  int64_t bad         = 0;
  auto test = [&](uint32_t value, uint32_t meta, T x, uint32_t k) -> bool {
    if (meta & META_CATEGORICAL) return goes_right<T, V>(static_cast<V>(value), meta, x, pf);
    bool left;
    if (sizeof(T) == 4) {
      float thr;
      std::memcpy(&thr, &value, 4);
      left = x < static_cast<T>(thr);
    } else {
      float lo;
      std::memcpy(&lo, &value, 4);
      left = static_cast<double>(x) < static_cast<double>(lo);
      if (!left && k != C_NO_NODE) {
        // x rounded down to float
        float xf = static_cast<float>(x);
        if (static_cast<double>(xf) > static_cast<double>(x))
          xf = std::nextafter(xf, -std::numeric_limits<float>::infinity());
        if (xf == lo) {
          ++*n_exact;
          left = static_cast<double>(x) < pf.c_exact[k];
        }
      }
    }
    if (x != x) left = (meta & META_DEFAULT_LEFT) != 0;
    return !left;
  };
  for (int64_t r = 0; r < n_rows; ++r) {
    const T* row = X + r * stride;
    for (int p = 0; p < v.n_trees; ++p) {
      const uint8_t* top = pf.c_top.data() + static_cast<size_t>(v.c_top_stride) * p;
      uint32_t h         = 1;
      for (int l = 0; l < TL; ++l) {
        uint32_t value, meta;
        std::memcpy(&value, top + h * 8, 4);
        std::memcpy(&meta, top + h * 8 + 4, 4);
        const uint32_t feat = meta & CMETA_LOW27;
        const uint32_t src  = pf.c_top_src.empty() ? C_NO_NODE : pf.c_top_src[p * heap_n + h];
        h = 2 * h + (test(value, meta, row[feat], src) ? 1 : 0);
      }
      uint32_t exit[2];
      std::memcpy(exit, top + size_t(h) * 8, 8);  // exit e follows the 2^T node slots
      uint32_t leaf;
      if (exit[0] & C_EXIT_LEAF) {
        leaf = exit[0] & ~C_EXIT_LEAF;
      } else {
        uint32_t k = exit[0], L = exit[1];
        if (L != pf.c_leaves_before[k]) ++bad;
        int steps  = 0;
        for (;;) {
          if (++steps > v.c_bottom_steps) {
            ++bad;  // the kernel's loop bound would have cut this walk short
          }
          const uint32_t value = pf.c_nodes[size_t(k) * 2], meta = pf.c_nodes[size_t(k) * 2 + 1];
          const uint32_t feat  = meta & ((1u << fb) - 1u);
          const uint32_t off   = (meta & CMETA_LOW27) >> fb;
          const bool right     = test(value, meta, row[feat], k);
          // the first child (adjacent) is the left one unless the node says otherwise
          const bool second    = right != ((meta & CMETA_SWAPPED) != 0);
          bool at_leaf;
          if (second) {
            at_leaf = (meta & CMETA_SECOND_LEAF) != 0;
            L += off;
            k += off;
          } else {
            at_leaf = (meta & CMETA_FIRST_LEAF) != 0;
            k += 1;
          }
          if (at_leaf) break;
        }
        leaf = L;
      }
      const int orig = pf.tree_orig[p];
      if (pf.c_leaf_ids[leaf] != ids[r * v.n_trees + orig]) ++bad;
      V pay;
      std::memcpy(&pay, pf.c_leaf_payload.data() + size_t(leaf) * sizeof(V), sizeof(V));
      double got;
      if (v.leaf_vector_len > 1) {
        got = static_cast<double>(static_cast<uint32_t>(pay));
      } else {
        T val;
        std::memcpy(&val, &pay, sizeof(T));
        got = static_cast<double>(val);
      }
      if (got != payload[r * v.n_trees + orig]) ++bad;
    }
  }
  return bad;
}
}  // namespace

extern "C" {
const char* pack_check_error() { return g_err.c_str(); }

// Packs `desc` and walks n_rows rows.  ids: leaf id per (row, tree); payload: scalar leaf value
// (or vector index) per (row, tree).  info[0..5] = format, storage, dense_depth, node_bytes,
// n_nodes_packed, feat_bits; info[6] = 1 when a rank-quantised copy was built, info[7] = number of
// (row, tree) pairs where the walk over that copy reaches another leaf; info[8..11] = feature
// groups of the quantised copy, most halvings of a group's search window, largest group blob in
// bytes, features in the first group; info[12] = 1 when a sparse forest got its compact image,
// info[13] = (row, tree) pairs where the walk over that image reaches another leaf or payload,
// info[14] = heap levels, info[15] = exact-threshold look-ups of that walk (fp64).
int pack_check(const b2fil_forest_desc* desc, const b2fil_create_opts* opts, const void* X,
               int64_t n_rows, int64_t stride, uint32_t* ids, double* payload, int64_t* info)
{
  PackedForest pf;
  const int rc = pack_forest(*desc, *opts, always_dense, pf, g_err);
  if (rc != B2FIL_OK) return rc;
  info[0] = pf.view.format;
  info[1] = pf.storage;
  info[2] = pf.view.dense_depth;
  info[3] = pf.node_bytes;
  info[4] = pf.n_nodes_packed;
  info[5] = pf.view.feat_bits;
  info[6] = pf.view.q_enabled;
  info[7] = 0;
  info[8] = static_cast<int64_t>(pf.q_groups.size());
  info[9] = info[10] = info[11] = 0;
  for (const QGroup& g : pf.q_groups) {
    info[9]  = std::max<int64_t>(info[9], g.steps);
    info[10] = std::max<int64_t>(info[10], g.blob_bytes);
  }
  if (!pf.q_groups.empty()) info[11] = pf.q_groups[0].f_end - pf.q_groups[0].f_begin;
  info[12] = pf.view.c_enabled;
  info[13] = info[15] = 0;
  info[14] = pf.view.c_enabled ? pf.view.c_top_levels : 0;
  if (n_rows > 0) {
    if (opts->precision == B2FIL_F32) {
      walk<float>(pf, static_cast<const float*>(X), n_rows, stride, ids, payload);
      if (pf.view.q_enabled)
        info[7] = walk_quantised<float>(pf, static_cast<const float*>(X), n_rows, stride, ids);
      if (pf.view.c_enabled)
        info[13] = walk_compact<float>(pf, static_cast<const float*>(X), n_rows, stride, ids,
                                       payload, &info[15]);
    } else {
      walk<double>(pf, static_cast<const double*>(X), n_rows, stride, ids, payload);
      if (pf.view.q_enabled)
        info[7] = walk_quantised<double>(pf, static_cast<const double*>(X), n_rows, stride, ids);
      if (pf.view.c_enabled)
        info[13] = walk_compact<double>(pf, static_cast<const double*>(X), n_rows, stride, ids,
                                        payload, &info[15]);
    }
  }
  return B2FIL_OK;
}
}
