// Forest import / packing: validates a host description, normalises every test to one operator
// and lays the nodes out for the device (see forest.hpp for the two storages).
//
// This is the work the reference delegates to nvforest.load_from_treelite_model /
// nvforest::import_from_treelite_handle (python/cuml/cuml/ensemble/randomforest_common.pyx:402-409,
// cpp/tests/sg/rf_test.cu:257-263): walk every tree on the host, choose precision and node order,
// pad trees to `align_bytes`, produce one contiguous node array.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <numeric>

#include "forest.hpp"

namespace b2fil {
namespace {

struct Test {
  bool is_cat;
  bool default_left;
  int32_t left, right;  // relative indices after normalisation
  double thr;           // numerical threshold in the target precision, operator is `<`
};

template <typename T>
T bump_up(T t, bool& always_left)
{
  always_left = false;
  if (std::isnan(t)) return t;
  if (t == std::numeric_limits<T>::infinity()) {
    always_left = true;
    return t;
  }
  return std::nextafter(t, std::numeric_limits<T>::infinity());
}

// Rewrite the test of node g as "x < thr -> left" (numerical) or "listed -> right" (categorical).
//  x <= t  <=>  x < next(t);  x > t -> L  <=>  x <= t -> R;  x >= t -> L  <=>  x < t -> R.
// A swap of the children flips the missing-value direction so that it names the same child.
Test normalise(const b2fil_forest_desc& d, int64_t g, int precision)
{
  Test t{};
  t.left         = d.left[g];
  t.right        = d.right[g];
  t.default_left = d.default_left[g] != 0;
  t.is_cat       = d.node_kind[g] == B2FIL_NODE_CATEGORICAL;
  auto swap_children = [&]() {
    std::swap(t.left, t.right);
    t.default_left = !t.default_left;
  };
  if (t.is_cat) {
    const bool right_on_match = d.cat_right ? d.cat_right[g] != 0 : true;
    if (!right_on_match) swap_children();
    t.thr = 0;
    return t;
  }
  int op        = d.op ? d.op[g] : d.op_all;
  double thr    = d.threshold[g];
  const bool sp = precision == B2FIL_F32;
  if (sp) thr = static_cast<double>(static_cast<float>(thr));
  if (op == B2FIL_OP_GT) {
    swap_children();
    op = B2FIL_OP_LE;
  } else if (op == B2FIL_OP_GE) {
    swap_children();
    op = B2FIL_OP_LT;
  }
  if (op == B2FIL_OP_LE) {
    bool always_left = false;
    if (sp) {
      thr = static_cast<double>(bump_up(static_cast<float>(thr), always_left));
    } else {
      thr = bump_up(thr, always_left);
    }
    if (always_left) {  // x <= +inf holds for every number: send numbers right after a swap
      swap_children();
      thr = -std::numeric_limits<double>::infinity();
    }
  }
  t.thr = thr;
  return t;
}

template <typename T>
void put(std::vector<uint8_t>& buf, size_t byte_off, const T& v)
{
  std::memcpy(buf.data() + byte_off, &v, sizeof(T));
}

uint32_t f32_bits(double v)
{
  float f = static_cast<float>(v);
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
}
uint64_t f64_bits(double v)
{
  uint64_t u;
  std::memcpy(&u, &v, 8);
  return u;
}

int bits_for(uint32_t max_value)
{
  int b = 1;
  while (b < 32 && (max_value >> b) != 0) ++b;
  return b;
}

struct Packer {
  const b2fil_forest_desc& d;
  const b2fil_create_opts& o;
  PackedForest& out;
  std::string& err;
  int precision;
  bool vec;
  int64_t n_vectors = 0;
  bool cat_inline   = true;
  bool has_cat      = false;
  std::vector<int32_t> depth_of;   // per node of the description (global index), -1 = unreachable
  std::vector<int32_t> tree_depth;

  Packer(const b2fil_forest_desc& d_, const b2fil_create_opts& o_, PackedForest& out_,
         std::string& err_)
    : d(d_), o(o_), out(out_), err(err_), precision(o_.precision), vec(d_.leaf_vector_len > 1)
  {
  }

  int fail(int code, const std::string& msg)
  {
    err = msg;
    return code;
  }

  int validate()
  {
    if (d.n_trees <= 0) return fail(B2FIL_ERR_INVALID_ARG, "n_trees must be positive");
    if (d.n_features <= 0) return fail(B2FIL_ERR_INVALID_ARG, "n_features must be positive");
    if (d.n_features > (1 << 29))
      return fail(B2FIL_ERR_UNSUPPORTED, "more than 2^29 features");
    if (d.n_outputs <= 0) return fail(B2FIL_ERR_INVALID_ARG, "n_outputs must be positive");
    if (d.leaf_vector_len != 1 && d.leaf_vector_len != d.n_outputs)
      return fail(B2FIL_ERR_INVALID_ARG, "leaf_vector_len must be 1 or n_outputs");
    if (!d.tree_offsets || !d.node_kind || !d.feature || !d.threshold || !d.left || !d.right ||
        !d.default_left || !d.leaf_value)
      return fail(B2FIL_ERR_INVALID_ARG, "a required array of the forest description is NULL");
    if (d.postproc < 0 || d.postproc > B2FIL_POST_EXP_STD_RATIO)
      return fail(B2FIL_ERR_INVALID_ARG, "unknown postprocessor");
    if (d.postproc == B2FIL_POST_EXP_STD_RATIO && d.ratio_c == 0.0)
      return fail(B2FIL_ERR_INVALID_ARG, "ratio_c must not be zero");
    if (d.tree_offsets[0] != 0) return fail(B2FIL_ERR_BAD_FOREST, "tree_offsets[0] must be 0");
    for (int t = 0; t < d.n_trees; ++t) {
      const int64_t n = d.tree_offsets[t + 1] - d.tree_offsets[t];
      if (n <= 0) return fail(B2FIL_ERR_BAD_FOREST, "tree " + std::to_string(t) + " is empty");
      if (n > (int64_t(1) << 31) - 1)
        return fail(B2FIL_ERR_TOO_LARGE, "tree " + std::to_string(t) + " has too many nodes");
      if (d.class_id && !vec && (d.class_id[t] < 0 || d.class_id[t] >= d.n_outputs))
        return fail(B2FIL_ERR_BAD_FOREST, "class_id of tree " + std::to_string(t) + " out of range");
    }
    return B2FIL_OK;
  }

  // Depth of every reachable node; rejects out-of-range children, bad features, shared nodes.
  int measure()
  {
    const int64_t total = d.tree_offsets[d.n_trees];
    depth_of.assign(static_cast<size_t>(total), -1);
    tree_depth.assign(d.n_trees, 0);
    std::vector<int32_t> stack;
    for (int t = 0; t < d.n_trees; ++t) {
      const int64_t base = d.tree_offsets[t];
      const int64_t n    = d.tree_offsets[t + 1] - base;
      stack.clear();
      stack.push_back(0);
      depth_of[base] = 0;
      int md         = 0;
      while (!stack.empty()) {
        const int32_t r = stack.back();
        stack.pop_back();
        const int64_t g = base + r;
        const int dep   = depth_of[g];
        md              = std::max(md, dep);
        const uint8_t k = d.node_kind[g];
        if (k == B2FIL_NODE_LEAF) {
          if (vec) ++n_vectors;
          continue;
        }
        if (k != B2FIL_NODE_NUMERICAL && k != B2FIL_NODE_CATEGORICAL)
          return fail(B2FIL_ERR_BAD_FOREST, "unknown node kind in tree " + std::to_string(t));
        if (d.feature[g] < 0 || d.feature[g] >= d.n_features)
          return fail(B2FIL_ERR_BAD_FOREST, "feature index out of range in tree " +
                                              std::to_string(t) + " node " + std::to_string(r));
        if (k == B2FIL_NODE_NUMERICAL) {
          const int op = d.op ? d.op[g] : d.op_all;
          if (op < B2FIL_OP_LT || op > B2FIL_OP_GE)
            return fail(B2FIL_ERR_BAD_FOREST, "unknown comparison operator");
        } else {
          if (!d.cat_ptr || !d.cat_values)
            return fail(B2FIL_ERR_BAD_FOREST, "categorical node without category arrays");
          if (d.cat_ptr[g + 1] < d.cat_ptr[g])
            return fail(B2FIL_ERR_BAD_FOREST, "cat_ptr is not monotone");
          has_cat = true;
          for (int64_t c = d.cat_ptr[g]; c < d.cat_ptr[g + 1]; ++c) {
            if (d.cat_values[c] >= 32) cat_inline = false;
            if (d.cat_values[c] >= (1u << 24))
              return fail(B2FIL_ERR_UNSUPPORTED, "category value of 2^24 or more");
          }
        }
        const int32_t ch[2] = {d.left[g], d.right[g]};
        for (int32_t c : ch) {
          if (c < 0 || c >= n)
            return fail(B2FIL_ERR_BAD_FOREST, "child index out of range in tree " +
                                                std::to_string(t) + " node " + std::to_string(r));
          if (depth_of[base + c] != -1)
            return fail(B2FIL_ERR_BAD_FOREST, "node reached twice (cycle or shared child) in tree " +
                                                std::to_string(t));
          depth_of[base + c] = dep + 1;
          stack.push_back(c);
        }
      }
      tree_depth[t] = md;
    }
    return B2FIL_OK;
  }

  // Category list of node g as a record in the pool: [n_words, words...]; returns its offset.
  uint32_t pool_record(int64_t g)
  {
    uint32_t mx = 0;
    for (int64_t c = d.cat_ptr[g]; c < d.cat_ptr[g + 1]; ++c) mx = std::max(mx, d.cat_values[c]);
    const uint32_t n_words = (d.cat_ptr[g + 1] > d.cat_ptr[g]) ? mx / 32 + 1 : 0;
    const uint32_t off     = static_cast<uint32_t>(out.cat_pool.size());
    out.cat_pool.push_back(n_words);
    out.cat_pool.resize(out.cat_pool.size() + n_words, 0u);
    for (int64_t c = d.cat_ptr[g]; c < d.cat_ptr[g + 1]; ++c) {
      const uint32_t v = d.cat_values[c];
      out.cat_pool[off + 1 + v / 32] |= 1u << (v % 32);
    }
    return off;
  }
  uint32_t inline_bitset(int64_t g)
  {
    uint32_t b = 0;
    for (int64_t c = d.cat_ptr[g]; c < d.cat_ptr[g + 1]; ++c) b |= 1u << d.cat_values[c];
    return b;
  }
  // value word(s) of a test node
  uint64_t test_value(int64_t g, const Test& t)
  {
    if (t.is_cat) return cat_inline ? inline_bitset(g) : pool_record(g);
    return precision == B2FIL_F32 ? f32_bits(t.thr) : f64_bits(t.thr);
  }
  // payload of a leaf: scalar in the forest precision or the index of its vector
  uint64_t leaf_payload(int64_t g, int64_t& vec_counter)
  {
    if (!vec) {
      return precision == B2FIL_F32 ? f32_bits(d.leaf_value[g]) : f64_bits(d.leaf_value[g]);
    }
    const int64_t idx = vec_counter++;
    const int k       = d.n_outputs;
    for (int c = 0; c < k; ++c) {
      const double v = d.leaf_value[g * k + c];
      if (precision == B2FIL_F32) {
        put(out.leaf_vectors, (idx * k + c) * 4, static_cast<float>(v));
      } else {
        put(out.leaf_vectors, (idx * k + c) * 8, v);
      }
    }
    return static_cast<uint64_t>(idx);
  }

  void common_tables()
  {
    const int k   = d.n_outputs;
    const int nt  = d.n_trees;
    out.tree_orig.resize(nt);
    std::iota(out.tree_orig.begin(), out.tree_orig.end(), 0);
    std::vector<int32_t> cls(nt, 0);
    if (!vec) {
      for (int t = 0; t < nt; ++t) cls[t] = d.class_id ? d.class_id[t] : t % k;
      // trees of one output run back to back so that a thread keeps one running sum
      std::stable_sort(out.tree_orig.begin(), out.tree_orig.end(),
                       [&](int a, int b) { return cls[a] < cls[b]; });
    }
    out.tree_class.resize(nt);
    for (int t = 0; t < nt; ++t) out.tree_class[t] = vec ? 0 : cls[out.tree_orig[t]];
    std::vector<double> count(k, 0.0);
    for (int t = 0; t < nt; ++t) {
      if (vec) {
        for (int c = 0; c < k; ++c) count[c] += 1;
      } else {
        count[cls[t]] += 1;
      }
    }
    const size_t es = precision == B2FIL_F32 ? 4 : 8;
    out.out_scale.resize(k * es);
    out.out_bias.resize(k * es);
    for (int c = 0; c < k; ++c) {
      const double s = (d.average_tree_output && count[c] > 0) ? 1.0 / count[c] : 1.0;
      const double b = d.base_scores ? d.base_scores[c] : 0.0;
      if (precision == B2FIL_F32) {
        put(out.out_scale, c * 4, static_cast<float>(s));
        put(out.out_bias, c * 4, static_cast<float>(b));
      } else {
        put(out.out_scale, c * 8, s);
        put(out.out_bias, c * 8, b);
      }
    }
    if (vec) out.leaf_vectors.resize(static_cast<size_t>(n_vectors) * k * es);
  }

  // ---- dense ----------------------------------------------------------------------------------
  int pack_dense(int D)
  {
    const bool sp        = precision == B2FIL_F32;
    const size_t nb      = sp ? sizeof(DenseNodeF) : sizeof(DenseNodeD);
    const size_t lb      = sp ? 4 : 8;
    const int64_t width  = int64_t(1) << D;
    int64_t stride       = width * static_cast<int64_t>(nb + lb);
    stride               = (stride + 15) / 16 * 16;
    const int nt         = d.n_trees;
    out.nodes.assign(static_cast<size_t>(stride) * nt, 0);
    out.leaf_ids.assign(static_cast<size_t>(width) * nt, 0);
    int64_t vec_counter = 0;
    struct Item {
      int32_t rel;
      uint32_t heap;
      int32_t level;
      bool leaf_fill;
      uint64_t payload;
    };
    std::vector<Item> stack;
    for (int p = 0; p < nt; ++p) {
      const int t        = out.tree_orig[p];
      const int64_t base = d.tree_offsets[t];
      const size_t tb    = static_cast<size_t>(stride) * p;
      stack.clear();
      stack.push_back({0, 1u, 0, false, 0});
      while (!stack.empty()) {
        Item it = stack.back();
        stack.pop_back();
        const int64_t g = base + it.rel;
        if (!it.leaf_fill && d.node_kind[g] != B2FIL_NODE_LEAF) {
          const Test ts     = normalise(d, g, precision);
          const uint64_t v  = test_value(g, ts);
          uint32_t meta     = static_cast<uint32_t>(d.feature[g]);
          if (ts.default_left) meta |= META_DEFAULT_LEFT;
          if (ts.is_cat) meta |= META_CATEGORICAL;
          if (sp) {
            put(out.nodes, tb + it.heap * nb, DenseNodeF{static_cast<uint32_t>(v), meta});
          } else {
            put(out.nodes, tb + it.heap * nb, DenseNodeD{v, meta, 0});
          }
          stack.push_back({ts.right, it.heap * 2 + 1, it.level + 1, false, 0});
          stack.push_back({ts.left, it.heap * 2, it.level + 1, false, 0});
          continue;
        }
        // a leaf above the last level is repeated below itself: both children of a filler test
        // lead to the same payload, so its outcome does not matter
        if (!it.leaf_fill) {
          it.payload   = leaf_payload(g, vec_counter);
          it.leaf_fill = true;
        }
        if (it.level == D) {
          const uint64_t slot = it.heap - static_cast<uint32_t>(width);
          if (sp) {
            put(out.nodes, tb + width * nb + slot * 4, static_cast<uint32_t>(it.payload));
          } else {
            put(out.nodes, tb + width * nb + slot * 8, it.payload);
          }
          out.leaf_ids[static_cast<size_t>(width) * p + slot] = static_cast<uint32_t>(it.rel);
        } else {
          if (sp) {
            put(out.nodes, tb + it.heap * nb, DenseNodeF{f32_bits(0.0), 0u});
          } else {
            put(out.nodes, tb + it.heap * nb, DenseNodeD{f64_bits(0.0), 0u, 0u});
          }
          stack.push_back({it.rel, it.heap * 2 + 1, it.level + 1, true, it.payload});
          stack.push_back({it.rel, it.heap * 2, it.level + 1, true, it.payload});
        }
      }
    }
    out.view.format       = sp ? FMT_DENSE_F : FMT_DENSE_D;
    out.view.dense_depth  = D;
    out.view.tree_stride  = stride;
    out.storage           = B2FIL_STORAGE_DENSE;
    out.node_bytes        = static_cast<int32_t>(nb);
    out.n_nodes_packed    = width * 2 * nt;
    return B2FIL_OK;
  }

  // ---- rank-quantised copy of a dense forest ----------------------------------------------------
  // Returns false (and leaves the forest unquantised) when a limit is exceeded.
  template <typename T>
  bool build_quantised(int D)
  {
    const int F = d.n_features;
    if (F > static_cast<int>(Q_MAX_FEATURES)) return false;
    if (D < 1) return false;  // forests of single leaves have nothing to rank
    if (has_cat && !cat_inline) return false;  // category sets must fit 32 bits
    const int nt = d.n_trees;
    // 1. distinct thresholds per feature, in the forest precision, after normalisation to `<`;
    //    a feature is either numerical or categorical in the whole forest
    std::vector<std::vector<T>> per(F);
    std::vector<uint8_t> used_num(F, 0), used_cat(F, 0);
    for (int t = 0; t < nt; ++t) {
      const int64_t base = d.tree_offsets[t];
      const int64_t n    = d.tree_offsets[t + 1] - base;
      for (int64_t r = 0; r < n; ++r) {
        const int64_t g = base + r;
        if (depth_of[g] < 0) continue;
        if (d.node_kind[g] == B2FIL_NODE_CATEGORICAL) used_cat[d.feature[g]] = 1;
        if (d.node_kind[g] != B2FIL_NODE_NUMERICAL) continue;
        used_num[d.feature[g]] = 1;
        const T thr = static_cast<T>(normalise(d, g, precision).thr);
        if (!std::isnan(thr)) per[d.feature[g]].push_back(thr);
      }
    }
    for (int f = 0; f < F; ++f) {
      if (used_num[f] && used_cat[f]) return false;
    }
    for (int f = 0; f < F; ++f) {
      auto& v = per[f];
      std::sort(v.begin(), v.end());
      v.erase(std::unique(v.begin(), v.end()), v.end());  // -0.0 == +0.0: one threshold
      if (v.size() > Q_MAX_RANK) return false;
    }
    // 2. bucket tables.  The table of one feature for a given number of buckets per threshold:
    //    grid over the finite thresholds, lut[b] = thresholds in buckets below b, fullest bucket.
    struct FeatTable {
      uint32_t n_buckets = 1, max_occupancy = 0;
      T scale = 0, offset = 0;
      std::vector<uint16_t> lut;
    };
    auto make_table = [&](int f, double factor) {
      const auto& v = per[f];
      FeatTable t;
      if (v.empty()) {
        t.lut.assign(1, 0);
        return t;
      }
      const double want = std::ceil(factor * static_cast<double>(v.size()));
      t.n_buckets       = static_cast<uint32_t>(std::min(4096.0, std::max(16.0, want)));
      size_t lo = 0, hi = v.size();
      while (lo < hi && !std::isfinite(v[lo])) ++lo;
      while (hi > lo && !std::isfinite(v[hi - 1])) --hi;
      if (hi - lo >= 2) {
        const double range = static_cast<double>(v[hi - 1]) - static_cast<double>(v[lo]);
        const T sc         = static_cast<T>(static_cast<double>(t.n_buckets) / range);
        const T of         = static_cast<T>(-static_cast<double>(v[lo]) * static_cast<double>(sc));
        if (std::isfinite(sc) && std::isfinite(of) && sc > T(0)) {
          t.scale  = sc;
          t.offset = of;
        }
      }
      std::vector<uint32_t> count(t.n_buckets + 1, 0);
      for (size_t i = 0; i < v.size(); ++i)
        ++count[q_bucket_host<T>(v[i], t.scale, t.offset, t.n_buckets) + 1];
      t.lut.resize(t.n_buckets);
      uint32_t run = 0;
      for (uint32_t b = 0; b < t.n_buckets; ++b) {
        run += count[b];  // thresholds in buckets below b
        t.lut[b]        = static_cast<uint16_t>(run);
        t.max_occupancy = std::max(t.max_occupancy, count[b + 1]);
      }
      return t;
    };
    // 3. feature groups, one blob each.  Inside a blob the tables of the group's GF features are
    //    interleaved element by element (entry k of feature i sits at index k * GF + i), so that
    //    the lanes of a warp, which hold one feature each, read different shared-memory banks
    //    whatever k they probe.  Wide groups matter more than fine buckets: with 32 features a
    //    warp's lookups never collide, and one more halving of a longer search window costs one
    //    conflict-free load.  So for every run of features the widest power-of-two group is taken
    //    for which some bucket density fits shared memory, densest first.
    auto steps_for = [](uint32_t occ) {
      uint32_t k = 0;
      while ((1u << k) <= occ) ++k;  // 2^k > occ
      return k;
    };
    std::vector<double> factors = {2.0, 1.0, 0.5, 0.25, 0.125};
    int max_group = static_cast<int>(kQMaxGroupFeatures);
    if (const char* e = std::getenv("B2FIL_Q_BUCKETS")) {  // tuning aid: buckets per threshold
      const double forced = std::atof(e);
      if (forced >= 0.01 && forced <= 16.0) factors = {forced};
    }
    if (const char* e = std::getenv("B2FIL_Q_GROUP")) {  // tuning aid: widest feature group
      const int forced = std::atoi(e);
      if (forced >= 1 && forced <= max_group && (forced & (forced - 1)) == 0) max_group = forced;
    }
    out.q_feats.assign(F, QFeature{});
    out.q_groups.clear();
    out.q_blob.clear();
    out.view.q_max_blob_bytes = 0;
    const uint32_t rec_bytes  = kQMaxGroupFeatures * sizeof(QFeatRec);
    for (int f = 0; f < F;) {
      int n = 0;
      std::vector<FeatTable> tables;
      uint32_t steps = 0, n_thr = 0, lut_bytes = 0, thr_bytes = 0;
      for (int want = max_group; want >= 1 && n == 0; want /= 2) {
        if (f + want > F) continue;  // a short tail is split into smaller powers of two
        for (double factor : factors) {
          std::vector<FeatTable> cand;
          uint32_t st = 0, n_lut = 0, m_max = 0;
          for (int g = f; g < f + want; ++g) {
            cand.push_back(make_table(g, factor));
            st    = std::max(st, steps_for(cand.back().max_occupancy));
            n_lut = std::max(n_lut, cand.back().n_buckets);
            m_max = std::max<uint32_t>(m_max, static_cast<uint32_t>(per[g].size()));
          }
          const uint32_t nt_ = m_max + (1u << st);  // window padding behind the longest table
          const uint32_t lb  = (n_lut * want * 2 + 15) / 16 * 16;
          const uint32_t tb  = static_cast<uint32_t>((static_cast<size_t>(nt_) * want * sizeof(T) + 15) / 16 * 16);
          if (rec_bytes + lb + tb <= kQGroupSmemBudget) {
            n         = want;
            tables    = std::move(cand);
            steps     = st;
            n_thr     = nt_;
            lut_bytes = lb;
            thr_bytes = tb;
            break;
          }
        }
      }
      if (n == 0) return false;  // one feature alone exceeds the budget
      QGroup g{};
      g.f_begin  = static_cast<uint32_t>(f);
      g.f_end    = static_cast<uint32_t>(f + n);
      g.steps    = steps;
      g.blob_off = static_cast<uint32_t>(out.q_blob.size());
      std::vector<uint8_t> blob(rec_bytes + lut_bytes + thr_bytes, 0);
      const T nan = std::numeric_limits<T>::quiet_NaN();
      for (int h = f; h < f + n; ++h) {
        const FeatTable& t = tables[h - f];
        const auto& v      = per[h];
        const uint32_t i   = static_cast<uint32_t>(h - f);
        QFeature& qf       = out.q_feats[h];
        qf.is_cat          = used_cat[h];
        qf.m               = static_cast<uint32_t>(v.size());
        qf.n_buckets       = t.n_buckets;
        qf.max_occupancy   = t.max_occupancy;
        qf.scale           = static_cast<double>(t.scale);
        qf.offset          = static_cast<double>(t.offset);
        QFeatRec rec{};
        rec.is_cat  = qf.is_cat;
        rec.nbm1    = t.n_buckets - 1;
        rec.scale   = qf.scale;
        rec.offset  = qf.offset;
        rec.lut_off = rec_bytes + i * 2;  // entry k: + k * n * 2
        rec.thr_off = rec_bytes + lut_bytes + i * static_cast<uint32_t>(sizeof(T));
        for (uint32_t k = 0; k < t.n_buckets; ++k)
          put(blob, rec.lut_off + static_cast<size_t>(k) * n * 2, t.lut[k]);
        for (uint32_t k = 0; k < n_thr; ++k)
          put(blob, rec.thr_off + static_cast<size_t>(k) * n * sizeof(T), k < v.size() ? v[k] : nan);
        std::memcpy(blob.data() + i * sizeof(QFeatRec), &rec, sizeof(rec));
      }
      g.blob_bytes = static_cast<uint32_t>(blob.size());
      out.q_blob.insert(out.q_blob.end(), blob.begin(), blob.end());
      out.view.q_max_blob_bytes = std::max<int64_t>(out.view.q_max_blob_bytes, g.blob_bytes);
      out.q_groups.push_back(g);
      f += n;
    }
    // 4. nodes: same heap layout as the dense blocks, 4 bytes per test node; in forests with
    //    categorical tests a node is 8 bytes {node, 32-bit category set}, so that one load brings
    //    both (a numerical node holds an empty set)
    const size_t nb      = sizeof(T) == 4 ? sizeof(DenseNodeF) : sizeof(DenseNodeD);
    const size_t es      = sizeof(T);
    const int64_t width  = int64_t(1) << D;
    const int64_t qnb    = has_cat ? 8 : 4;  // bytes per test node in the quantised image
    // vector leaves of forests with few outputs go into the tree block itself: the traversal
    // then reads them from shared memory instead of gathering them from global memory per
    // (row, tree), which costs a divergent load each
    const bool inline_vec = vec && d.n_outputs <= kQInlineClasses;
    const int64_t lbytes  = inline_vec ? static_cast<int64_t>(d.n_outputs) * es : static_cast<int64_t>(es);
    int64_t qstride       = width * static_cast<int64_t>(qnb + lbytes);
    qstride              = (qstride + 15) / 16 * 16;
    out.q_nodes.assign(static_cast<size_t>(qstride) * nt, 0);
    for (int p = 0; p < nt; ++p) {
      const uint8_t* src = out.nodes.data() + static_cast<size_t>(out.view.tree_stride) * p;
      uint8_t* dst       = out.q_nodes.data() + static_cast<size_t>(qstride) * p;
      for (int64_t i = 1; i < width; ++i) {
        T thr;
        uint32_t meta;
        std::memcpy(&thr, src + i * nb, sizeof(T));
        std::memcpy(&meta, src + i * nb + sizeof(T), 4);
        const uint32_t feat = meta & 0x3FFFFFFFu;
        uint32_t node       = ((meta & META_DEFAULT_LEFT) ? 0u : Q_DEFAULT_RIGHT) | (feat << Q_FEATURE_SHIFT);
        if (meta & META_CATEGORICAL) {
          uint32_t bits;  // the inline category set sits in the low word of the value slot
          std::memcpy(&bits, src + i * nb, 4);
          // stored bit-reversed (category c in bit 31 - c): shifting the word left by the
          // category then puts the answer in the sign bit
          uint32_t rev = 0;
          for (int c = 0; c < 32; ++c) rev |= ((bits >> c) & 1u) << (31 - c);
          std::memcpy(dst + i * qnb + 4, &rev, 4);
          // the rank comparison of such a node must never say "right": the largest rank field
          node |= Q_MAX_RANK_FIELD << Q_RANK_SHIFT;  // the largest rank marks a categorical node
        } else {
          uint32_t j;
          if (std::isnan(thr)) {
            j = Q_NEVER_LEFT;  // x < NaN never holds: always right
          } else {
            const auto& v = per[feat];
            const auto it = std::lower_bound(v.begin(), v.end(), thr);
            // filler tests (both subtrees equal) need no real threshold
            j = (it != v.end() && *it == thr) ? static_cast<uint32_t>(it - v.begin()) : 0u;
          }
          node |= j << Q_RANK_SHIFT;
        }
        std::memcpy(dst + i * qnb, &node, 4);
      }
      if (!inline_vec) {
        std::memcpy(dst + width * qnb, src + width * nb, static_cast<size_t>(width) * es);
      } else {
        for (int64_t sl = 0; sl < width; ++sl) {
          uint32_t vi;  // index of the leaf's vector (low word of the dense payload)
          std::memcpy(&vi, src + width * nb + sl * es, 4);
          std::memcpy(dst + width * qnb + sl * lbytes,
                      out.leaf_vectors.data() + static_cast<size_t>(vi) * d.n_outputs * es,
                      static_cast<size_t>(lbytes));
        }
      }
    }
    // the same image with the leaf id in every payload slot, for predictions that report leaves
    out.q_nodes_ids = out.q_nodes;
    for (int p = 0; p < nt; ++p) {
      uint8_t* leaves = out.q_nodes_ids.data() + static_cast<size_t>(qstride) * p + width * qnb;
      std::memset(leaves, 0, static_cast<size_t>(width) * lbytes);
      for (int64_t s = 0; s < width; ++s) {
        const uint32_t id = out.leaf_ids[static_cast<size_t>(width) * p + s];
        std::memcpy(leaves + s * lbytes, &id, 4);
      }
    }
    bool in_order = true;
    for (int p = 0; p < nt; ++p) in_order = in_order && out.tree_orig[p] == p;
    out.view.q_trees_in_order = in_order ? 1 : 0;
    out.q_top.clear();
    if (!has_cat && D >= 2 && nt <= kQTopTrees) {
      out.q_top.resize(static_cast<size_t>(nt) * 3);
      for (int p = 0; p < nt; ++p)  // heap words 1..3 of the tree
        std::memcpy(out.q_top.data() + static_cast<size_t>(p) * 3,
                    out.q_nodes.data() + static_cast<size_t>(qstride) * p + 4, 12);
    }
    out.view.q_has_cat     = has_cat ? 1 : 0;
    out.view.q_enabled     = 1;
    out.view.q_n_groups    = static_cast<int32_t>(out.q_groups.size());
    out.view.q_tree_stride = qstride;
    out.view.q_leaf_bytes  = static_cast<int32_t>(lbytes);
    return true;
  }

  // ---- sparse ---------------------------------------------------------------------------------
  int pack_sparse()
  {
    const bool sp = precision == B2FIL_F32;
    const int nt  = d.n_trees;
    const int layout = o.layout;
    // position of every reachable node in the packed array
    const int64_t total = d.tree_offsets[nt];
    std::vector<uint32_t> pos(static_cast<size_t>(total), 0xFFFFFFFFu);
    out.roots.assign(nt, 0);
    size_t node_bytes_guess = sp ? 8 : 16;
    int64_t cursor          = 0;
    uint32_t max_offset     = 0;
    std::vector<int32_t> order;  // scratch
    auto align_cursor = [&](size_t nbytes) {
      if (o.align_bytes > 0) {
        const int64_t per = std::max<int64_t>(1, o.align_bytes / static_cast<int64_t>(nbytes));
        cursor            = (cursor + per - 1) / per * per;
      }
    };
    if (layout == B2FIL_LAYOUT_LAYERED) {
      // level by level over the whole forest; siblings adjacent
      int maxd = 0;
      for (int p = 0; p < nt; ++p) maxd = std::max(maxd, tree_depth[out.tree_orig[p]]);
      std::vector<std::vector<int32_t>> frontier(nt), next(nt);
      for (int p = 0; p < nt; ++p) frontier[p].push_back(0);
      for (int lvl = 0; lvl <= maxd; ++lvl) {
        for (int p = 0; p < nt; ++p) {
          const int64_t base = d.tree_offsets[out.tree_orig[p]];
          next[p].clear();
          for (int32_t r : frontier[p]) {
            pos[base + r] = static_cast<uint32_t>(cursor++);
            if (d.node_kind[base + r] != B2FIL_NODE_LEAF) {
              const Test ts = normalise(d, base + r, precision);
              next[p].push_back(ts.left);
              next[p].push_back(ts.right);
            }
          }
        }
        frontier.swap(next);
      }
    } else {
      for (int p = 0; p < nt; ++p) {
        const int64_t base = d.tree_offsets[out.tree_orig[p]];
        align_cursor(node_bytes_guess);
        order.clear();
        if (layout == B2FIL_LAYOUT_DEPTH_FIRST) {
          std::vector<int32_t>& stack = order;  // positions are assigned on pop
          stack.push_back(0);
          while (!stack.empty()) {
            const int32_t r = stack.back();
            stack.pop_back();
            pos[base + r] = static_cast<uint32_t>(cursor++);
            if (d.node_kind[base + r] != B2FIL_NODE_LEAF) {
              const Test ts = normalise(d, base + r, precision);
              stack.push_back(ts.right);
              stack.push_back(ts.left);  // left is popped next: it sits right after its parent
            }
          }
        } else {
          size_t head = 0;
          order.push_back(0);
          while (head < order.size()) {
            const int32_t r = order[head++];
            pos[base + r]   = static_cast<uint32_t>(cursor++);
            if (d.node_kind[base + r] != B2FIL_NODE_LEAF) {
              const Test ts = normalise(d, base + r, precision);
              order.push_back(ts.left);
              order.push_back(ts.right);
            }
          }
        }
      }
    }
    if (cursor >= (int64_t(1) << 32))
      return fail(B2FIL_ERR_TOO_LARGE, "packed forest has 2^32 nodes or more");
    const int64_t n_packed = cursor;
    // offsets decide the node format
    for (int p = 0; p < nt; ++p) {
      const int t        = out.tree_orig[p];
      const int64_t base = d.tree_offsets[t];
      const int64_t n    = d.tree_offsets[t + 1] - base;
      out.roots[p]       = pos[base];
      for (int64_t r = 0; r < n; ++r) {
        const int64_t g = base + r;
        if (depth_of[g] < 0 || d.node_kind[g] == B2FIL_NODE_LEAF) continue;
        const Test ts      = normalise(d, g, precision);
        const uint32_t far = layout == B2FIL_LAYOUT_DEPTH_FIRST ? pos[base + ts.right]
                                                                : pos[base + ts.left];
        max_offset = std::max(max_offset, far - pos[g]);
      }
    }
    const int feat_bits = bits_for(static_cast<uint32_t>(d.n_features - 1));
    int format          = FMT_SPARSE_16D;
    if (sp) {
      const int off_bits = 29 - feat_bits;
      format = (off_bits >= 1 && max_offset < (1u << off_bits)) ? FMT_SPARSE_8 : FMT_SPARSE_16F;
    }
    const size_t nb = format == FMT_SPARSE_8 ? 8 : 16;
    // tree starts were aligned assuming the narrowest node of the precision; with wider nodes a
    // tree start stays on a multiple of align_bytes because its byte offset only doubles
    out.nodes.assign(static_cast<size_t>(n_packed) * nb, 0);
    out.leaf_ids.assign(static_cast<size_t>(n_packed), 0);
    int64_t vec_counter = 0;
    for (int p = 0; p < nt; ++p) {
      const int t        = out.tree_orig[p];
      const int64_t base = d.tree_offsets[t];
      const int64_t n    = d.tree_offsets[t + 1] - base;
      for (int64_t r = 0; r < n; ++r) {
        const int64_t g = base + r;
        if (depth_of[g] < 0) continue;
        const uint32_t at = pos[g];
        uint64_t value;
        uint32_t meta = 0, offset = 0;
        if (d.node_kind[g] == B2FIL_NODE_LEAF) {
          value = leaf_payload(g, vec_counter);
          meta  = META_LEAF;
          out.leaf_ids[at] = static_cast<uint32_t>(r);
        } else {
          const Test ts = normalise(d, g, precision);
          value         = test_value(g, ts);
          meta          = static_cast<uint32_t>(d.feature[g]);
          if (ts.default_left) meta |= META_DEFAULT_LEFT;
          if (ts.is_cat) meta |= META_CATEGORICAL;
          const uint32_t far = layout == B2FIL_LAYOUT_DEPTH_FIRST ? pos[base + ts.right]
                                                                  : pos[base + ts.left];
          offset = far - at;
        }
        if (format == FMT_SPARSE_8) {
          meta |= offset << feat_bits;
          put(out.nodes, at * nb, SparseNode8{static_cast<uint32_t>(value), meta});
        } else if (format == FMT_SPARSE_16F) {
          put(out.nodes, at * nb, SparseNode16F{static_cast<uint32_t>(value), meta, offset, 0});
        } else {
          put(out.nodes, at * nb, SparseNode16D{value, meta, offset});
        }
      }
    }
    out.view.format      = format;
    out.view.feat_bits   = feat_bits;
    out.view.dense_depth = -1;
    out.view.tree_stride = 0;
    out.storage          = B2FIL_STORAGE_SPARSE;
    out.node_bytes       = static_cast<int32_t>(nb);
    out.n_nodes_packed   = n_packed;
    if (o.compact_image != 1) build_compact(pos, nb, format);
    return B2FIL_OK;
  }

  // Largest float that is <= t (t itself when it is a float).
  static float round_down_to_float(double t)
  {
    float f = static_cast<float>(t);
    if (static_cast<double>(f) > t) f = std::nextafter(f, -std::numeric_limits<float>::infinity());
    return f;
  }

  // Second image of a sparse forest (see forest.hpp): internal nodes only, depth first, 8 bytes
  // each; leaves apart; the top levels of every tree as a heap.  Values and payloads are taken
  // from the primary image, so both images agree bit for bit.  Leaves the image out (and the
  // view's c_enabled at 0) when a field does not fit.
  void build_compact(const std::vector<uint32_t>& pos, size_t nb, int format)
  {
    const bool sp    = precision == B2FIL_F32;
    const int nt     = d.n_trees;
    const int es     = sp ? 4 : 8;
    const int fb     = bits_for(static_cast<uint32_t>(d.n_features - 1));
    const int maxd   = *std::max_element(tree_depth.begin(), tree_depth.end());
    int T            = compact_pick_top_levels(es, d.n_features, d.n_outputs, maxd);
    if (o.compact_image > 100 && T >= 1)  // tuning aid: another number of heap levels
      T = std::max(1, std::min({o.compact_image - 100, kCMaxTopLevels, std::max(1, maxd)}));
    if (T < 1 || fb >= 27) return;
    auto primary_value = [&](int64_t g) -> uint64_t {
      const uint8_t* at = out.nodes.data() + static_cast<size_t>(pos[g]) * nb;
      if (format == FMT_SPARSE_16D) {
        uint64_t v;
        std::memcpy(&v, at, 8);
        return v;
      }
      uint32_t v;
      std::memcpy(&v, at, 4);
      return v;
    };
    auto primary_meta = [&](int64_t g) -> uint32_t {
      uint32_t m;
      std::memcpy(&m, out.nodes.data() + static_cast<size_t>(pos[g]) * nb + (format == FMT_SPARSE_16D ? 8 : 4), 4);
      return m;
    };
    // value word of the compact node of test g
    auto compact_value = [&](int64_t g, bool is_cat) -> uint32_t {
      const uint64_t v = primary_value(g);
      if (is_cat || sp) return static_cast<uint32_t>(v);
      double thr;
      std::memcpy(&thr, &v, 8);
      const float lo = round_down_to_float(thr);
      uint32_t bits;
      std::memcpy(&bits, &lo, 4);
      return bits;
    };

    std::vector<uint32_t> cn;      // {value, meta without the offset field} per internal node
    std::vector<uint32_t> coff;    // offset field per internal node
    std::vector<uint32_t>& lb = out.c_leaves_before;
    std::vector<double>& ex   = out.c_exact;
    std::vector<uint32_t> number;  // per node of the current tree: its internal or leaf number
    struct Frame {
      int32_t rel;
      int64_t parent;   // forest-wide internal number of the parent, -1 for the root
      bool is_second;   // the parent's second (far) child
    };
    std::vector<Frame> stack;
    std::vector<int32_t> heap, order;
    std::vector<uint32_t> weight;  // internal nodes in the subtree of every node of the current tree
    const size_t heap_n    = size_t(1) << T;
    const size_t top_bytes = heap_n * 16;  // 8-byte nodes, 8-byte exits
    out.c_top.assign(static_cast<size_t>(nt) * top_bytes, 0);
    if (!sp) out.c_top_src.assign(static_cast<size_t>(nt) * heap_n, C_NO_NODE);
    uint32_t max_off = 0;
    uint64_t n_leaf  = 0;
    for (int p = 0; p < nt; ++p) {
      const int t        = out.tree_orig[p];
      const int64_t base = d.tree_offsets[t];
      const int64_t n    = d.tree_offsets[t + 1] - base;
      number.assign(static_cast<size_t>(n), 0);
      // subtree sizes, children before parents (reverse of a pre-order listing)
      weight.assign(static_cast<size_t>(n), 0);
      order.clear();
      order.push_back(0);
      for (size_t i = 0; i < order.size(); ++i) {
        const int64_t g = base + order[i];
        if (d.node_kind[g] == B2FIL_NODE_LEAF) continue;
        const Test ts = normalise(d, g, precision);
        order.push_back(ts.left);
        order.push_back(ts.right);
      }
      for (size_t i = order.size(); i-- > 0;) {
        const int64_t g = base + order[i];
        if (d.node_kind[g] == B2FIL_NODE_LEAF) continue;
        const Test ts    = normalise(d, g, precision);
        weight[order[i]] = 1 + weight[ts.left] + weight[ts.right];
      }
      stack.clear();
      stack.push_back({0, -1, false});
      while (!stack.empty()) {
        const Frame fr = stack.back();
        stack.pop_back();
        const int64_t g = base + fr.rel;
        const uint64_t n_int = cn.size() / 2;
        if (fr.is_second) {
          // everything between the parent and here is the subtree of the parent's first child
          const uint64_t off = n_int - static_cast<uint64_t>(fr.parent);
          coff[static_cast<size_t>(fr.parent)] = static_cast<uint32_t>(off);
          max_off = std::max<uint64_t>(max_off, off);
        }
        if (d.node_kind[g] == B2FIL_NODE_LEAF) {
          number[fr.rel] = static_cast<uint32_t>(n_leaf++);
          const uint64_t pay = primary_value(g);
          const size_t at    = out.c_leaf_payload.size();
          out.c_leaf_payload.resize(at + es);
          if (sp) {
            const uint32_t v = static_cast<uint32_t>(pay);
            std::memcpy(out.c_leaf_payload.data() + at, &v, 4);
          } else {
            std::memcpy(out.c_leaf_payload.data() + at, &pay, 8);
          }
          out.c_leaf_ids.push_back(static_cast<uint32_t>(fr.rel));
          if (fr.parent >= 0)
            cn[static_cast<size_t>(fr.parent) * 2 + 1] |= fr.is_second ? CMETA_SECOND_LEAF : CMETA_FIRST_LEAF;
          continue;
        }
        const Test ts = normalise(d, g, precision);
        number[fr.rel] = static_cast<uint32_t>(n_int);
        // the child with the larger subtree comes first (ties: the left one)
        const bool swapped = weight[ts.right] > weight[ts.left];
        uint32_t meta      = static_cast<uint32_t>(d.feature[g]);
        meta |= primary_meta(g) & (META_DEFAULT_LEFT | META_CATEGORICAL);
        if (swapped) meta |= CMETA_SWAPPED;
        cn.push_back(compact_value(g, ts.is_cat));
        cn.push_back(meta);
        coff.push_back(1);
        lb.push_back(static_cast<uint32_t>(n_leaf));
        if (!sp) {
          double thr = 0;
          if (!ts.is_cat) {
            const uint64_t v = primary_value(g);
            std::memcpy(&thr, &v, 8);
          }
          ex.push_back(thr);
        }
        stack.push_back({swapped ? ts.left : ts.right, static_cast<int64_t>(n_int), true});
        stack.push_back({swapped ? ts.right : ts.left, static_cast<int64_t>(n_int), false});  // popped next
      }
      if (cn.size() / 2 >= (uint64_t(1) << 31) || n_leaf >= (uint64_t(1) << 31)) {
        clear_compact();
        return;
      }
      // the top T levels as a complete heap; a leaf above the last level fills its whole subtree
      heap.assign(heap_n * 2, 0);
      heap[1] = 0;
      uint8_t* top = out.c_top.data() + static_cast<size_t>(p) * top_bytes;
      for (size_t h = 1; h < heap_n; ++h) {
        const int32_t rel = heap[h];
        const int64_t g   = base + rel;
        uint32_t value = 0x7F800000u, meta = 0;  // padding: "x < +inf", both children the same leaf
        if (d.node_kind[g] == B2FIL_NODE_LEAF) {
          heap[2 * h] = heap[2 * h + 1] = rel;
        } else {
          const Test ts   = normalise(d, g, precision);
          heap[2 * h]     = ts.left;
          heap[2 * h + 1] = ts.right;
          const uint32_t k = number[rel];
          value            = cn[static_cast<size_t>(k) * 2];
          meta             = cn[static_cast<size_t>(k) * 2 + 1] &
                 ~(CMETA_FIRST_LEAF | CMETA_SECOND_LEAF | CMETA_SWAPPED);
          if (!sp) out.c_top_src[static_cast<size_t>(p) * heap_n + h] = k;
        }
        std::memcpy(top + h * 8, &value, 4);
        std::memcpy(top + h * 8 + 4, &meta, 4);
      }
      for (size_t e = 0; e < heap_n; ++e) {
        // exit = {internal node to continue at, leaves before it} or {leaf | flag, unused}
        const int32_t rel  = heap[heap_n + e];
        const bool is_leaf = d.node_kind[base + rel] == B2FIL_NODE_LEAF;
        uint32_t exit[2]   = {number[rel], 0u};
        if (is_leaf) {
          exit[0] |= C_EXIT_LEAF;
        } else {
          exit[1] = lb[number[rel]];
        }
        std::memcpy(top + heap_n * 8 + e * 8, exit, 8);
      }
    }
    if (fb + bits_for(max_off) > 27) {
      clear_compact();
      return;
    }
    const size_t n_int = cn.size() / 2;
    for (size_t k = 0; k < n_int; ++k) cn[k * 2 + 1] |= coff[k] << fb;
    out.c_nodes.swap(cn);
    // nodes are fetched as aligned pairs: an even count, and never an empty array
    if (out.c_nodes.empty() || (out.c_nodes.size() / 2) % 2 != 0) out.c_nodes.resize(out.c_nodes.size() + 2, 0);
    if (lb.empty()) lb.push_back(0);
    if (!sp && ex.empty()) ex.push_back(0.0);
    out.view.c_enabled      = 1;
    out.view.c_top_levels   = T;
    out.view.c_feat_bits    = fb;
    out.view.c_bottom_steps = std::max(0, maxd - T);
    out.view.c_top_stride   = static_cast<int64_t>(top_bytes);
  }

  void clear_compact()
  {
    out.c_nodes.clear();
    out.c_leaves_before.clear();
    out.c_exact.clear();
    out.c_leaf_payload.clear();
    out.c_leaf_ids.clear();
    out.c_top.clear();
    out.c_top_src.clear();
    out.view.c_enabled = 0;
  }
};

}  // namespace

int pack_forest(const b2fil_forest_desc& desc, const b2fil_create_opts& opts,
                int (*dense_ok)(int, int, int, int), PackedForest& out, std::string& err)
{
  if (opts.precision != B2FIL_F32 && opts.precision != B2FIL_F64) {
    err = "precision must be B2FIL_F32 or B2FIL_F64";
    return B2FIL_ERR_INVALID_ARG;
  }
  if (opts.layout < B2FIL_LAYOUT_DEPTH_FIRST || opts.layout > B2FIL_LAYOUT_LAYERED) {
    err = "unknown layout";
    return B2FIL_ERR_INVALID_ARG;
  }
  if (opts.storage < B2FIL_STORAGE_AUTO || opts.storage > B2FIL_STORAGE_SPARSE) {
    err = "unknown storage";
    return B2FIL_ERR_INVALID_ARG;
  }
  if (opts.align_bytes < 0 || (opts.align_bytes & (opts.align_bytes - 1)) != 0) {
    err = "align_bytes must be 0 or a power of two";
    return B2FIL_ERR_INVALID_ARG;
  }
  Packer pk(desc, opts, out, err);
  int rc = pk.validate();
  if (rc != B2FIL_OK) return rc;
  rc = pk.measure();
  if (rc != B2FIL_OK) return rc;
  out.precision   = opts.precision;
  out.align_bytes = opts.align_bytes;
  out.n_nodes_in  = desc.tree_offsets[desc.n_trees];
  pk.common_tables();
  const int max_depth = *std::max_element(pk.tree_depth.begin(), pk.tree_depth.end());

  ForestView& v     = out.view;
  v.n_trees         = desc.n_trees;
  v.n_features      = desc.n_features;
  v.n_outputs       = desc.n_outputs;
  v.leaf_vector_len = desc.leaf_vector_len;
  v.postproc        = desc.postproc;
  v.has_categorical = pk.has_cat ? 1 : 0;
  v.cat_inline      = pk.cat_inline ? 1 : 0;
  v.max_depth       = max_depth;
  v.layout          = opts.layout;
  v.sigmoid_alpha   = desc.sigmoid_alpha;
  v.ratio_c         = desc.ratio_c;

  bool dense = false;
  // 2: only the traversal over rank-quantised rows fits, so dense storage stands or falls with
  // the rank tables
  int fit = 0;
  if (opts.storage != B2FIL_STORAGE_SPARSE) {
    fit = max_depth <= 16 ? dense_ok(max_depth, opts.precision, desc.n_features, desc.n_outputs) : 0;
    bool fits = fit == 1 || (fit == 2 && opts.row_quantization == 0);
    if (fit == 2 && opts.storage == B2FIL_STORAGE_AUTO) {
      // The rank pre-pass costs time in proportion to the features of a row, the walks in
      // proportion to the nodes a row visits.  With few visits per feature the sparse kernels,
      // which rank nothing, are faster.  Measured break-even in node visits per feature and row
      // (complete trees of depth 4 to 10, 100 to 1000 trees): about 2 at 1024 features, where
      // the sparse forest still gets a compact image with 24 warps per CTA; about 0.33 at 1536,
      // where that image runs with few warps; about 1.1 at 2048 and 3000, where there is no
      // compact image but the pre-pass has more feature groups than half the SMs and reads
      // every row in 128-byte pieces.
      const double nodes_per_tree = static_cast<double>(out.n_nodes_in) / std::max(1, desc.n_trees);
      const double visits = desc.n_trees * std::min<double>(max_depth, std::log2(nodes_per_tree + 1.0));
      const double per_feature = desc.n_features < 1280 ? 2.0 : (desc.n_features <= 1792 ? 0.33 : 1.1);
      if (visits < per_feature * desc.n_features) fits = false;
    }
    if (opts.storage == B2FIL_STORAGE_DENSE) {
      if (!fits) {
        err = "dense storage cannot hold this forest: depth " + std::to_string(max_depth) +
              " with " + std::to_string(desc.n_features) +
              " features exceeds the shared memory of one SM";
        return B2FIL_ERR_UNSUPPORTED;
      }
      dense = true;
    } else if (fits) {
      // padded size against the real size: padding a ragged forest is worth it only while the
      // padded forest stays small (it streams through shared memory once per row tile)
      const double padded = static_cast<double>(desc.n_trees) * std::ldexp(2.0, max_depth);
      dense = padded <= 4.0 * static_cast<double>(out.n_nodes_in) + 4096.0 ||
              padded * 6.0 <= 8.0 * 1024 * 1024;
    }
  }
  if (!dense) return pk.pack_sparse();
  rc = pk.pack_dense(max_depth);
  if (rc != B2FIL_OK) return rc;
  if (opts.row_quantization == 0) {
    const bool ok = opts.precision == B2FIL_F32 ? pk.build_quantised<float>(max_depth)
                                                : pk.build_quantised<double>(max_depth);
    if (!ok) {
      out.q_nodes.clear();
      out.q_thresholds.clear();
      out.q_top.clear();
      out.q_nodes_ids.clear();
      out.q_lut.clear();
      out.q_feats.clear();
      out.q_groups.clear();
      out.q_blob.clear();
      out.view.q_enabled        = 0;
      out.view.q_max_blob_bytes = 0;
    }
  }
  if (fit == 2 && !out.view.q_enabled) {
    // no rank tables for this forest (category sets too large, a feature used both ways, ...)
    // and no other dense kernel that fits: sparse storage after all
    if (opts.storage == B2FIL_STORAGE_DENSE) {
      err = "dense storage cannot hold this forest: its row tile only fits as ranks and the "
            "forest cannot be rank-quantised";
      return B2FIL_ERR_UNSUPPORTED;
    }
    b2fil_create_opts sparse_opts = opts;
    sparse_opts.storage           = B2FIL_STORAGE_SPARSE;
    PackedForest fresh;
    rc = pack_forest(desc, sparse_opts, dense_ok, fresh, err);
    if (rc == B2FIL_OK) out = std::move(fresh);
    return rc;
  }
  return B2FIL_OK;
}

}  // namespace b2fil
