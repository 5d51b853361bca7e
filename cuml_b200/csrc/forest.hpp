// Packed-forest types shared by the host packer, the kernels and the C-ABI layer.
//
// Two device storages exist.
//
// DENSE: every tree is padded to a complete binary tree of depth D (the forest's maximum depth)
// and stored in heap order with 1-based indices: the root is node 1, the children of node i are
// 2i and 2i+1, level d is [2^d, 2^(d+1)), leaf slot j is heap index 2^D + j.  One tree is one
// contiguous block
//     [ 2^D test nodes (entry 0 unused) ][ 2^D leaf payloads ]
// so that a whole tree moves to shared memory with one bulk copy and no child index is stored.
//
// SPARSE: nodes keep an offset to their children and honour the requested node order
// (depth-first: left child adjacent, offset to the right child; breadth-first / layered:
// children adjacent to each other, offset to the left child).
//
// In both storages every numerical test is normalised at import to "x < threshold goes left" and
// every categorical test to "listed category goes right", by swapping children and moving
// thresholds to the next representable value where needed, so the kernels evaluate one operator.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/b2fil.h"

namespace b2fil {

// ---- meta word of a test node -----------------------------------------------------------------
// bit 31: a missing value goes left; bit 30: categorical test; bit 29: leaf (sparse only).
// Dense nodes keep the feature index in bits 0..29.  The two top bits fall off the end of the
// 32-bit shared-memory address when the meta word is multiplied by a row stride that is a
// multiple of four bytes, so the hot loop never masks them.
constexpr uint32_t META_DEFAULT_LEFT = 0x80000000u;
constexpr uint32_t META_CATEGORICAL  = 0x40000000u;
constexpr uint32_t META_LEAF         = 0x20000000u;
constexpr uint32_t META_LOW29        = 0x1FFFFFFFu;

// ---- node records -----------------------------------------------------------------------------
struct DenseNodeF {  // 8 bytes
  uint32_t value;    // float threshold bits | inline category bitset | category pool offset
  uint32_t meta;     // flags | feature
};
struct DenseNodeD {  // 16 bytes
  uint64_t value;    // double threshold bits | bitset / pool offset in the low word
  uint32_t meta;
  uint32_t pad;
};
struct SparseNode8 {  // fp32, compact: feature and child offset share the low 29 meta bits
  uint32_t value;     // threshold | bitset | pool offset | leaf scalar | leaf-vector index
  uint32_t meta;      // flags | offset << feat_bits | feature
};
struct SparseNode16F {  // fp32, wide
  uint32_t value;
  uint32_t meta;  // flags | feature
  uint32_t offset;
  uint32_t pad;
};
struct SparseNode16D {  // fp64
  uint64_t value;
  uint32_t meta;  // flags | feature
  uint32_t offset;
};

// ---- rank quantisation of rows (dense storage without categorical tests) -----------------------
// For every feature the distinct thresholds of the forest are sorted: T[0] < T[1] < ...  The rank
// of a value, r(x) = #{i : T[i] <= x}, decides every test on that feature exactly:
//     x < T[j]  <=>  r(x) <= j.
// A pre-pass kernel turns each row into 16-bit ranks (NaN becomes 0x3FFF); the traversal kernel
// then reads 2-byte values and 4-byte nodes
//     bits 31..17: j (0x7FFF = never left)   bit 16: missing goes right
//     bits 15..2: feature                    bits 1..0: zero
// so a test is one signed subtraction: right <=> int(node) - (rank << 17) < 0 (the flag in bit 16
// is below the weight of one rank and cannot change the sign), and the low half is the feature
// times four: one 16-bit x 8-bit dot-product instruction scales it by a quarter of the byte
// stride between features and adds the row's address.
// Categorical features (every test on them is categorical, every listed category below 32) keep
// their place in the same scheme: the "rank" of a value is its category (Q_NO_CATEGORY when it is
// negative, fractional-truncated out of range or too large), and in such forests every node is
// 8 bytes {node, 32-bit category set} (a numerical node holds an empty set), fetched with one
// load; a set bit sends the row right.  (A categorical node is recognisable by j = Q_MAX_RANK_FIELD; the walk does not need
// to know, and the low half of every node stays a clean feature * 4 for the address arithmetic.)  The sets are stored bit-reversed (category c in bit 31 - c) and a categorical node
// carries the largest rank, so its rank comparison always says "left" and the walk can simply OR
// the two answers: sign(node - (code << 17)) | sign(set << code).
// The rank is found through a per-feature bucket table: bucket(x) = clamp(int(fma(x, scale,
// offset)), 0, n_buckets-1) is monotone in x, lut[b] is the number of thresholds in buckets below
// b (all of them are <= x), thresholds of higher buckets are all > x, so the rank is lut[b] plus
// the number of thresholds <= x in a window of 2^steps - 1 entries starting at lut[b], found with
// `steps` branch-free halvings (2^steps exceeds the fullest bucket; the array ends with NaN
// padding, for which `T <= x` is false).
struct QFeature {      // host-side table of one feature
  uint32_t t_off;      // first threshold of the feature in PackedForest::q_thresholds
  uint32_t lut_off;    // first entry of the feature's bucket table in PackedForest::q_lut
  uint32_t m;          // number of distinct thresholds
  uint32_t n_buckets;
  uint32_t max_occupancy;  // thresholds in the fullest bucket
  uint32_t is_cat;         // categorical feature: no tables
  double scale;        // bucket(x) = fma(x, scale, offset) evaluated in the forest precision
  double offset;
};
// Device tables are grouped: a power-of-two run of GF consecutive features whose tables fit one
// CTA's shared memory forms a group, stored as one contiguous blob that the pre-pass pulls in with
// a single bulk copy:
//   [kQMaxGroupFeatures x QFeatRec][bucket tables (uint16)][thresholds + NaN padding]
// Both tables are interleaved across the group: entry k of the group's i-th feature sits at
// element k * GF + i, and every feature's columns are padded to the longest table of the group
// (zeros / NaN).  The lanes of a warp hold one feature each, so whatever entries they probe they
// read different shared-memory banks.
struct QFeatRec {      // 32 bytes
  uint32_t lut_off;    // byte offset of entry 0 from the start of the blob; entry k: + k * GF * 2
  uint32_t thr_off;    // same for the thresholds; entry k: + k * GF * sizeof(T)
  uint32_t nbm1;       // n_buckets - 1
  uint32_t is_cat;     // 1: the value's code is its category, no table lookup
  double scale, offset;
};
struct QGroup {        // 32 bytes
  uint32_t f_begin, f_end;
  uint32_t blob_off;   // byte offset of the group's blob in ForestView::q_blob (16-byte multiple)
  uint32_t blob_bytes; // 16-byte multiple
  uint32_t steps;      // halvings of the window search, shared by the group's features
  uint32_t pad[3];
};
constexpr uint32_t Q_NAN_CODE      = 0x3FFFu;
constexpr uint32_t Q_MAX_RANK      = 0x3FFEu;
constexpr uint32_t Q_NO_CATEGORY   = 0x3FFEu;
constexpr uint32_t Q_MAX_FEATURES  = 0x4000u;
constexpr uint32_t Q_FEATURE_FIELD = 0xFFFCu;  // feature << 2
constexpr uint32_t Q_FEATURE_SHIFT = 2;
constexpr uint32_t Q_DEFAULT_RIGHT = 0x10000u;  // missing values go right (stored in this sense: << 15 makes it the sign)
constexpr uint32_t Q_RANK_SHIFT    = 17;
constexpr uint32_t Q_NEVER_LEFT    = 0x7FFFu;  // j of a test that no value passes
constexpr uint32_t Q_MAX_RANK_FIELD = 0x3FFFu;  // j of a test that every code passes (categorical nodes)
// Forests of at most this many trees, at least two levels deep and without categorical tests also
// keep the three top nodes of every tree on the host: the traversal kernel takes them as a launch
// parameter and reads them through the constant cache instead of shared memory.
constexpr int kQTopTrees = 2048;
// Vector leaves of forests with at most this many outputs are stored in the tree blocks of the
// rank-quantised image (and summed in registers): the walk then never leaves shared memory.
constexpr int kQInlineClasses = 4;

// ---- compact image of a sparse forest -----------------------------------------------------------
// Deep, ragged forests are bound by the chain of dependent node fetches from L2 / HBM.  Sparse
// forests whose fields fit therefore carry a second image built for exactly that:
//  * internal nodes only, 8 bytes each {value, meta}, in depth-first order per tree, the child
//    with the larger subtree first (rows are more likely to go where the training data went), so
//    the node array is half the size of an array that also holds the leaves and a quarter of the
//    16-byte fp64 array: it stays in L2.  The first child of node k is node k + 1: an aligned
//    16-byte load brings a node and its neighbour, and half of the steps to a first child need no
//    fetch at all;
//  * leaves live in their own arrays (payload, id), numbered in the same depth-first order.  A
//    walk carries the pair (k, L) = (internal node, number of leaves that precede it); with
//    `off` = 1 + internal nodes of the first child's subtree,
//        first child : k + 1,   L          second child : k + off, L + off
//    (a subtree with m internal nodes has m + 1 leaves), and two flags in the node say when the
//    child reached is a leaf, whose number is then L (first) or L + off (second);
//  * meta = default-left << 31 | categorical << 30 | first-is-leaf << 29 | second-is-leaf << 28 |
//    first-child-is-the-right-child << 27 | off << feat_bits | feature;
//  * fp64 forests keep `value` = the largest float <= threshold, and the kernel stages rows as
//    floats rounded down: xl < value proves x < threshold, xl > value proves x > threshold, and
//    only when xl == value the row's double and the exact threshold (`c_exact`) are read (one in
//    2^24 visits on continuous data), so 8-byte nodes and 4-byte row values decide every fp64
//    test exactly;
//  * the top `c_top_levels` levels of every tree are also stored as a complete heap
//    [2^T nodes {value, feature | flags}][2^T exits {k, L}], which the kernel streams through
//    shared memory: a walk starts with T steps that cost no global fetch and leaves the heap
//    through an exit = the pair (k, L) to continue at, or the leaf reached (bit 31 of k).
constexpr uint32_t CMETA_FIRST_LEAF  = 0x20000000u;
constexpr uint32_t CMETA_SECOND_LEAF = 0x10000000u;
constexpr uint32_t CMETA_SWAPPED     = 0x08000000u;  // the first (adjacent) child is the right child
constexpr uint32_t CMETA_LOW27       = 0x07FFFFFFu;
constexpr uint32_t C_EXIT_LEAF      = 0x80000000u;
constexpr uint32_t C_NO_NODE        = 0xFFFFFFFFu;
constexpr int kCMaxTopLevels        = 10;
struct CompactNode {  // 8 bytes
  uint32_t value;     // float threshold bits (fp64 forests: rounded down) | bitset | pool offset
  uint32_t meta;
};
// Levels of every tree that go into the heap (0: no compact image).  Measured on a 200-tree
// depth-20 forest: the walk below the heap is bound by how many dependent fetches an SM keeps in
// flight (warps x walks per warp, and the L1 that tracks the misses: it shrinks as shared memory
// grows), so heap levels are only worth their shared memory while they do not cost warps.  Eight
// levels (4 KB per tree) with 28 warps on 128-row tiles were the best trade (9.5e7 rows/s; six
// levels 8.9e7, nine levels - room for 12 warps only - 5.8e7).
constexpr int kCDefaultTopLevels = 8;
// With many features the row tile leaves little room: the heaps then get fewer levels, so that
// 24 warps still fit under the 160 KiB that the launch code prefers (one warp per CTA next to
// eight-level heaps ran a 1024-feature forest at 3.7e7 rows/s).
inline int compact_pick_top_levels(int elem_bytes, int n_features, int n_outputs, int max_depth)
{
  const size_t hard = 218 * 1024, soft = 160 * 1024;
  constexpr int kWalks = 4;  // trees a warp walks at once (kCompactTreesInFlight)
  int fallback = 0;
  for (int T = kCDefaultTopLevels; T >= 1; --T) {
    const size_t heap = static_cast<size_t>(16) << T;
    for (int R = 128; R >= 32; R /= 2) {
      const size_t tile = static_cast<size_t>(n_features) * (R + 1) * 4;  // rows are staged as floats
      const int G       = (24 + R / 32 - 1) / (R / 32);
      const size_t acc  = static_cast<size_t>(G) * n_outputs * R * elem_bytes;
      if (tile + acc + heap * G * kWalks <= soft) return std::max(1, std::min(T, max_depth));
      if (fallback == 0 && tile + static_cast<size_t>(8) * n_outputs * R * elem_bytes + heap * 8 <= hard)
        fallback = T;
    }
  }
  return fallback == 0 ? 0 : std::max(1, std::min(fallback, max_depth));
}

enum NodeFormat : int32_t {
  FMT_DENSE_F   = 0,
  FMT_DENSE_D   = 1,
  FMT_SPARSE_8  = 2,
  FMT_SPARSE_16F = 3,
  FMT_SPARSE_16D = 4,
};

// Device view handed to kernels by value.  Pointers are device pointers on the forest's device.
struct ForestView {
  int32_t format;
  int32_t n_trees;
  int32_t n_features;
  int32_t n_outputs;
  int32_t leaf_vector_len;
  int32_t postproc;
  int32_t has_categorical;
  int32_t cat_inline;       // 1: every category list fits a 32-bit inline bitset
  int32_t max_depth;        // loop bound of sparse traversal
  int32_t dense_depth;      // D
  int32_t feat_bits;        // SparseNode8: width of the feature field
  int32_t layout;
  int64_t tree_stride;      // dense: bytes between trees
  const void* nodes;        // dense: tree blocks; sparse: node array
  const uint32_t* roots;    // sparse: index of every tree's root in `nodes`
  const uint32_t* leaf_ids; // dense: [n_trees << D] id per leaf slot; sparse: [n_nodes] id per node
  const uint32_t* cat_pool; // [n_words, words...] records of large category lists
  const int32_t* tree_class;// [n_trees] output a scalar leaf adds to (packed tree order)
  const int32_t* tree_orig; // [n_trees] index of the packed tree in the description
  const void* leaf_vectors; // [n_vectors * n_outputs] of the forest precision
  const void* out_scale;    // [n_outputs] 1/divisor of average_tree_output (or 1)
  const void* out_bias;     // [n_outputs] base scores
  double sigmoid_alpha;
  double ratio_c;
  // rank-quantised copy of a dense forest (q_enabled != 0)
  int32_t q_enabled;
  int32_t q_n_groups;
  int32_t q_has_cat;            // 1: tree blocks carry a third array of 32-bit category sets
  int32_t q_trees_in_order;     // 1: packed tree t is the caller's tree t (tree_orig is the identity)
  int32_t q_leaf_bytes;         // bytes per leaf payload: the element size (scalar, or index of the
                                // leaf's vector), or n_outputs elements when the vectors of a
                                // forest with few outputs sit in the tree blocks themselves
  int32_t q_pad_;
  int64_t q_tree_stride;        // bytes between trees: 2^D * (node bytes + leaf bytes), 16-byte multiple
  const void* q_nodes;          // [n_trees] blocks of [2^D nodes][2^D leaf payloads]; a node is a
                                // uint32, or {uint32 node, uint32 category set} when q_has_cat
  const void* q_nodes_ids;      // same blocks with the leaf id (uint32) in every leaf payload slot:
                                // what the traversal streams when it reports leaf ids
  int64_t q_max_blob_bytes;     // largest group blob
  const unsigned char* q_blob;  // group blobs
  const QGroup* q_groups;       // [q_n_groups]
  // compact image of a sparse forest (c_enabled != 0), see above
  int32_t c_enabled;
  int32_t c_top_levels;         // T
  int32_t c_feat_bits;
  int32_t c_bottom_steps;       // most steps a walk takes below the heap
  int64_t c_top_stride;         // bytes between the heaps of two trees: 2^T * 16
  const CompactNode* c_nodes;   // [n_internal, rounded up to even]: pairs are loaded together
  const double* c_exact;        // [n_internal] exact thresholds (fp64 forests), else null
  const void* c_leaf_payload;   // [n_leaves] scalar in the forest precision or vector index
  const uint32_t* c_leaf_ids;   // [n_leaves] id of the leaf in the imported model
  const unsigned char* c_top;   // [n_trees] heaps
  const uint32_t* c_top_src;    // [n_trees << T] internal node behind every heap node (fp64), C_NO_NODE = padding
};

// Host-side result of packing, before upload.
struct PackedForest {
  ForestView view{};  // pointer members unset
  int32_t precision = B2FIL_F32;
  int32_t storage   = B2FIL_STORAGE_SPARSE;
  int32_t align_bytes = 0;
  int32_t node_bytes = 0;
  int64_t n_nodes_in = 0;
  int64_t n_nodes_packed = 0;
  std::vector<uint8_t> nodes;
  std::vector<uint32_t> roots;
  std::vector<uint32_t> leaf_ids;
  std::vector<uint32_t> cat_pool;
  std::vector<int32_t> tree_class;
  std::vector<int32_t> tree_orig;
  std::vector<uint8_t> leaf_vectors;
  std::vector<uint8_t> out_scale;
  std::vector<uint8_t> out_bias;
  std::vector<uint8_t> q_nodes;
  std::vector<uint8_t> q_nodes_ids;  // q_nodes with leaf ids in the payload slots
  std::vector<uint32_t> q_top;  // root and its two children of every tree (3 words per tree), or empty
  std::vector<uint8_t> q_thresholds;
  std::vector<uint16_t> q_lut;
  std::vector<QFeature> q_feats;
  std::vector<QGroup> q_groups;
  std::vector<uint8_t> q_blob;
  std::vector<uint32_t> c_nodes;          // two words per internal node
  std::vector<uint32_t> c_leaves_before;  // L of every internal node (host only: the exits carry it)
  std::vector<double> c_exact;
  std::vector<uint8_t> c_leaf_payload;
  std::vector<uint32_t> c_leaf_ids;
  std::vector<uint8_t> c_top;
  std::vector<uint32_t> c_top_src;
};

// Bucket of a value in a feature's table; the same expression runs on the device
// (fma and float->int truncation are exactly specified, so host and device agree bit for bit).
template <typename T>
inline uint32_t q_bucket_host(T x, T scale, T offset, uint32_t n_buckets)
{
  T v = std::fma(x, scale, offset);
  v   = std::fmax(v, T(0));  // also turns NaN (inf * 0) into 0
  v   = std::fmin(v, static_cast<T>(n_buckets - 1));
  return static_cast<uint32_t>(v);
}

// Shared memory the quantisation kernel may spend on the tables of one feature group.
constexpr uint32_t kQGroupSmemBudget = 208 * 1024;
constexpr uint32_t kQMaxGroupFeatures = 32;

// Validate `desc`, normalise its tests and lay its nodes out.  Returns B2FIL_OK or an error code
// with `err` set.  `dense_ok(depth, precision, n_features, n_outputs)` tells whether the dense
// kernels can run a forest of that shape (shared-memory fit): 0 no, 1 yes, 2 only the traversal
// over rank-quantised rows (its 2-byte row tile fits where a tile of reals does not: forests with
// a thousand features and more); AUTO storage asks it.
int pack_forest(const b2fil_forest_desc& desc, const b2fil_create_opts& opts,
                int (*dense_ok)(int depth, int precision, int n_features, int n_outputs),
                PackedForest& out,
                std::string& err);

}  // namespace b2fil
