// Host-side interface between the launch code (kernels.cu) and the translation units that
// instantiate the traversal kernels over rank-quantised rows.
#pragma once

#include <cuda_runtime.h>

#include <string>

#include "kernels.hpp"

namespace b2fil {

// One launch of a quantised traversal kernel.
struct QLaunch {
  PredictParams p;
  const uint16_t* Q;      // rank image of the chunk
  const int32_t* flags;   // per tile: non-zero when the tile holds a NaN
  DenseCfg c;
  int grid;
  cudaStream_t stream;
};

// Raise the dynamic shared memory limit of `kernel` on the current device to `bytes` (cached per
// device and kernel).
int set_smem_bytes(const void* kernel, size_t bytes, std::string& err);

// fp32, scalar leaves, no categorical tests, depth 4..10, six trees in flight; `top6` takes the
// top nodes of every tree from p.q_top (at most kQTopTrees trees).
int launch_q_top6(const QLaunch& L, std::string& err);
int launch_q_plain6(const QLaunch& L, std::string& err);
// fp32, scalar leaves, no categorical tests, depth 4..10, four trees in flight.
int launch_q_plain4(const QLaunch& L, std::string& err);
// fp32, scalar leaves, no categorical tests, depth 9..10, two or three trees in flight.
int launch_q_plain23(const QLaunch& L, std::string& err);
// fp32, vector leaves, no categorical tests, depth 4..10, six or four trees in flight.
int launch_q_vec(const QLaunch& L, std::string& err);
// fp32, scalar leaves, no categorical tests, any depth, 1, 2 or 4 trees in flight: the walk that
// fetches both children of a node ahead of the test (for launch shapes with few walks in flight).
int launch_q_pair(const QLaunch& L, std::string& err);
// fp32 scalar leaves of depth 9 and 10, two to four trees in flight, payloads left in global memory.
int launch_q_leafg(const QLaunch& L, std::string& err);
// Forests with categorical tests: every precision, output mode and depth; 1, 2 or 4 trees in
// flight (depth-specialised bodies for fp32 scalar leaves of depth 4..8 with four trees).
int launch_q_cat(const QLaunch& L, int mode, bool f64, std::string& err);
// Everything else: generic depth, every precision and output mode; 1, 2 or 4 trees in flight.
int launch_q_generic(const QLaunch& L, int mode, bool f64, std::string& err);

// Sparse forests with a compact image (kernels_sparse_c.cu).
constexpr int kCompactTreesInFlight = 4;
struct CompactCfg {
  int rows_per_tile;  // R
  int tree_groups;    // G
  int stages;         // S: depth of the ring of heap batches
  size_t smem_bytes;
  int threads;
  int grid;
  int splits;         // CTAs that share the tree batches of a row tile (small batches), else 1
};
// Value of a named tuning knob (b2fil_set_tuning), or `fallback` when it was never set.
int tuning_value(const char* key, int fallback);
void set_tuning_value(const char* key, int value);
// Launch shape for `n_rows` rows starting from tiles of `rows_per_tile`; false when the forest has
// no compact image or no shape fits shared memory (the plain sparse kernel runs then).
// `may_split`: small batches may split the forest over CTAs (needs scratch for reduced outputs).
bool compact_config(const ForestView& f, bool reduce, int rows_per_tile, int64_t n_rows,
                    int sm_count, bool may_split, CompactCfg& cfg);
int launch_sparse_compact(const PredictParams& p, int mode, const CompactCfg& c,
                          cudaStream_t stream, cudaMemPool_t pool, std::string& err,
                          int64_t* launches);
// Second step of a split prediction: add the raw sums `partial` [split][output][row] and finish
// the rows (kernels.cu).
void launch_finish_rows(const PredictParams& p, void* partial, int n_splits, bool f64,
                        cudaStream_t stream);

}  // namespace b2fil
