// Launch interface of the prediction kernels (host side).
#pragma once

#include <cuda_runtime.h>

#include <string>

#include "forest.hpp"

namespace b2fil {

// Everything a prediction launch needs; passed to kernels by value.
struct PredictParams {
  ForestView f;
  const void* X;       // device, row-major, forest precision
  int64_t n_rows;
  int64_t row_stride;  // elements between rows
  void* out;           // device
  int32_t kind;        // B2FIL_INFER_*
  double threshold;    // binary decision threshold of B2FIL_INFER_CLASS
  int32_t* status;     // device word: set non-zero when a bounded wait inside a kernel ran out
  // HOST memory, never read on the device: three top nodes per tree of the rank-quantised copy
  // (PackedForest::q_top), or null; the launch code copies them into a kernel parameter
  const uint32_t* q_top;
};

// Shape of one dense launch.
struct DenseCfg {
  int rows_per_tile;   // R: rows staged in shared memory per CTA, multiple of 32
  int tree_groups;     // G: warp groups that split the trees of a batch
  int trees_in_flight; // NT: trees one warp walks at once
  int stages;          // S: depth of the tree pipeline
  size_t smem_bytes;
  int threads;
  int sub_batches;     // K: sub-batches of G * NT trees per stage (quantised kernel)
  int leaves_global;   // quantised kernel: the stages hold test nodes only, payloads stay in global memory
};

// Largest dynamic shared memory a CTA may use on sm_100 (227 KiB).
constexpr size_t kMaxSmemBytes = 227 * 1024;

// Pick a dense launch shape for `n_rows` rows; false when no shape fits shared memory.
bool dense_config(int depth, int precision, int n_features, int n_outputs, bool reduce_kind,
                  int64_t n_rows, int chunk_size, int sm_count, DenseCfg& cfg);

// Can the dense kernels run forests of this shape?  0 no, 1 yes, 2 only the traversal over
// rank-quantised rows.
int dense_ok(int depth, int precision, int n_features, int n_outputs);

// Enqueue a prediction on `stream`.  Returns B2FIL_OK or an error code with `err` set.
// `launches` (optional) is incremented by the number of kernels enqueued.
// Forests with rank-quantised rows take stream-ordered scratch for the ranks from `pool`.
int launch_predict(const PredictParams& p, int chunk_size, int sm_count, cudaStream_t stream,
                   cudaMemPool_t pool, std::string& err, int64_t* launches);

// Same as launch_predict for forests that predict on rank-quantised rows, except that the rank
// image goes into a fixed device array inside the library instead of pool memory: nothing is
// allocated.  `device` is the ordinal of the current device.  The whole batch must fit the array.
int launch_predict_fixed_scratch(const PredictParams& p, int chunk_size, int sm_count, int device,
                                 cudaStream_t stream, std::string& err, int64_t* launches);

// What the calling thread's most recent launch_predict* call enqueued: kernel family, template
// arguments and launch shape, e.g. "quantise_kernel<float> + dense_q_top_kernel<float,scalar,
// NT=6,DEPTH=8> R=256 G=3 S=2 K=2".  Empty before the first launch.
std::string last_launch_variant();

// Launch a one-CTA kernel whose only work is a bounded wait that nothing ends (an mbarrier that
// never receives its arrival): after `tries` tries it sets *status exactly like the prediction
// kernels do when one of their waits runs out, and returns.  Exercises the timeout reporting.
int launch_bounded_wait_selftest(int32_t* status, uint32_t tries, cudaStream_t stream,
                                 std::string& err);

}  // namespace b2fil
