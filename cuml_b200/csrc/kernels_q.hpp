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
// Forests with categorical tests: every precision, output mode and depth; 1, 2 or 4 trees in
// flight (depth-specialised bodies for fp32 scalar leaves of depth 4..8 with four trees).
int launch_q_cat(const QLaunch& L, int mode, bool f64, std::string& err);
// Everything else: generic depth, every precision and output mode; 1, 2 or 4 trees in flight.
int launch_q_generic(const QLaunch& L, int mode, bool f64, std::string& err);

}  // namespace b2fil
