// dense_q_kernel for forests with categorical tests.
#include "dense_q.cuh"

namespace b2fil {
namespace {
template <typename T>
int launch_cat(const QLaunch& L, int mode, std::string& err)
{
  switch (L.c.trees_in_flight) {
    case 4: return launch_q_modes<T, 4, true>(L, mode, err);
    case 2: return launch_q_modes<T, 2, true>(L, mode, err);
    default: return launch_q_modes<T, 1, true>(L, mode, err);
  }
}
}  // namespace

int launch_q_cat(const QLaunch& L, int mode, bool f64, std::string& err)
{
  if (!f64 && mode == MODE_SCALAR && L.c.trees_in_flight == 4) {
    // fp32 scalar leaves: depth-specialised bodies
    switch (L.p.f.dense_depth) {
      case 4: return launch_q<float, MODE_SCALAR, 4, 4, true>(L, err);
      case 5: return launch_q<float, MODE_SCALAR, 4, 5, true>(L, err);
      case 6: return launch_q<float, MODE_SCALAR, 4, 6, true>(L, err);
      case 7: return launch_q<float, MODE_SCALAR, 4, 7, true>(L, err);
      case 8: return launch_q<float, MODE_SCALAR, 4, 8, true>(L, err);
      default: break;
    }
  }
  return f64 ? launch_cat<double>(L, mode, err) : launch_cat<float>(L, mode, err);
}
}  // namespace b2fil
