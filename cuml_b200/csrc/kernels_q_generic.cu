// dense_q_kernel with the depth read at run time, forests without categorical tests.
#include "dense_q.cuh"

namespace b2fil {
namespace {
template <typename T>
int launch_generic(const QLaunch& L, int mode, std::string& err)
{
  switch (L.c.trees_in_flight) {
    case 4: return launch_q_modes<T, 4, false>(L, mode, err);
    case 2: return launch_q_modes<T, 2, false>(L, mode, err);
    default: return launch_q_modes<T, 1, false>(L, mode, err);
  }
}
}  // namespace

int launch_q_generic(const QLaunch& L, int mode, bool f64, std::string& err)
{
  return f64 ? launch_generic<double>(L, mode, err) : launch_generic<float>(L, mode, err);
}
}  // namespace b2fil
