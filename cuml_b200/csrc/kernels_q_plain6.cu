// dense_q_kernel<float, scalar leaves, 6 trees in flight, depth 4..10, no categorical tests>.
#include "dense_q.cuh"

namespace b2fil {
int launch_q_plain6(const QLaunch& L, std::string& err)
{
  switch (L.p.f.dense_depth) {
    case 4: return launch_q<float, MODE_SCALAR, 6, 4, false>(L, err);
    case 5: return launch_q<float, MODE_SCALAR, 6, 5, false>(L, err);
    case 6: return launch_q<float, MODE_SCALAR, 6, 6, false>(L, err);
    case 7: return launch_q<float, MODE_SCALAR, 6, 7, false>(L, err);
    case 8: return launch_q<float, MODE_SCALAR, 6, 8, false>(L, err);
    case 9: return launch_q<float, MODE_SCALAR, 6, 9, false>(L, err);
    default: return launch_q<float, MODE_SCALAR, 6, 10, false>(L, err);
  }
}
}  // namespace b2fil
