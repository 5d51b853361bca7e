// dense_q_kernel<float, scalar leaves, 4 trees in flight, depth 4..10, no categorical tests>.
#include "dense_q.cuh"

namespace b2fil {
int launch_q_plain4(const QLaunch& L, std::string& err)
{
  switch (L.p.f.dense_depth) {
    case 4: return launch_q<float, MODE_SCALAR, 4, 4, false>(L, err);
    case 5: return launch_q<float, MODE_SCALAR, 4, 5, false>(L, err);
    case 6: return launch_q<float, MODE_SCALAR, 4, 6, false>(L, err);
    case 7: return launch_q<float, MODE_SCALAR, 4, 7, false>(L, err);
    case 8: return launch_q<float, MODE_SCALAR, 4, 8, false>(L, err);
    case 9: return launch_q<float, MODE_SCALAR, 4, 9, false>(L, err);
    default: return launch_q<float, MODE_SCALAR, 4, 10, false>(L, err);
  }
}

// Depth 9 and 10 with two or three trees in flight: shapes whose trees are so large (8 KB at depth
// 10) that shared memory holds only a dozen of them next to the row tile.
int launch_q_plain23(const QLaunch& L, std::string& err)
{
  const int d = L.p.f.dense_depth;
  if (L.c.trees_in_flight == 3) {
    return d == 9 ? launch_q<float, MODE_SCALAR, 3, 9, false>(L, err)
                  : launch_q<float, MODE_SCALAR, 3, 10, false>(L, err);
  }
  return d == 9 ? launch_q<float, MODE_SCALAR, 2, 9, false>(L, err)
                : launch_q<float, MODE_SCALAR, 2, 10, false>(L, err);
}
}  // namespace b2fil
