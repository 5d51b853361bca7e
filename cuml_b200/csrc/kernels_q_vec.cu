// dense_q_kernel<float, vector leaves, depth 4..10, no categorical tests>, six or four trees in
// flight: random-forest classifiers in the scikit-learn style (every leaf holds one value per
// class) with depth-specialised, fully unrolled walks.
#include "dense_q.cuh"

namespace b2fil {
namespace {
template <int NT>
int launch_vec(const QLaunch& L, std::string& err)
{
  switch (L.p.f.dense_depth) {
    case 4: return launch_q<float, MODE_VECTOR, NT, 4, false>(L, err);
    case 5: return launch_q<float, MODE_VECTOR, NT, 5, false>(L, err);
    case 6: return launch_q<float, MODE_VECTOR, NT, 6, false>(L, err);
    case 7: return launch_q<float, MODE_VECTOR, NT, 7, false>(L, err);
    case 8: return launch_q<float, MODE_VECTOR, NT, 8, false>(L, err);
    case 9: return launch_q<float, MODE_VECTOR, NT, 9, false>(L, err);
    default: return launch_q<float, MODE_VECTOR, NT, 10, false>(L, err);
  }
}
}  // namespace

int launch_q_vec(const QLaunch& L, std::string& err)
{
  return L.c.trees_in_flight == 6 ? launch_vec<6>(L, err) : launch_vec<4>(L, err);
}
}  // namespace b2fil
