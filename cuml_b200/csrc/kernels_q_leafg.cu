// dense_q_leafg_kernel: fp32 scalar leaves without categorical tests, depth 9 and 10, two to four
// trees in flight, leaf payloads fetched from global memory instead of riding in the stages.
#include "dense_q.cuh"

namespace b2fil {
namespace {
template <int NT, int DEPTH>
int launch_leafg(const QLaunch& L, std::string& err)
{
  auto k = dense_q_leafg_kernel<NT, DEPTH>;
  const int rc = set_smem_bytes(reinterpret_cast<const void*>(k), L.c.smem_bytes, err);
  if (rc != B2FIL_OK) return rc;
  k<<<L.grid, L.c.threads, L.c.smem_bytes, L.stream>>>(L.p, L.Q, L.flags, L.c.rows_per_tile,
                                                       L.c.tree_groups, L.c.stages,
                                                       L.c.sub_batches);
  return B2FIL_OK;
}

template <int DEPTH>
int launch_leafg_depth(const QLaunch& L, std::string& err)
{
  switch (L.c.trees_in_flight) {
    case 4: return launch_leafg<4, DEPTH>(L, err);
    case 3: return launch_leafg<3, DEPTH>(L, err);
    default: return launch_leafg<2, DEPTH>(L, err);
  }
}
}  // namespace

int launch_q_leafg(const QLaunch& L, std::string& err)
{
  return L.p.f.dense_depth == 9 ? launch_leafg_depth<9>(L, err) : launch_leafg_depth<10>(L, err);
}
}  // namespace b2fil
