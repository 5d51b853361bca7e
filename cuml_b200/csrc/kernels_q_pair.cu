// dense_q_pair_kernel: fp32 scalar leaves without categorical tests, generic depth, 1, 2 or 4
// trees in flight, both children of a node fetched ahead of the test.
#include "dense_q.cuh"

namespace b2fil {
namespace {
template <int NT>
int launch_pair(const QLaunch& L, std::string& err)
{
  auto k = dense_q_pair_kernel<NT>;
  const int rc = set_smem_bytes(reinterpret_cast<const void*>(k), L.c.smem_bytes, err);
  if (rc != B2FIL_OK) return rc;
  k<<<L.grid, L.c.threads, L.c.smem_bytes, L.stream>>>(L.p, L.Q, L.flags, L.c.rows_per_tile,
                                                       L.c.tree_groups, L.c.stages,
                                                       L.c.sub_batches);
  return B2FIL_OK;
}
}  // namespace

int launch_q_pair(const QLaunch& L, std::string& err)
{
  switch (L.c.trees_in_flight) {
    case 4: return launch_pair<4>(L, err);
    case 2: return launch_pair<2>(L, err);
    default: return launch_pair<1>(L, err);
  }
}
}  // namespace b2fil
