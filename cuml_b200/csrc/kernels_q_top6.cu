// dense_q_top_kernel<float, scalar leaves, 6 trees in flight, depth 4..10>.
#include "dense_q.cuh"

namespace b2fil {
namespace {
template <int DEPTH>
int launch_top(const QLaunch& L, const QTop& top, std::string& err)
{
  auto k = dense_q_top_kernel<float, MODE_SCALAR, 6, DEPTH>;
  const int rc = set_smem_bytes(reinterpret_cast<const void*>(k), L.c.smem_bytes, err);
  if (rc != B2FIL_OK) return rc;
  k<<<L.grid, L.c.threads, L.c.smem_bytes, L.stream>>>(L.p, L.Q, L.flags, L.c.rows_per_tile,
                                                       L.c.tree_groups, L.c.stages,
                                                       L.c.sub_batches, top);
  return B2FIL_OK;
}
}  // namespace

int launch_q_top6(const QLaunch& L, std::string& err)
{
  // the three top nodes of every tree travel in the parameter block
  static thread_local QTop top;
  std::memcpy(top.w, L.p.q_top, static_cast<size_t>(L.p.f.n_trees) * 3 * sizeof(uint32_t));
  switch (L.p.f.dense_depth) {
    case 4: return launch_top<4>(L, top, err);
    case 5: return launch_top<5>(L, top, err);
    case 6: return launch_top<6>(L, top, err);
    case 7: return launch_top<7>(L, top, err);
    case 8: return launch_top<8>(L, top, err);
    case 9: return launch_top<9>(L, top, err);
    default: return launch_top<10>(L, top, err);
  }
}
}  // namespace b2fil
