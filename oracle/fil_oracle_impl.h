/*
 * Body of the CPU oracle, included twice by fil_oracle.c with REAL = float and REAL = double.
 * TEST INFRASTRUCTURE ONLY: nothing in the product may call this.
 *
 * Every rule cites the statement of tree-ensemble arithmetic in NVIDIA/cuml 26.10 that it
 * restates (paths inside that project).
 */

/* Decide the child for one test node.
 *  - missing value (NaN) -> default child:      cpp/src/explainer/tree_shap.cu:156, :279
 *  - categorical: reject x < 0 or |x| > 2^digits, truncate to an unsigned integer, look it up in
 *    the node's category list; a listed category goes to the right child iff cat_right:
 *                                               cpp/src/explainer/tree_shap.cu:154-165, :300-307
 *  - numerical: the comparison being true -> left child; `<=` for random forests, `<` for
 *    isolation forests:  cpp/src/decisiontree/decisiontree.cuh:379-383,
 *                        cpp/src/isolation_forest/isolation_tree_builder.cuh:354-355
 */
static inline int32_t FN(next_node)(const b2fil_forest_desc* d, int64_t base, int32_t n, REAL x)
{
  const int64_t g = base + n;
  if (x != x) { return d->default_left[g] ? d->left[g] : d->right[g]; }
  if (d->node_kind[g] == B2FIL_NODE_CATEGORICAL) {
    const REAL max_int = (REAL)((uint64_t)1 << REAL_DIGITS);
    int matched        = 0;
    if (!(x < (REAL)0) && !(FABS(x) > max_int)) {
      const uint64_t cat = (uint64_t)x;
      for (int64_t k = d->cat_ptr[g]; k < d->cat_ptr[g + 1]; ++k) {
        if ((uint64_t)d->cat_values[k] == cat) {
          matched = 1;
          break;
        }
      }
    }
    const int right_on_match = d->cat_right ? d->cat_right[g] : 1;
    return (matched == right_on_match) ? d->right[g] : d->left[g];
  }
  const REAL t = (REAL)d->threshold[g]; /* forest precision decides the compare type */
  const int o  = d->op ? d->op[g] : d->op_all;
  int cond;
  switch (o) {
    case B2FIL_OP_LT: cond = x < t; break;
    case B2FIL_OP_LE: cond = x <= t; break;
    case B2FIL_OP_GT: cond = x > t; break;
    default: cond = x >= t; break;
  }
  return cond ? d->left[g] : d->right[g];
}

static inline int32_t FN(find_leaf)(const b2fil_forest_desc* d, int t, const REAL* row)
{
  const int64_t base = d->tree_offsets[t];
  int32_t n          = 0;
  while (d->node_kind[base + n] != B2FIL_NODE_LEAF) {
    n = FN(next_node)(d, base, n, row[d->feature[base + n]]);
  }
  return n;
}

/* ---- packed walk --------------------------------------------------------------------------------
 * The same traversal over a packed copy of the forest: one 24-byte (fp32) / 32-byte (fp64) record
 * per node instead of five parallel arrays, and eight rows walked side by side through a tree so
 * that their dependent loads overlap.  Same operators, same missing-value rule, same leaves as
 * find_leaf above; it exists so that the CPU baseline that bench.py reports is not slowed down by
 * the structure-of-arrays description, which is a convenient input format and a poor layout to
 * traverse.  Forests with categorical tests keep the plain walk.  tests/test_oracle.py checks the
 * two walks against each other. */
typedef struct {
  REAL thr;
  int32_t feat;
  int32_t left, right;
  uint8_t leaf, default_left, op, pad;
} FN(pnode);

static FN(pnode)* FN(pack_nodes)(const b2fil_forest_desc* d)
{
  const int64_t total = d->tree_offsets[d->n_trees];
  for (int64_t g = 0; g < total; ++g)
    if (d->node_kind[g] == B2FIL_NODE_CATEGORICAL) return NULL;
  FN(pnode)* p = (FN(pnode)*)malloc(sizeof(FN(pnode)) * (size_t)(total > 0 ? total : 1));
  if (!p) return NULL;
  for (int64_t g = 0; g < total; ++g) {
    p[g].thr          = (REAL)d->threshold[g];
    p[g].feat         = d->feature[g];
    p[g].left         = d->left[g];
    p[g].right        = d->right[g];
    p[g].leaf         = d->node_kind[g] == B2FIL_NODE_LEAF;
    p[g].default_left = d->default_left[g] != 0;
    p[g].op           = (uint8_t)(d->op ? d->op[g] : d->op_all);
    p[g].pad          = 0;
  }
  return p;
}

#define OR_LANES 8
/* Leaves of rows r0 .. r0+n-1 (n <= OR_LANES) in tree t. */
static inline void FN(find_leaves_packed)(const FN(pnode)* nodes, int64_t base, const REAL* X,
                                          int64_t row_stride, int64_t r0, int n, int32_t* leaf)
{
  int32_t at[OR_LANES];
  for (int j = 0; j < n; ++j) at[j] = 0;
  for (;;) {
    int walking = 0;
    for (int j = 0; j < n; ++j) {
      const FN(pnode)* nd = nodes + base + at[j];
      if (nd->leaf) continue;
      const REAL x = X[(r0 + j) * row_stride + nd->feat];
      const REAL t = nd->thr;
      int cond;
      switch (nd->op) {
        case B2FIL_OP_LT: cond = x < t; break;
        case B2FIL_OP_LE: cond = x <= t; break;
        case B2FIL_OP_GT: cond = x > t; break;
        default: cond = x >= t; break;
      }
      if (x != x) cond = nd->default_left;
      at[j]   = cond ? nd->left : nd->right;
      walking = 1;
    }
    if (!walking) break;
  }
  for (int j = 0; j < n; ++j) leaf[j] = at[j];
}

/* Postprocessing of one row of summed outputs (Treelite postprocessor names; cuML sets
 * "identity" / "identity_multiclass": cpp/src/randomforest/randomforest.cu:263,267). */
static void FN(postprocess)(const b2fil_forest_desc* d, double* s)
{
  const int k = d->n_outputs;
  switch (d->postproc) {
    case B2FIL_POST_SIGMOID:
    case B2FIL_POST_MULTICLASS_OVA:
      for (int c = 0; c < k; ++c) s[c] = 1.0 / (1.0 + exp(-d->sigmoid_alpha * s[c]));
      break;
    case B2FIL_POST_EXPONENTIAL:
      for (int c = 0; c < k; ++c) s[c] = exp(s[c]);
      break;
    case B2FIL_POST_LOG1PEXP:
      for (int c = 0; c < k; ++c) s[c] = log1p(exp(s[c]));
      break;
    case B2FIL_POST_SIGNED_SQUARE:
      for (int c = 0; c < k; ++c) s[c] = (s[c] < 0 ? -1.0 : 1.0) * s[c] * s[c];
      break;
    case B2FIL_POST_HINGE:
      for (int c = 0; c < k; ++c) s[c] = s[c] > 0 ? 1.0 : 0.0;
      break;
    case B2FIL_POST_EXP_STD_RATIO:
      for (int c = 0; c < k; ++c) s[c] = exp2(-s[c] / d->ratio_c);
      break;
    case B2FIL_POST_SOFTMAX: {
      double m = s[0];
      for (int c = 1; c < k; ++c) m = s[c] > m ? s[c] : m;
      double z = 0;
      for (int c = 0; c < k; ++c) {
        s[c] = exp(s[c] - m);
        z += s[c];
      }
      for (int c = 0; c < k; ++c) s[c] /= z;
      break;
    }
    default: break;
  }
}

#define OR_BLOCK 64

int FN(fil_oracle_predict)(const b2fil_forest_desc* d, int infer_kind, const REAL* X,
                           int64_t n_rows, int64_t row_stride, void* out, double threshold,
                           int n_threads, int packed_walk)
{
  const int k       = d->n_outputs;
  const int vec     = d->leaf_vector_len > 1;
  const int n_trees = d->n_trees;
  /* number of trees feeding each output: the divisor of average_tree_output.  Random forests
   * divide by n_trees (cpp/src/randomforest/randomforest.cuh:439-441); for forests with one
   * group of trees per class the divisor is the number of trees of that class. */
  double* divisor = (double*)calloc((size_t)k, sizeof(double));
  if (!divisor) return -5;
  for (int t = 0; t < n_trees; ++t) {
    if (vec) {
      for (int c = 0; c < k; ++c) divisor[c] += 1;
    } else {
      divisor[d->class_id ? d->class_id[t] : t % k] += 1;
    }
  }
  const int64_t n_blocks = (n_rows + OR_BLOCK - 1) / OR_BLOCK;
  int failed             = 0;
  FN(pnode)* packed      = packed_walk ? FN(pack_nodes)(d) : NULL;
  if (n_threads < 1) n_threads = 1;
#pragma omp parallel num_threads(n_threads)
  {
    double* acc = (double*)malloc(sizeof(double) * OR_BLOCK * (size_t)k);
    if (!acc) {
#pragma omp atomic write
      failed = 1;
    }
#pragma omp for schedule(dynamic, 4)
    for (int64_t b = 0; b < n_blocks; ++b) {
      if (!acc) continue;
      const int64_t r0 = b * OR_BLOCK;
      const int nb     = (int)((n_rows - r0) < OR_BLOCK ? (n_rows - r0) : OR_BLOCK);
      for (int i = 0; i < nb * k; ++i) acc[i] = 0.0;
      /* trees outermost inside a row block so that a tree's nodes stay in cache */
      for (int t = 0; t < n_trees; ++t) {
        const int64_t base = d->tree_offsets[t];
        /* scalar leaf of a multi-output forest adds to class_id[t]; implicit convention
         * tree_idx % num_class: cpp/src/explainer/tree_shap.cu:589 */
        const int cls = vec ? -1 : (d->class_id ? d->class_id[t] : t % k);
        int32_t lanes[OR_LANES];
        for (int i = 0; i < nb; ++i) {
          const int64_t r = r0 + i;
          if (packed && i % OR_LANES == 0) {
            const int n = nb - i < OR_LANES ? nb - i : OR_LANES;
            FN(find_leaves_packed)(packed, base, X, row_stride, r, n, lanes);
          }
          const int32_t lf = packed ? lanes[i % OR_LANES] : FN(find_leaf)(d, t, X + r * row_stride);
          if (infer_kind == B2FIL_INFER_LEAF_ID) {
            ((uint32_t*)out)[r * n_trees + t] = (uint32_t)lf;
          } else if (infer_kind == B2FIL_INFER_PER_TREE) {
            if (vec) {
              for (int c = 0; c < k; ++c)
                ((REAL*)out)[(r * n_trees + t) * k + c] =
                  (REAL)d->leaf_value[(base + lf) * (int64_t)k + c];
            } else {
              ((REAL*)out)[r * n_trees + t] = (REAL)d->leaf_value[base + lf];
            }
          } else if (vec) {
            /* vector leaf added element-wise: cpp/src/decisiontree/decisiontree.cuh:386-388 */
            for (int c = 0; c < k; ++c)
              acc[i * k + c] += (double)(REAL)d->leaf_value[(base + lf) * (int64_t)k + c];
          } else {
            acc[i * k + cls] += (double)(REAL)d->leaf_value[base + lf];
          }
        }
      }
      if (infer_kind == B2FIL_INFER_LEAF_ID || infer_kind == B2FIL_INFER_PER_TREE) continue;
      for (int i = 0; i < nb; ++i) {
        const int64_t r = r0 + i;
        double* s       = acc + i * k;
        for (int c = 0; c < k; ++c) {
          /* average, then base score, then postprocessor
           * (cpp/src/randomforest/randomforest.cu:277-278, cpp/src/explainer/tree_shap.cu:726) */
          if (d->average_tree_output && divisor[c] > 0) s[c] /= divisor[c];
          if (d->base_scores) s[c] += d->base_scores[c];
        }
        FN(postprocess)(d, s);
        if (infer_kind == B2FIL_INFER_DEFAULT) {
          for (int c = 0; c < k; ++c) ((REAL*)out)[r * k + c] = (REAL)s[c];
        } else if (infer_kind == B2FIL_INFER_PROBA2) {
          ((REAL*)out)[r * 2 + 0] = (REAL)(1.0 - s[0]);
          ((REAL*)out)[r * 2 + 1] = (REAL)s[0];
        } else { /* B2FIL_INFER_CLASS */
          int best = 0;
          if (k == 1) {
            /* binary: positive-class score against the threshold
             * (python/cuml/cuml/ensemble/randomforestclassifier.py:298,337) */
            best = ((REAL)s[0] > (REAL)threshold) ? 1 : 0;
          } else {
            /* first maximum wins: cpp/src/randomforest/randomforest.cuh:443-450 */
            for (int c = 1; c < k; ++c)
              if ((REAL)s[c] > (REAL)s[best]) best = c;
          }
          ((int32_t*)out)[r] = best;
        }
      }
    }
    free(acc);
  }
  free(divisor);
  free(packed);
  return failed ? -5 : 0;
}
