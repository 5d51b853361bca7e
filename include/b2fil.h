/*
 * b2fil.h - C ABI of the B200 forest-inference library (libb2fil.so).
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns 0 on success or a
 * negative B2FIL_ERR_* code, never throws and never aborts.  The text of the last error of the
 * calling thread is read with b2fil_last_error(), the same convention the Treelite C API uses
 * (reference: python/cuml/cuml/internals/treelite.pxd:7-12, treelite.pyx:5-12).
 *
 * The functions replace what cuML binds from the un-vendored nvForest library for batched
 * tree-ensemble prediction.  Reference call sites (paths inside NVIDIA/cuml 26.10):
 *   - import:   nvforest.load_from_treelite_model(tl_model, device, layout, default_chunk_size,
 *               align_bytes, handle)          python/cuml/cuml/ensemble/randomforest_common.pyx:402-409
 *               nvforest::import_from_treelite_handle(model, tree_layout, align_bytes, use_double,
 *               device_type, device_id, stream)                     cpp/tests/sg/rf_test.cu:257-263
 *   - predict:  forest_model.predict(handle, out, in, n_rows, out_mem, in_mem, infer_kind,
 *               chunk_size)                                         cpp/tests/sg/rf_test.cu:268-275
 *               .predict / .predict_proba / .predict_per_tree
 *               python/cuml/cuml/ensemble/randomforestclassifier.py:337,388
 *               python/cuml/cuml/ensemble/randomforest_common.pyx:652
 *
 * Device work is stream ordered: calls that take a `cuda_stream` enqueue on it and return without
 * synchronising; the caller owns input and output buffers and synchronises the stream.  A forest
 * is immutable after creation, so several host threads may predict with it on different streams.
 */
#ifndef B2FIL_H_
#define B2FIL_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- error codes ------------------------------------------------------------------------- */
#define B2FIL_OK 0
#define B2FIL_ERR_INVALID_ARG (-1)   /* NULL pointer, negative size, unknown enum value          */
#define B2FIL_ERR_BAD_FOREST (-2)    /* malformed tree: child out of range, cycle, bad feature   */
#define B2FIL_ERR_UNSUPPORTED (-3)   /* legal model that this build cannot represent             */
#define B2FIL_ERR_CUDA (-4)          /* a CUDA runtime call failed; message holds its text       */
#define B2FIL_ERR_NO_MEMORY (-5)     /* host or device allocation failed                         */
#define B2FIL_ERR_TOO_LARGE (-6)     /* size beyond a documented fixed limit                     */
#define B2FIL_ERR_TIMEOUT (-7)       /* a bounded host wait ran out                              */

/* ---- enums --------------------------------------------------------------------------------- */
/* precision of thresholds, leaves, inputs and outputs on the device (nvForest: use_double) */
#define B2FIL_F32 0
#define B2FIL_F64 1

/* node kinds in a forest description */
#define B2FIL_NODE_LEAF 0
#define B2FIL_NODE_NUMERICAL 1
#define B2FIL_NODE_CATEGORICAL 2

/* comparison operator of a numerical test; the test being TRUE sends the row to the LEFT child
 * (reference: cpp/src/decisiontree/decisiontree.cuh:204-205,379-383 uses <=;
 *  cpp/src/isolation_forest/isolation_forest.cu:75-79 uses <) */
#define B2FIL_OP_LT 0
#define B2FIL_OP_LE 1
#define B2FIL_OP_GT 2
#define B2FIL_OP_GE 3

/* node order on the device (nvforest::tree_layout; randomforest_common.pyx:381-383) */
#define B2FIL_LAYOUT_DEPTH_FIRST 0
#define B2FIL_LAYOUT_BREADTH_FIRST 1
#define B2FIL_LAYOUT_LAYERED 2

/* storage of the packed forest: SPARSE keeps child offsets in every node and honours `layout`;
 * DENSE pads every tree to a complete binary tree of the forest's maximum depth and indexes
 * children implicitly (heap order), which removes the offset arithmetic from the hot loop and
 * lets whole trees be staged in shared memory.  AUTO picks DENSE when the padded forest is small
 * enough and a row tile fits shared memory next to it.  Forests with so many features (from
 * about 800 on) that only a tile of 16-bit ranks fits are dense only together with
 * row_quantization = 0: AUTO then weighs the cost of ranking a row against the nodes it visits,
 * and DENSE is refused with B2FIL_ERR_UNSUPPORTED when the forest cannot be rank-quantised. */
#define B2FIL_STORAGE_AUTO 0
#define B2FIL_STORAGE_DENSE 1
#define B2FIL_STORAGE_SPARSE 2

/* what predict writes (nvforest::infer_kind) */
#define B2FIL_INFER_DEFAULT 0   /* (n_rows, n_outputs) scores after averaging/base/postprocess  */
#define B2FIL_INFER_PER_TREE 1  /* (n_rows, n_trees[, n_classes]) raw per-tree outputs          */
#define B2FIL_INFER_LEAF_ID 2   /* (n_rows, n_trees) uint32 id of the leaf reached              */
#define B2FIL_INFER_CLASS 3     /* (n_rows,) int32 class index (argmax or threshold)            */
#define B2FIL_INFER_PROBA2 4    /* (n_rows, 2): [1-p, p] for one-output binary classifiers      */

/* postprocessing applied to the summed tree outputs (Treelite postprocessor names) */
#define B2FIL_POST_IDENTITY 0
#define B2FIL_POST_SIGMOID 1
#define B2FIL_POST_EXPONENTIAL 2
#define B2FIL_POST_LOG1PEXP 3
#define B2FIL_POST_SIGNED_SQUARE 4
#define B2FIL_POST_HINGE 5
#define B2FIL_POST_SOFTMAX 6
#define B2FIL_POST_MULTICLASS_OVA 7
#define B2FIL_POST_EXP_STD_RATIO 8

/* ---- forest description (host, structure of arrays) ----------------------------------------- */
/*
 * Mirrors the Treelite fields cuML reads and writes (cpp/src/decisiontree/decisiontree.cuh:165-221,
 * cpp/src/randomforest/randomforest.cu:262-279,308-333, cpp/src/explainer/tree_shap.cu:268-300).
 * Nodes of tree t occupy [tree_offsets[t], tree_offsets[t+1]) of every per-node array; node 0 of
 * that range is the root; `left` / `right` are indices relative to the tree's first node; the
 * relative index of a node is also the id that B2FIL_INFER_LEAF_ID reports for it.
 */
typedef struct b2fil_forest_desc {
  int32_t n_trees;
  int32_t n_features;
  int32_t n_outputs;       /* classes for classifiers, 1 for regression and one-score binary     */
  int32_t leaf_vector_len; /* 1: scalar leaves; n_outputs: every leaf holds a vector             */
  const int64_t* tree_offsets; /* [n_trees + 1]                                                  */
  const uint8_t* node_kind;    /* [n_nodes] B2FIL_NODE_*                                         */
  const int32_t* feature;      /* [n_nodes] split feature (ignored for leaves)                   */
  const double* threshold;     /* [n_nodes] numerical threshold (ignored otherwise)              */
  const int32_t* left;         /* [n_nodes] relative index of the left child                     */
  const int32_t* right;        /* [n_nodes] relative index of the right child                    */
  const uint8_t* default_left; /* [n_nodes] 1: a missing (NaN) value goes left                   */
  const uint8_t* op;           /* [n_nodes] B2FIL_OP_* or NULL = every numerical test uses op_all */
  int32_t op_all;
  const int64_t* cat_ptr;      /* [n_nodes + 1] CSR into cat_values, or NULL: no categorical node */
  const uint32_t* cat_values;  /* categories listed by the node                                  */
  const uint8_t* cat_right;    /* [n_nodes] 1: a listed category goes right, 0: goes left; NULL=1 */
  const double* leaf_value;    /* [n_nodes * leaf_vector_len]                                    */
  const int32_t* class_id;     /* [n_trees] output a scalar leaf adds to; NULL = t % n_outputs   */
  int32_t average_tree_output; /* divide sums by the number of trees feeding each output         */
  const double* base_scores;   /* [n_outputs] or NULL = zeros                                    */
  int32_t postproc;            /* B2FIL_POST_*                                                   */
  double sigmoid_alpha;        /* sigmoid(x) = 1 / (1 + exp(-alpha x))                           */
  double ratio_c;              /* exp_std_ratio(x) = exp2(-x / c)                                */
} b2fil_forest_desc;

typedef struct b2fil_create_opts {
  int32_t precision;   /* B2FIL_F32 / B2FIL_F64                                                  */
  int32_t layout;      /* B2FIL_LAYOUT_*                                                          */
  int32_t storage;     /* B2FIL_STORAGE_*                                                         */
  int32_t align_bytes; /* 0 or a power of two: pad every tree of a sparse forest to this size    */
  int32_t device_id;   /* CUDA device ordinal that will hold the forest                          */
  int32_t default_chunk_size; /* 0 = choose; else the value predict uses when given chunk_size 0 */
  int32_t row_quantization;   /* REQUEST: 0 = automatic (dense forests whose categorical tests, if
                                 any, only list categories below 32 predict on 16-bit per-feature
                                 ranks of the inputs, which is exact), 1 = never.  What the forest
                                 actually does is reported by b2fil_info.row_quantization, where
                                 1 means "on".                                                    */
  int32_t compact_image;      /* REQUEST, sparse storage: 0 = automatic (forests whose fields fit
                                 also get the compact image - 8-byte internal nodes, leaves apart,
                                 top levels of every tree as a heap for shared memory - that the
                                 fast sparse kernel reads), 1 = never, 100 + T = automatic with at
                                 most T heap levels (tuning aid).  b2fil_info.compact_image says
                                 whether it exists.                                               */
} b2fil_create_opts;

typedef struct b2fil_info {
  int32_t precision, layout, storage, device_id;
  int32_t n_trees, n_features, n_outputs, leaf_vector_len;
  int32_t max_depth;       /* edges on the longest root-to-leaf path                             */
  int32_t dense_depth;     /* depth every tree is padded to (dense storage), else -1             */
  int32_t node_bytes;      /* size of one packed node                                            */
  int32_t has_categorical;
  int64_t n_nodes_in;      /* nodes in the description                                           */
  int64_t n_nodes_packed;  /* nodes stored on the device (with padding)                          */
  int64_t device_bytes;    /* device memory held by the forest                                   */
  int32_t default_chunk_size;
  int32_t row_quantization; /* 1: predictions run on rank-quantised rows                        */
  int32_t peer_direct;      /* forests made by b2fil_forest_clone_to_device: 1 = the copy went
                               over a direct peer path (NVLink / PCIe peer-to-peer), 0 = staged
                               through host memory; -1 for forests made by b2fil_forest_create   */
  int32_t clone_src_device; /* device the forest was replicated from, or -1                     */
  int32_t compact_image;    /* 1: sparse forest with the compact image                          */
  int32_t top_levels;       /* levels of every tree kept as a heap for shared memory, else 0    */
  int64_t scratch_pool_bytes; /* device memory the forest's scratch pool holds right now (grows
                                 with the largest batch b2fil_predict has seen; never touched by
                                 b2fil_predict_fixed_scratch)                                    */
} b2fil_info;

typedef struct b2fil_forest b2fil_forest; /* opaque */

/* ---- entry points --------------------------------------------------------------------------- */

/* Text of the last error raised on the calling thread ("" if none).
 * Replaces TreeliteGetLastError (python/cuml/cuml/internals/treelite.pxd:12). */
const char* b2fil_last_error(void);

/* Library version as major*10000 + minor*100 + patch. */
int b2fil_version(void);

/* Validate a description, pack it (layout / storage / precision) and upload it to opts->device_id.
 * Synchronous.  Replaces nvforest.load_from_treelite_model / nvforest::import_from_treelite_handle
 * (randomforest_common.pyx:402-409, cpp/tests/sg/rf_test.cu:257-263). */
int b2fil_forest_create(const b2fil_forest_desc* desc, const b2fil_create_opts* opts,
                        b2fil_forest** out);

/* Copy a packed forest to another device of the same box (peer copy when the devices can reach
 * each other, else through the host).  Model replication of the row-sharded multi-GPU path
 * (python/cuml/cuml/dask/ensemble/base.py:153-175 broadcasts the model to every worker). */
int b2fil_forest_clone_to_device(const b2fil_forest* src, int device_id, b2fil_forest** out);

/* Release a forest and its device memory.
 * (cpp/tests/sg/rf_test.cu:266 deletes the model handle explicitly.) */
int b2fil_forest_free(b2fil_forest* f);

/* Describe a packed forest.  `forest.get_dtype()` of the reference
 * (python/cuml/cuml/ensemble/randomforestclassifier.py:333) is info->precision. */
int b2fil_forest_info(const b2fil_forest* f, b2fil_info* info);

/* Read the forest's device status word.  Prediction kernels bound every internal wait; when a
 * bound is hit they set the word, stop working and return (their outputs are then incomplete).
 * The call waits for ALL work on the forest's device (cudaDeviceSynchronize, so non-blocking
 * streams are covered too), reads the word, and returns B2FIL_ERR_TIMEOUT when it is set; the word
 * is cleared by the read, so one timeout is reported once.  b2fil_predict_host and
 * b2fil_predict_sharded check the word themselves before they return; callers of the
 * stream-ordered b2fil_predict / b2fil_predict_fixed_scratch should poll it after they have
 * synchronised (e.g. once per batch of requests).  No counterpart in the reference. */
int b2fil_forest_status(const b2fil_forest* f, int32_t* status);

/* Self test of the timeout reporting: enqueues, on cuda_stream of the forest's device, a one-CTA
 * kernel whose only work is a bounded wait that nothing ends (an mbarrier that never receives
 * its arrival).  After `tries` tries (1..4096; a try lasts at most a few microseconds) the kernel
 * sets the forest's status word exactly like a prediction kernel whose wait ran out, and returns;
 * nothing hangs and the context stays usable.  b2fil_forest_status must then report
 * B2FIL_ERR_TIMEOUT once.  No counterpart in the reference. */
int b2fil_forest_selftest_timeout(b2fil_forest* f, int tries, void* cuda_stream);

/* Describe the kernels the calling thread's most recent prediction call enqueued (kernel family,
 * template arguments, launch shape), e.g. "quantise_kernel<float> + dense_q_top_kernel<float,
 * scalar,NT=6,DEPTH=8> R=256 G=3 S=2 K=2".  Writes a NUL-terminated string of at most
 * buf_bytes - 1 characters and returns the full length.  No counterpart in the reference. */
int b2fil_last_variant(char* buf, size_t buf_bytes);

/* Tuning aid for experiments (defaults are the measured best; nothing needs it in normal use):
 * set a named integer knob for the whole process.  Knobs: "q_R", "q_G", "q_NT", "q_S", "q_K" force
 * the launch shape of the traversal over rank-quantised rows (rows per tile, tree groups, trees
 * in flight per warp, ring depth, sub-batches per stage; q_R = 0: automatic), "q_pair" = 1 / 0
 * forces / forbids its variant that fetches both children of a node ahead of the test (-1:
 * automatic), "q_leafg" = 1 / 0 forces / forbids its variant that keeps only the test nodes of
 * depth-9 and depth-10 trees in shared memory and fetches leaf payloads from global memory (-1:
 * automatic, taken when it puts a third more walks in flight); "compact_R", "compact_G",
 * "compact_S" force the launch shape of the kernel over the compact image of sparse forests (rows
 * per tile, tree groups, ring depth; 0 = automatic).  Unknown keys are stored and ignored.
 * No counterpart in the reference. */
int b2fil_set_tuning(const char* key, int value);

/* Switch peer access between two devices on, in both directions, if the hardware allows it (a
 * per-process setting; forest replication and the sharded gather do this themselves).  Returns 1
 * when copies between the two devices are direct, 0 when they are staged through host memory,
 * or a negative error code.  No counterpart in the reference. */
int b2fil_enable_peer_access(int device_a, int device_b);

/* Number of prediction kernels this process has launched through the library so far. */
int64_t b2fil_kernel_launches(void);

/* Number of elements predict writes per row for `infer_kind` (0 and an error for a bad kind). */
int64_t b2fil_output_elems_per_row(const b2fil_forest* f, int infer_kind);

/* Batched prediction, device buffers.  X_dev: row-major (n_rows, n_features) of the forest's
 * precision with `row_stride` elements between rows; out_dev: n_rows *
 * b2fil_output_elems_per_row() elements (precision type; uint32 for LEAF_ID, int32 for CLASS).
 * chunk_size 0 = the forest's default.  `threshold` is the binary decision threshold of
 * B2FIL_INFER_CLASS for one-output classifiers.  Enqueues on cuda_stream (NULL = default stream)
 * of the forest's device and does not synchronise.  Two cases take stream-ordered scratch from a
 * memory pool owned by the forest (cached between calls): forests whose b2fil_info reports
 * row_quantization = 1 keep the 16-bit rank image of the batch there, and small batches of dense forests (fewer 128-row
 * tiles than half the SMs) keep the partial sums of the CTAs that share the forest there.
 * Replaces forest_model.predict(...) (cpp/tests/sg/rf_test.cu:268-275). */
int b2fil_predict(const b2fil_forest* f, int infer_kind, const void* X_dev, int64_t n_rows,
                  int64_t row_stride, void* out_dev, int chunk_size, double threshold,
                  void* cuda_stream);

/* Size of the fixed scratch array used by b2fil_predict_fixed_scratch (32 MiB per GPU). */
#define B2FIL_FIXED_SCRATCH_BYTES 33554432

/* Batched prediction, device buffers, for callers that must not allocate device memory while
 * they predict.  It has no counterpart in the reference.
 *
 * b2fil_predict keeps the 16-bit rank image of the batch (forests whose b2fil_info reports
 * row_quantization = 1) in scratch that it takes from a CUDA memory pool.  A process whose GPU memory is handed out in
 * full to its own allocator at start-up, or a serving loop that cannot afford the lock and the
 * possible failure of an allocation in the middle of a request, cannot accept that.  For them this
 * call writes the rank image into a B2FIL_FIXED_SCRATCH_BYTES array that is part of the library
 * image on every GPU that loads the library; it calls no cudaMalloc / cudaFree and no allocating
 * library routine.
 *
 * Arguments, outputs and errors are those of b2fil_predict, with these differences:
 *  - the whole batch must fit the array: ceil(n_rows / T) * T * n_features * 2 bytes plus four
 *    bytes per tile of T rows (T <= 256) may not exceed B2FIL_FIXED_SCRATCH_BYTES, i.e. about
 *    B2FIL_FIXED_SCRATCH_BYTES / (2 * n_features) rows per call (about 65,000 rows of 256 features);
 *    larger batches return B2FIL_ERR_TOO_LARGE with the numbers in the message: split them;
 *  - all calls on one GPU share the array: two calls whose kernels can overlap on the GPU (two
 *    streams, two threads) race on it; issue them on one stream or serialise them yourself;
 *  - the first call on each device looks up the array's device address (with that device current)
 *    and caches it; make that first call before any stream capture is started;
 *  - "allocates nothing" holds from the second call on.  The first call on a device for a given
 *    forest shape and infer_kind makes the CUDA runtime load the kernels it needs (with lazy module
 *    loading that is when the driver reserves the array itself and the kernels' code) and raises
 *    their shared-memory limit.  A process that wants to hand ALL remaining GPU memory to its own
 *    allocator must make one warm-up call per device and per (forest shape, infer_kind) BEFORE it
 *    does so; after that warm-up a call changes neither the free device memory nor the forest's
 *    pool;
 *  - forests that predict without rank scratch (sparse storage, b2fil_info.row_quantization = 0) are
 *    forwarded to the ordinary kernels with the forest-splitting of small batches switched off,
 *    so nothing is allocated for them either. */
int b2fil_predict_fixed_scratch(const b2fil_forest* f, int infer_kind, const void* X_dev,
                                int64_t n_rows, int64_t row_stride, void* out_dev, int chunk_size,
                                double threshold, void* cuda_stream);

/* Batched prediction, host buffers: copies row blocks to the device, predicts and copies results
 * back, with copies and kernels overlapped on internal streams.  Pinned host memory gives
 * full copy bandwidth.  Ordinary (pageable) arrays of 8 MiB or more are staged by the library
 * itself: a few host threads gather 64 MiB row blocks into three pinned buffers while earlier
 * blocks are copied and predicted, which is about three times faster than handing pageable
 * memory to cudaMemcpyAsync.  Synchronous: returns when out_host is complete -
 * also when it returns an error, every copy that was already enqueued has finished, so the
 * caller may free its buffers.  This is the call a host-array user of `.predict_proba(X)` reaches. */
int b2fil_predict_host(b2fil_forest* f, int infer_kind, const void* X_host, int64_t n_rows,
                       int64_t row_stride, void* out_host, int chunk_size, double threshold);

/* Row-sharded prediction over several devices of one box from a single process: forests[i] lives
 * on device i of the set, rows are split into contiguous shards, shard i is predicted on its
 * device, and results are gathered into out (a device buffer on forests[0]'s device, by peer
 * copies; no collective library).  X_shards[i] is the device pointer of shard i's first row on
 * device i; shard_rows[i] its row count.  Synchronous: on return, with or without an error,
 * nothing the call enqueued is still running.  Peer access between every device and forests[0]'s
 * device is switched on at the first use, so that the gather crosses NVLink instead of host
 * memory where the hardware allows it.  Callers may pass the same forests in any order from
 * several threads (their locks are taken in a fixed order).
 * (python/cuml/cuml/dask/ensemble/base.py:210-218, dask/common/base.py:276-316: model replicated,
 *  row partitions predicted where they live, results concatenated by rows.) */
int b2fil_predict_sharded(b2fil_forest* const* forests, int n_devices, int infer_kind,
                          const void* const* X_shards, const int64_t* shard_rows,
                          int64_t row_stride, void* out_dev0, int chunk_size, double threshold);

/* Device-side times of the calling thread's last b2fil_predict_sharded call, from CUDA events on
 * each device's stream: compute_ms = the slowest device's prediction kernels, gather_ms = the
 * slowest peer copy into forests[0]'s device, wall_ms = host clock from the first launch to the
 * last device done, gather_direct = 1 when every gather copy used a direct peer path.  Any
 * pointer may be NULL.  No counterpart in the reference. */
int b2fil_last_sharded_timing(double* compute_ms, double* gather_ms, double* wall_ms,
                              int* gather_direct);

#ifdef __cplusplus
}
#endif
#endif /* B2FIL_H_ */
