/* C interface of the compiler core: build computation graphs, (de)serialise them in the v1 JSON format and
 * run the strategy search, through opaque handles.  Counterpart of the reference's C headers
 * (lib/pcg/ffi/include/flexflow/pcg.h, lib/compiler/ffi/include/flexflow/compiler.h,
 * lib/ffi/include/flexflow/flexflow.h), whose implementation files are one-line stubs; this one is complete.
 *
 * The symbols live in the same shared object as the Python module (_ffcore*.so): load it with dlopen / ctypes.
 * Every function that can fail returns 0 on success and non-zero on failure; ffc_last_error() then describes
 * the failure (thread-local).  Strings returned by the library are released with ffc_string_free.  */
#ifndef FFC_FFI_H
#define FFC_FFI_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct ffc_builder ffc_builder_t;
typedef struct ffc_graph ffc_graph_t;
typedef struct {
  int node;
  int slot; /* value of the Slot enumeration; ffc_slot_name / ffc_slot_from_name convert */
} ffc_value_t;

const char *ffc_last_error(void);
void ffc_string_free(char *s);
const char *ffc_slot_name(int slot);
int ffc_slot_from_name(const char *name);

/* ---- computation graph builder */
ffc_builder_t *ffc_builder_create(void);
void ffc_builder_destroy(ffc_builder_t *b);
int ffc_builder_create_input(ffc_builder_t *b, const int64_t *dims, int ndims, const char *dtype, const char *name, ffc_value_t *out);
int ffc_builder_create_weight(ffc_builder_t *b, const int64_t *dims, int ndims, const char *dtype, const char *initializer_json,
                              const char *name, ffc_value_t *out);
/* Generic layer: op_type is the operator's name ("LINEAR", "EW_ADD", ...), attrs_json its attribute object,
 * inputs/input_slots the operands by slot name.  Missing weight operands are created with default initializers. */
int ffc_builder_add_layer(ffc_builder_t *b, const char *op_type, const char *attrs_json, const ffc_value_t *inputs,
                          const char *const *input_slots, int num_inputs, const char *name, ffc_value_t *outputs, int max_outputs,
                          int *num_outputs);
/* Convenience wrappers of the most common layers (activation: NULL or "RELU", "GELU", "SIGMOID", "TANH") */
int ffc_builder_dense(ffc_builder_t *b, ffc_value_t x, int64_t out_channels, const char *activation, int use_bias, const char *name,
                      ffc_value_t *out);
int ffc_builder_conv2d(ffc_builder_t *b, ffc_value_t x, int64_t out_channels, int kernel_h, int kernel_w, int stride_h, int stride_w,
                       int padding_h, int padding_w, const char *activation, int groups, int use_bias, const char *name, ffc_value_t *out);
int ffc_builder_unary(ffc_builder_t *b, const char *op, ffc_value_t x, int has_scalar, double scalar, const char *name, ffc_value_t *out);
int ffc_builder_binary(ffc_builder_t *b, const char *op, ffc_value_t x, ffc_value_t y, const char *name, ffc_value_t *out);
int ffc_builder_softmax(ffc_builder_t *b, ffc_value_t x, int dim, const char *name, ffc_value_t *out);
int ffc_builder_value_shape(const ffc_builder_t *b, ffc_value_t v, int64_t *dims, int max_dims, int *ndims);
const char *ffc_builder_value_dtype(const ffc_builder_t *b, ffc_value_t v);
/* One function per layer of the builder (the reference's flexflow_model_add_* family, lib/ffi/include/flexflow/ffi.h).
 * Optional strings may be NULL; initializers are the defaults of the layer. */
int ffc_builder_pool2d(ffc_builder_t *b, ffc_value_t x, int kernel_h, int kernel_w, int stride_h, int stride_w, int padding_h, int padding_w,
                       const char *pool_type, const char *activation, const char *name, ffc_value_t *out);
int ffc_builder_batch_norm(ffc_builder_t *b, ffc_value_t x, int affine, const char *activation, double eps, double momentum, const char *name,
                           ffc_value_t *out);
int ffc_builder_layer_norm(ffc_builder_t *b, ffc_value_t x, const int *axes, int num_axes, int affine, double eps, const char *name,
                           ffc_value_t *out);
int ffc_builder_embedding(ffc_builder_t *b, ffc_value_t ids, int64_t num_entries, int64_t out_dim, const char *aggr, const char *dtype,
                          const char *name, ffc_value_t *out);
int ffc_builder_multihead_attention(ffc_builder_t *b, ffc_value_t q, ffc_value_t k, ffc_value_t v, int64_t embed_dim, int64_t num_heads,
                                    int64_t kdim, int64_t vdim, double dropout, int bias, int add_bias_kv, int add_zero_attn, const char *name,
                                    ffc_value_t *out);
int ffc_builder_batch_matmul(ffc_builder_t *b, ffc_value_t a, ffc_value_t bb, const char *name, ffc_value_t *out);
int ffc_builder_dropout(ffc_builder_t *b, ffc_value_t x, double rate, uint64_t seed, const char *name, ffc_value_t *out);
int ffc_builder_cast(ffc_builder_t *b, ffc_value_t x, const char *dtype, const char *name, ffc_value_t *out);
int ffc_builder_concat(ffc_builder_t *b, const ffc_value_t *xs, int num, int axis, const char *name, ffc_value_t *out);
int ffc_builder_split(ffc_builder_t *b, ffc_value_t x, const int64_t *sizes, int num, int axis, const char *name, ffc_value_t *outs);
int ffc_builder_flat(ffc_builder_t *b, ffc_value_t x, const char *name, ffc_value_t *out);
int ffc_builder_transpose(ffc_builder_t *b, ffc_value_t x, const int *perm, int num, const char *name, ffc_value_t *out);
int ffc_builder_reshape(ffc_builder_t *b, ffc_value_t x, const int64_t *dims, int num, const char *name, ffc_value_t *out);
int ffc_builder_reverse(ffc_builder_t *b, ffc_value_t x, int axis, const char *name, ffc_value_t *out);
int ffc_builder_gather(ffc_builder_t *b, ffc_value_t x, ffc_value_t index, int dim, const char *name, ffc_value_t *out);
int ffc_builder_top_k(ffc_builder_t *b, ffc_value_t x, int k, int sorted, const char *name, ffc_value_t *values, ffc_value_t *indices);
/* op: "REDUCE_SUM" or "REDUCE_MEAN" (also MAX / MIN / PROD) */
int ffc_builder_reduce(ffc_builder_t *b, const char *op, ffc_value_t x, const int *axes, int num_axes, int keepdims, const char *name,
                       ffc_value_t *out);
int ffc_builder_broadcast(ffc_builder_t *b, ffc_value_t x, const int64_t *target, int num, const char *name, ffc_value_t *out);
/* Parallel builder: the four parallel operators are available and implicit weights get their Repartition / Replicate chains. */
ffc_builder_t *ffc_builder_create_parallel(void);
int ffc_builder_parallel_partition(ffc_builder_t *b, ffc_value_t x, int dim, int degree, const char *name, ffc_value_t *out);
int ffc_builder_parallel_combine(ffc_builder_t *b, ffc_value_t x, int dim, int degree, const char *name, ffc_value_t *out);
int ffc_builder_parallel_replicate(ffc_builder_t *b, ffc_value_t x, int degree, const char *name, ffc_value_t *out);
int ffc_builder_parallel_reduce(ffc_builder_t *b, ffc_value_t x, int degree, const char *name, ffc_value_t *out);
/* Parallel shape of a value: per-dim degrees, sum degree and discard-copy degree (degrees has room for max_dims entries). */
int ffc_builder_value_degrees(const ffc_builder_t *b, ffc_value_t v, int *degrees, int max_dims, int *ndims, int *sum_degree, int *copy_degree);

/* A copy of the graph built so far */
ffc_graph_t *ffc_builder_graph(const ffc_builder_t *b);

/* ---- graphs */
ffc_graph_t *ffc_model_build(const char *model_name, const char *config_json);
ffc_graph_t *ffc_graph_from_json(const char *v1_json);
char *ffc_graph_to_json(const ffc_graph_t *g, int parallel, int indent);
char *ffc_graph_to_dot(const ffc_graph_t *g);
int ffc_graph_num_nodes(const ffc_graph_t *g);
/* The same serialisation to and from a file (parallel != 0 writes the parallel / mapped variant). */
int ffc_graph_save_file(const ffc_graph_t *g, const char *path, int parallel, int indent);
ffc_graph_t *ffc_graph_load_file(const char *path);
/* Node ids in topological order (ids has room for max_ids entries; *num is the node count either way). */
int ffc_graph_node_ids(const ffc_graph_t *g, int *ids, int max_ids, int *num);
/* Operator type name ("LINEAR", ...), layer name and attribute object of a node; malloc'd strings. */
char *ffc_graph_node_op_type(const ffc_graph_t *g, int node);
char *ffc_graph_node_name(const ffc_graph_t *g, int node);
char *ffc_graph_node_attrs_json(const ffc_graph_t *g, int node);
/* Machine view of a node of a mapped graph as JSON ({"start": {"node_idx", "device_idx"}, "dimensions": [...]}); NULL with an
 * error when the node has none. */
char *ffc_graph_node_view_json(const ffc_graph_t *g, int node);
/* Shape, data type name and gradient flag of a node's output value. */
int ffc_graph_value_shape(const ffc_graph_t *g, ffc_value_t v, int64_t *dims, int max_dims, int *ndims);
const char *ffc_graph_value_dtype(const ffc_graph_t *g, ffc_value_t v);
int ffc_graph_value_create_grad(const ffc_graph_t *g, ffc_value_t v, int *create_grad);
/* Bytes of one element of a data type given by name; -1 with an error for an unknown name. */
int ffc_datatype_size(const char *dtype);
/* Estimated step time (ms) of a parallel computation graph on num_nodes x gpus_per_node devices under the analytic cost
 * model, with the machine mapping the dynamic program finds. */
int ffc_graph_estimate(const ffc_graph_t *pcg, int num_nodes, int gpus_per_node, double *runtime_ms);
/* Series-parallel decomposition of the graph's operators as JSON (malloc'd; NULL with an error when there is none). */
char *ffc_graph_sp_decomposition(const ffc_graph_t *g);

void ffc_graph_destroy(ffc_graph_t *g);

/* ---- strategy search.  algorithm: "unity", "mcmc" or "data_parallel".  On success *out is the mapped parallel
 * computation graph (owned by the caller) and *runtime_ms its estimated step time. */
int ffc_graph_optimize(const ffc_graph_t *cg, int num_nodes, int gpus_per_node, const char *algorithm, int budget, double alpha,
                       unsigned seed, ffc_graph_t **out, double *runtime_ms);

#ifdef __cplusplus
}
#endif
#endif
