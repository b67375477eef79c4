// builder.h -- graph builders.
//
// GraphBuilder is the PyTorch-style layer API of the reference's
// ComputationGraphBuilder (lib/pcg/include/pcg/computation_graph_builder.h:16-294):
// weights are implicit, shapes are inferred, default initializers are attached.
// Constructed with parallel = true it is the ParallelComputationGraphBuilder
// (lib/pcg/include/pcg/parallel_computation_graph/parallel_computation_graph_builder.h:10-159):
// the four parallel operators become available and every implicit weight is
// followed by the Repartition / Replicate chain that brings it to the parallel
// shape its consumer expects (generate_weight_transform.cc:9-31).
// Methods the reference declares but never defines (batch_matmul, mean, split,
// transpose, reduce_sum, reshape, reverse, top_k, cache) are implemented here.
#pragma once
#include <optional>
#include <string>
#include <vector>

#include "ir.h"

namespace ff {

using V = ValueRef;
using OptInit = std::optional<Json>;

class GraphBuilder {
public:
  explicit GraphBuilder(bool parallel = false) : parallel_(parallel) {}
  Graph graph;
  bool parallel() const { return parallel_; }

  V create_input(const std::vector<int64_t> &dims, DataType dt, bool create_grad = false, const std::string &name = "");
  V create_weight(const std::vector<int64_t> &dims, DataType dt, const OptInit &init = std::nullopt,
                  bool create_grad = true, const std::string &name = "");
  // Generic entry: infers shapes, materialises implicit weights, adds the node.
  std::vector<V> add_layer(OpType type, Json attrs, std::vector<std::pair<Slot, V>> inputs, const std::string &name = "",
                           const std::map<Slot, Json> &initializers = {});
  const PShape &shape(V v) const { return graph.shape(v); }

  // elementwise
  V unary(OpType t, V x, std::optional<double> scalar = std::nullopt, const std::string &name = "");
  V binary(OpType t, V a, V b, const std::string &name = "");
  V exp(V x, const std::string &n = "") { return unary(OpType::EXP, x, {}, n); }
  V relu(V x, const std::string &n = "") { return unary(OpType::RELU, x, {}, n); }
  V gelu(V x, const std::string &n = "") { return unary(OpType::GELU, x, {}, n); }
  V sigmoid(V x, const std::string &n = "") { return unary(OpType::SIGMOID, x, {}, n); }
  V tanh(V x, const std::string &n = "") { return unary(OpType::TANH, x, {}, n); }
  V elu(V x, const std::string &n = "") { return unary(OpType::ELU, x, {}, n); }
  V identity(V x, const std::string &n = "") { return unary(OpType::IDENTITY, x, {}, n); }
  V rsqrt(V x, const std::string &n = "") { return unary(OpType::RSQRT, x, {}, n); }
  V sin(V x, const std::string &n = "") { return unary(OpType::SIN, x, {}, n); }
  V cos(V x, const std::string &n = "") { return unary(OpType::COS, x, {}, n); }
  V pow(V x, double e, const std::string &n = "") { return unary(OpType::POW, x, e, n); }
  V scalar_multiply(V x, double s, const std::string &n = "") { return unary(OpType::SCALAR_MULTIPLY, x, s, n); }
  V scalar_add(V x, double s, const std::string &n = "") { return unary(OpType::SCALAR_ADD, x, s, n); }
  V scalar_sub(V x, double s, const std::string &n = "") { return unary(OpType::SCALAR_SUB, x, s, n); }
  V scalar_truediv(V x, double s, const std::string &n = "") { return unary(OpType::SCALAR_TRUE_DIV, x, s, n); }
  V add(V a, V b, const std::string &n = "") { return binary(OpType::EW_ADD, a, b, n); }
  V subtract(V a, V b, const std::string &n = "") { return binary(OpType::EW_SUB, a, b, n); }
  V multiply(V a, V b, const std::string &n = "") { return binary(OpType::EW_MUL, a, b, n); }
  V divide(V a, V b, const std::string &n = "") { return binary(OpType::EW_DIV, a, b, n); }
  V max(V a, V b, const std::string &n = "") { return binary(OpType::EW_MAX, a, b, n); }
  V min(V a, V b, const std::string &n = "") { return binary(OpType::EW_MIN, a, b, n); }

  // layers
  V dense(V x, int64_t out_channels, const std::optional<std::string> &activation = std::nullopt, bool use_bias = true,
          const OptInit &proj_init = std::nullopt, const OptInit &bias_init = std::nullopt, const std::string &name = "");
  V conv2d(V x, int64_t out_channels, int kh, int kw, int sh, int sw, int ph, int pw,
           const std::optional<std::string> &activation = std::nullopt, int groups = 1, bool use_bias = true,
           const OptInit &kernel_init = std::nullopt, const OptInit &bias_init = std::nullopt, const std::string &name = "");
  V pool2d(V x, int kh, int kw, int sh, int sw, int ph, int pw, const std::string &pool_type = "MAX",
           const std::optional<std::string> &activation = std::nullopt, const std::string &name = "");
  V adaptive_pool2d(V x, int out_h, int out_w, const std::string &pool_type = "AVG", const std::string &name = "");
  V batch_norm(V x, bool affine = true, const std::optional<std::string> &activation = std::nullopt, double eps = 1e-5,
               std::optional<double> momentum = 0.1, const std::string &name = "");
  V layer_norm(V x, const std::vector<int> &axes, bool affine = true, double eps = 1e-5, const std::string &name = "");
  V embedding(V x, int64_t num_entries, int64_t out_dim, const std::string &aggr = "SUM", DataType dt = DataType::FLOAT,
              const OptInit &init = std::nullopt, const std::string &name = "");
  V multihead_attention(V q, V k, V v, int64_t embed_dim, int64_t num_heads, std::optional<int64_t> kdim = std::nullopt,
                        std::optional<int64_t> vdim = std::nullopt, double dropout = 0.0, bool bias = false,
                        bool add_bias_kv = false, bool add_zero_attn = false, const OptInit &init = std::nullopt,
                        const std::string &name = "");
  V batch_matmul(V a, V b, const std::string &name = "");
  V dropout(V x, double rate, uint64_t seed = 0, const std::string &name = "");
  V softmax(V x, int dim = -1, const std::string &name = "");
  V cast(V x, DataType dt, const std::string &name = "");
  V concat(const std::vector<V> &xs, int axis, const std::string &name = "");
  std::vector<V> split(V x, const std::vector<int64_t> &sizes, int axis, const std::string &name = "");
  V flat(V x, int start_dim = 1, int end_dim = -1, const std::string &name = "");
  V transpose(V x, const std::vector<int> &perm, const std::string &name = "");
  V reshape(V x, const std::vector<int64_t> &dims, const std::string &name = "");
  V reverse(V x, int axis, const std::string &name = "");
  V gather(V x, V index, int dim, const std::string &name = "");
  std::vector<V> top_k(V x, int k, bool sorted = true, const std::string &name = "");
  V reduce(OpType t, V x, const std::vector<int> &axes, bool keepdims = false, const std::string &name = "");
  V reduce_sum(V x, const std::vector<int> &axes, bool keepdims = false, const std::string &n = "") { return reduce(OpType::REDUCE_SUM, x, axes, keepdims, n); }
  V mean(V x, const std::vector<int> &axes, bool keepdims = false, const std::string &n = "") { return reduce(OpType::REDUCE_MEAN, x, axes, keepdims, n); }
  V broadcast(V x, const std::vector<int64_t> &target, const std::string &name = "");
  V noop(V x, const std::string &name = "");

  // parallel operators (parallel builder only)
  V parallel_partition(V x, int dim, int degree, const std::string &name = "");
  V parallel_combine(V x, int dim, int degree, const std::string &name = "");
  V parallel_replicate(V x, int degree, const std::string &name = "");
  V parallel_reduce(V x, int degree, const std::string &name = "");

private:
  bool parallel_;
  V weight_for(const PShape &goal, const Json &init, const std::string &name);
};

// pcg_from_computation_graph (lib/pcg/src/pcg/pcg_from_computation_graph.cc:18): relabel 1:1.
Graph pcg_from_computation_graph(const Graph &cg);

}  // namespace ff
