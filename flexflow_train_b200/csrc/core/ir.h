// ir.h -- operator / tensor / graph data model of the compiler core.
//
// One graph type serves the three program representations of the reference:
//   ComputationGraph          (lib/pcg/include/pcg/computation_graph.h:15-81)
//   ParallelComputationGraph  (lib/pcg/include/pcg/parallel_computation_graph/parallel_computation_graph.h)
//   MappedParallelComputationGraph (lib/pcg/include/pcg/mapped_parallel_computation_graph/*.h)
// A computation graph is a parallel computation graph in which every degree is 1
// and no node carries a machine view; a mapped graph is one in which every
// operator node does.  Nodes are labelled with (operator type, attribute object,
// optional name); values are labelled with a parallel tensor shape and a
// create-gradient flag; edges connect named output slots to named input slots
// ("kwarg dataflow graph", lib/utils/include/utils/graph/index.dox).
#pragma once
#include <cstdint>
#include <functional>
#include <map>
#include <optional>
#include <set>
#include <stdexcept>
#include <string>
#include <vector>

#include "json.h"

namespace ff {

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// ---------------------------------------------------------------- enums
#define FF_DATATYPES(X) X(BOOL) X(INT32) X(INT64) X(HALF) X(FLOAT) X(DOUBLE) X(BFLOAT16)
enum class DataType {
#define X(n) n,
  FF_DATATYPES(X)
#undef X
};
std::string to_string(DataType);
DataType datatype_from_string(const std::string &);
int dtype_bytes(DataType);

// Plain tensor dims (lib/op-attrs/include/op-attrs/tensor_dims.h): broadcasting follows numpy -- a tensor reaches a goal of at
// least its rank when, aligned at the trailing dim, each of its dims equals the goal's or is 1.
bool tensor_dims_has_dim(const std::vector<int64_t> &dims, int idx);
bool tensor_dims_is_broadcastable_to(const std::vector<int64_t> &curr, const std::vector<int64_t> &goal);
// the one of `inputs` that all of them broadcast to, if there is one (a target that is not among the inputs does not count)
std::optional<std::vector<int64_t>> get_broadcast_target_dims(const std::vector<std::vector<int64_t>> &inputs);
// every coordinate of a tensor of these dims, last dim fastest (one empty coordinate for a zero-dimensional tensor)
std::vector<std::vector<int64_t>> get_tensor_dims_coord_set(const std::vector<int64_t> &dims);
std::vector<int64_t> tensor_dims_drop_dims(const std::vector<int64_t> &dims, const std::function<bool(int)> &should_drop);

// Operator types, same set and order as lib/op-attrs/include/op-attrs/operator_type.dtg.toml
#define FF_OPTYPES(X)                                                                                               \
  X(NOOP) X(INPUT) X(WEIGHT) X(CONV2D) X(DROPOUT) X(LINEAR) X(BATCHMATMUL) X(POOL2D) X(SCALAR_MULTIPLY)            \
  X(SCALAR_ADD) X(SCALAR_FLOOR_DIV) X(SCALAR_TRUE_DIV) X(SCALAR_SUB) X(RELU) X(IDENTITY) X(SIGMOID) X(TANH)       \
  X(ELU) X(FLAT) X(SOFTMAX) X(BATCHNORM) X(CONCAT) X(SPLIT) X(EMBEDDING) X(CACHE) X(RESHAPE) X(REVERSE)           \
  X(TRANSPOSE) X(EW_ADD) X(EW_MUL) X(MATMUL) X(MUL) X(ENLARGE) X(SQUEEZE) X(UNSQUEEZE) X(EW_SUB) X(EW_DIV)        \
  X(EW_EQUAL) X(EW_GREATER) X(EW_LESS) X(EW_MAX) X(EW_MIN) X(REDUCE_ARGMAX) X(REDUCE_ARGMIN) X(REDUCE_MAX)        \
  X(REDUCE_MEAN) X(REDUCE_MIN) X(REDUCE_PROD) X(REDUCE_SUM) X(PAD) X(SHAPE) X(SIZE) X(TOPK) X(WHERE) X(CEIL)      \
  X(CAST) X(EXP) X(ROUND) X(LOG) X(LOGICAL_NOT) X(SQRT) X(SIN) X(COS) X(LEAKYRELU) X(SLICE) X(RESIZE) X(PRELU)    \
  X(GELU) X(MULTIHEAD_ATTENTION) X(FUSED) X(RSQRT) X(POW) X(MEAN) X(LAYERNORM) X(GATHER) X(BROADCAST)             \
  X(REPARTITION) X(COMBINE) X(REPLICATE) X(REDUCTION) X(BATCH) X(PIPELINE) X(FUSED_PARALLEL)
enum class OpType {
#define X(n) n,
  FF_OPTYPES(X)
#undef X
};
std::string to_string(OpType);
OpType optype_from_string(const std::string &);
bool is_parallel_op(OpType);
bool is_element_unary(OpType);   // RELU ... POW family carried by ElementUnaryAttrs
bool is_element_binary(OpType);  // EW_ADD ... EW_MIN
// key of the attrs variant in the v1 file format ("linear", "element_unary", ...)
std::string attrs_variant_key(OpType);

// Tensor slot names, lib/op-attrs/include/op-attrs/tensor_slot_name.dtg.toml
#define FF_SLOTS(X)                                                                                            \
  X(INPUT) X(OUTPUT) X(FILTER) X(BIAS) X(INPUT_BIAS) X(OUTPUT_BIAS) X(LHS_INPUT) X(RHS_INPUT) X(INDEX)        \
  X(GAMMA) X(BETA) X(WEIGHT) X(QUERY) X(KEY) X(VALUE) X(LOGIT) X(INPUT_0) X(INPUT_1) X(INPUT_2) X(INPUT_3)    \
  X(INPUT_4) X(INPUT_5) X(INPUT_6) X(INPUT_7) X(OUTPUT_0) X(OUTPUT_1) X(OUTPUT_2) X(OUTPUT_3) X(OUTPUT_4)     \
  X(OUTPUT_5) X(SCALE)
enum class Slot {
#define X(n) n,
  FF_SLOTS(X)
#undef X
};
std::string to_string(Slot);
Slot slot_from_string(const std::string &);
Slot input_slot_n(int i);   // INPUT_0 + i
Slot output_slot_n(int i);  // OUTPUT_0 + i

// ---------------------------------------------------------------- tensors
struct ShardDim {
  int64_t size;
  int degree;
  bool operator==(const ShardDim &o) const { return size == o.size && degree == o.degree; }
};

// lib/op-attrs/include/op-attrs/parallel_tensor_shape.h:16-64
struct PShape {
  std::vector<ShardDim> dims;
  int sum_degree = 1;
  int discard_copy_degree = 1;
  DataType dtype = DataType::FLOAT;

  static PShape make(const std::vector<int64_t> &sizes, DataType dt);
  int ndim() const { return (int)dims.size(); }
  int norm_dim(int d) const;  // python-style negative index
  std::vector<int64_t> sizes() const;
  std::vector<int> degrees() const;
  std::vector<int64_t> piece_sizes() const;
  int64_t num_elements() const;
  int64_t piece_elements() const;
  int64_t piece_bytes() const { return piece_elements() * dtype_bytes(dtype); }
  int total_degree() const;  // product of shard, sum and discard-copy degrees
  bool is_unparallel() const { return total_degree() == 1; }
  PShape reduced() const;  // same sizes, all degrees 1  (get_reduced_shape)
  bool operator==(const PShape &o) const {
    return dims == o.dims && sum_degree == o.sum_degree && discard_copy_degree == o.discard_copy_degree &&
           dtype == o.dtype;
  }
  bool operator!=(const PShape &o) const { return !(*this == o); }
  std::string str() const;
  Json to_json_parallel() const;  // ParallelTensorShape layout
  Json to_json_plain() const;     // TensorShape layout
  static PShape from_json(const Json &);  // accepts either layout
};

// ---------------------------------------------------------------- machine
enum class DeviceType { GPU, CPU };
struct MachineSpec {  // lib/pcg/include/pcg/machine_specification.dtg.toml
  int num_nodes = 1;
  int num_cpus_per_node = 1;
  int num_gpus_per_node = 1;
  double inter_node_bandwidth = 25.0;   // GB/s
  double intra_node_bandwidth = 770.0;  // GB/s, NVLink 5 peer copy per direction
  // Which machine views the mapping search may give an operator (not part of the serialised specification):
  // 0 = contiguous, start-aligned blocks; 1 = those plus power-of-two strides inside a node; 2 = every start, stride vector
  // and inter- / intra-node projection that fits, the reference's enumeration (allowed_machine_views.cc:51-162).
  int view_enumeration = 0;
  int num_devices() const { return num_nodes * num_gpus_per_node; }
  Json to_json() const;
  static MachineSpec from_json(const Json &);
};
// lib/compiler: MachineView{start, dimensions[{stride, INTER_NODE|INTRA_NODE}]}
struct MachineViewDim {
  int stride;
  bool inter_node;
  bool operator==(const MachineViewDim &o) const { return stride == o.stride && inter_node == o.inter_node; }
  bool operator<(const MachineViewDim &o) const { return std::tie(stride, inter_node) < std::tie(o.stride, o.inter_node); }
};
struct MachineView {
  int start_node = 0;
  int start_device = 0;
  std::vector<MachineViewDim> dims;
  bool operator==(const MachineView &o) const {
    return start_node == o.start_node && start_device == o.start_device && dims == o.dims;
  }
  bool operator<(const MachineView &o) const {
    return std::tie(start_node, start_device, dims) < std::tie(o.start_node, o.start_device, o.dims);
  }
  Json to_json() const;
  static MachineView from_json(const Json &);
  std::string str() const;
};

// ---------------------------------------------------------------- graph
using NodeId = int;
struct ValueRef {
  NodeId node;
  Slot slot;
  bool operator==(const ValueRef &o) const { return node == o.node && slot == o.slot; }
  bool operator<(const ValueRef &o) const { return std::tie(node, slot) < std::tie(o.node, o.slot); }
};
struct InEdge {
  Slot dst_slot;
  ValueRef src;
};
struct OutValue {
  Slot slot;
  PShape shape;
  bool create_grad = true;
};
struct Node {
  OpType type;
  Json attrs;  // object keyed by the reference attrs field names
  std::string name;
  std::vector<InEdge> inputs;
  std::vector<OutValue> outputs;
  std::optional<MachineView> view;  // set in mapped graphs
  const OutValue &out(Slot s) const;
  const InEdge *in(Slot s) const;
};

class Graph {
public:
  NodeId add_node(OpType type, Json attrs, std::string name, std::vector<InEdge> inputs,
                  std::vector<OutValue> outputs);
  void remove_node(NodeId);
  bool has_node(NodeId n) const { return nodes_.count(n) > 0; }
  const Node &node(NodeId n) const;
  Node &node(NodeId n);
  const std::map<NodeId, Node> &nodes() const { return nodes_; }
  size_t num_nodes() const { return nodes_.size(); }
  const PShape &shape(const ValueRef &v) const { return node(v.node).out(v.slot).shape; }
  std::vector<NodeId> node_ids() const;
  std::vector<NodeId> topological_order() const;
  // (consumer node, consumer slot) pairs of a value
  std::vector<std::pair<NodeId, Slot>> consumers(const ValueRef &v) const;
  std::vector<NodeId> successors(NodeId n) const;
  std::vector<NodeId> predecessors(NodeId n) const;
  std::vector<ValueRef> all_values() const;
  // values that no node consumes
  std::vector<ValueRef> sink_values() const;
  void replace_uses(const ValueRef &from, const ValueRef &to);
  bool is_mapped() const;
  // structural signature independent of node ids (used to dedupe search states)
  std::string signature() const;
  std::string as_dot() const;
  int next_id() const { return next_id_; }

private:
  std::map<NodeId, Node> nodes_;
  int next_id_ = 0;
};

// ---------------------------------------------------------------- shape inference
using SlotShapes = std::vector<std::pair<Slot, PShape>>;
struct Inferred {
  SlotShapes weights;  // weight slots this operator expects, with their (parallel) shapes
  SlotShapes outputs;
};
// Parallel shape inference for every operator (reference: lib/op-attrs/src/op-attrs/ops/*.cc,
// lib/op-attrs/src/op-attrs/shape_inference.cc).  `inputs` are the data inputs by slot.
// Throws ff::Error when the attributes and shapes do not fit.
Inferred infer_shapes(OpType type, const Json &attrs, const SlotShapes &inputs);
// Slots of `type` that hold weights rather than activations.
bool is_weight_slot(OpType type, Slot s);
// Default initializer attrs (JSON) of a weight slot, lib/op-attrs/src/op-attrs/ops/linear.cc:234-287 etc.
Json default_initializer(OpType type, Slot s, const Json &attrs, const SlotShapes &inputs);
const PShape *find_slot(const SlotShapes &s, Slot slot);

// Operator task space: the grid of parallel tasks an operator runs as
// (lib/op-attrs/include/op-attrs/operator_task_space.h).  Degrees with value 1 are dropped.
std::vector<int> operator_task_space(const Node &n, const Graph &g);
// For a task coordinate of the operator, the shard coordinate of one of its tensors
// (lib/op-attrs/src/op-attrs/get_operator_space_to_parallel_tensor_space_mappings.cc:19-116,
// extended to every operator).  Returned: {sum_component, discard_copy_component, shard components...}.
struct TensorCoord {
  int sum_component = 0;
  int discard_copy_component = 0;
  std::vector<int> shard;
};
// full (non-minimal) task-space degrees of an operator: one entry per output shard dim,
// then sum, then discard-copy
std::vector<int> operator_full_task_degrees(const Node &n, const Graph &g);
// Implemented for Input, Weight, the element-wise unary and binary operators, Transpose, Linear (the reference's list)
// and the four parallel operators; other operators throw.
TensorCoord operator_tensor_coord(const Node &n, const Graph &g, const std::vector<int> &task, Slot slot, bool is_output);

// ---------------------------------------------------------------- v1 file format
// lib/pcg/include/pcg/file_format/v1/** : {"raw_graph": {"node_labels", "output_labels", "graph"}}
Json graph_to_v1(const Graph &g, bool parallel);
Graph graph_from_v1(const Json &j);

}  // namespace ff
