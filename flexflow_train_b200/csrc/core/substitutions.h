// substitutions.h -- graph substitution engine.
//
// A Substitution is a pattern graph over PCG operators plus an output graph expression:
//   * the pattern (lib/substitutions/include/substitutions/pcg_pattern.h) is an open dataflow graph whose
//     nodes carry operator-attribute constraints (EQUAL / DIVISIBLE_BY on an attribute, the reference's
//     OperatorAttributePattern) and whose open inputs carry tensor constraints;
//   * the output expression (output_graph_expr.h) creates operators either from literal attributes or by
//     copying a matched operator ("template") and overriding attributes;
//   * applying a match (apply_substitution.cc:20-182) materialises the new operators, re-runs parallel
//     shape inference, checks that the interface shapes are unchanged and splices the result in.
// The generated "Unity" rule set (unity_substitution_set.cc:24-76) and a loader for the legacy TASO-style
// JSON rule collections (lib/substitution-generator/include/substitution-generator/legacy_rules.h) are here too.
#pragma once
#include <map>
#include <optional>
#include <string>
#include <vector>

#include "ir.h"

namespace ff {

struct AttrConstraint {
  enum Kind { EQUAL, DIVISIBLE_BY } kind = EQUAL;
  std::string key;  // "op_type", or an attribute field name of the operator
  Json value;
};
struct TensorConstraint {
  enum Kind { DIM_DIVISIBLE_BY, NUM_DIMS_AT_LEAST, DIM_DEGREE_EQUAL, SUM_DEGREE_EQUAL, COPY_DEGREE_EQUAL } kind;
  int dim = 0;  // may be negative (from the end)
  long long value = 1;
};
struct PatternInput {
  Slot slot;
  bool from_graph_input = false;
  int index = 0;    // graph input index, or pattern node index
  Slot src_slot = Slot::OUTPUT;
};
struct PatternNode {
  std::vector<AttrConstraint> constraints;
  std::vector<PatternInput> inputs;
  bool allow_extra_inputs = false;  // operator may have further (e.g. optional BIAS) inputs not listed
};
struct Pattern {
  std::vector<PatternNode> nodes;
  int num_inputs = 0;
  std::map<int, std::vector<TensorConstraint>> input_constraints;
};

struct AttrExpr {
  enum Kind { LITERAL, ATTR_OF } kind = LITERAL;
  Json literal;
  int pattern_node = 0;
  std::string key;
};
struct OutInput {
  Slot slot;
  bool from_graph_input = false;
  int index = 0;
  Slot src_slot = Slot::OUTPUT;
};
struct OutNode {
  std::optional<int> template_node;  // copy type + attrs of this matched pattern node
  OpType type = OpType::NOOP;        // used when there is no template
  std::map<std::string, AttrExpr> assigns;
  std::vector<OutInput> inputs;
};
struct InterfaceOutput {  // value produced by the pattern  <->  value produced by the output graph
  int pattern_node;
  Slot pattern_slot;
  int out_node;
  Slot out_slot;
};
struct Substitution {
  std::string name;
  Pattern pattern;
  std::vector<OutNode> out_nodes;
  std::vector<InterfaceOutput> outputs;
  Json to_json() const;
};

struct Match {
  std::vector<NodeId> nodes;      // pattern node i -> graph node
  std::vector<ValueRef> inputs;   // pattern graph input i -> graph value
  bool operator<(const Match &o) const { return nodes < o.nodes; }
};

bool is_valid_substitution(const Substitution &s, std::string *why = nullptr);
std::vector<Match> find_pattern_matches(const Pattern &p, const Graph &g);
// nullopt when the substitution does not apply at this match (shape inference rejects the new operators or
// the interface shapes would change)
std::optional<Graph> apply_substitution(const Graph &g, const Substitution &s, const Match &m, std::string *why = nullptr);

// builders of the generated rule set
Substitution create_replicate_linear_combine(int degree, bool use_bias);
Substitution create_partition_linear_combine(int dim, int degree, bool use_bias);
Substitution create_partition_linear_reduce(int degree, bool use_bias);  // row-parallel: emits Reduction
Substitution create_partition_conv2d_combine(int degree, bool use_bias);
Substitution create_partition_attention_combine(int degree, bool bias);
Substitution create_replicate_attention_reduce(int degree, bool bias);
Substitution create_partition_unary_combine(OpType op, int dim, int degree);
Substitution create_partition_binary_combine(OpType op, int dim, int degree);
Substitution create_partition_softmax_combine(int softmax_dim, int dim, int degree);
Substitution create_partition_layernorm_combine(int dim, int degree, bool affine);
Substitution create_partition_embedding_combine(int dim, int degree);
Substitution create_partition_batchnorm_combine(int dim, int degree, bool affine);
Substitution create_partition_concat_combine(int num_inputs, int axis, int dim, int degree);
Substitution create_fuse_linear_activation(const std::string &activation);
Substitution create_cancel_combine_repartition();   // Combine(d,k) -> Repartition(d,k)  ==> identity
Substitution create_cancel_repartition_combine();
Substitution create_cancel_replicate_reduction_free();  // Replicate(k) feeding only a Combine-free noop (kept for completeness)
std::vector<Substitution> get_substitution_set(const MachineSpec &m, int max_dims = 4);
// Combine -> Replicate / Reduction  ==>  Replicate / Reduction -> Combine (not part of the default set: the
// tensor+sequence-parallel template wants Combine(0) -> Replicate to stay adjacent, as that pair is one all-gather)
std::vector<Substitution> get_commute_rules();

// legacy TASO rule files: {"_t":"RuleCollection","rule":[{"name","srcOp":[...],"dstOp":[...],"mappedOutput":[...]}]}
struct LegacyRuleStats {
  int num_rules = 0;
  int num_converted = 0;
  std::map<std::string, int> op_histogram;
};
std::vector<Substitution> load_legacy_rules(const Json &collection, LegacyRuleStats *stats = nullptr);
std::string substitution_as_dot(const Substitution &s);
std::string legacy_rule_as_dot(const Json &rule);

}  // namespace ff
