// search.h -- strategy search: cost model, machine views, machine-mapping DP (with a runtime/memory Pareto
// variant), Unity best-first search over substitutions, MCMC search and the task-graph simulator.
//
// Reference counterparts: lib/compiler/src/compiler/machine_mapping/get_optimal_machine_mapping.cc:36-294,
// memory_optimization/get_optimal_machine_mapping_with_memory.cc, allowed_machine_views.cc:51-162,
// unity_algorithm/unity_algorithm.cc:51-146, mcmc/mcmc_over_mapped_pcg.cc:18-66,
// task_graph_simulator/task_simulator.cc:23-75, cost_estimator/cost_estimator.h:14-41.
#pragma once
#include <cmath>
#include <functional>
#include <set>
#include <map>
#include <memory>
#include <optional>
#include <random>
#include <string>
#include <vector>

#include "graph_algos.h"
#include "ir.h"
#include "substitutions.h"

namespace ff {

struct OpCost {
  double fwd_ms = 0, bwd_ms = 0;
  double memory_bytes = 0;  // per device
  double total_ms() const { return fwd_ms + bwd_ms; }
};

// Hardware constants of the analytical model.  Defaults are measurements of one B200 of an 8-GPU NVSwitch
// box: bf16 GEMM throughput sustained under the power cap, stream-copy HBM bandwidth, peer-copy NVLink
// bandwidth per direction and the 8-rank all-reduce bus bandwidth.
struct CostParams {
  double matmul_tflops = 1400.0;
  double matmul_efficiency = 0.8;   // fraction of the above a real GEMM kernel reaches
  double hbm_gbs = 6450.0;
  double nvlink_gbs = 770.0;
  double allreduce_bus_gbs = 725.0;
  double launch_us = 4.0;
  double collective_latency_us = 12.0;
  double inter_node_gbs = 25.0;
  double fused_overlap = 0.85;      // fraction of a collective hidden when it is fused with its GEMM
  int bytes_per_float = 2;          // activations/weights are bf16 at run time
  // Achieved bandwidth (GB/s, in the units the formulas use: bus bandwidth for an all-reduce, bytes received or sent per
  // rank for an all-gather / reduce-scatter) of this library's collective kernels as measured on this machine, by kind and
  // group size: "allreduce@8" -> 513.  A collective of a size that was not measured takes the entry of the nearest smaller
  // measured size, else the nominal figures above.  The defaults are the 2- and 8-GPU measurements of the peer-memory
  // kernels (gradient all-reduce, all-gather into a GEMM, GEMM into reduce-scatter).
  std::map<std::string, double> measured_gbs = {{"allreduce@2", 457.0}, {"allreduce@8", 513.0}, {"allgather@8", 342.0}, {"reducescatter@8", 172.0}};
  double collective_gbs(const std::string &kind, int group, double nominal) const;
  Json to_json() const;
  static CostParams from_json(const Json &);
};

class CostEstimator {
public:
  explicit CostEstimator(CostParams p = CostParams(), MachineSpec m = MachineSpec()) : params(p), machine(m) {}
  virtual ~CostEstimator() = default;
  CostParams params;
  MachineSpec machine;
  // measured costs override the analytical model; key = op_cost_key(node, graph)
  std::map<std::string, OpCost> measured;
  virtual OpCost op_cost(const Node &n, const Graph &g) const;
  // cost of moving `bytes` between two (different) device sets of the same node / across nodes
  virtual double movement_cost_ms(double bytes, bool inter_node) const;
  static std::string op_cost_key(const Node &n, const Graph &g);
  long long num_queries = 0;
};

// contiguous, start-aligned machine views of an operator with `task_degrees` on `resources`
struct Resources {
  int start = 0;
  int count = 1;
  bool operator<(const Resources &o) const { return std::tie(start, count) < std::tie(o.start, o.count); }
};
std::vector<MachineView> allowed_machine_views(const std::vector<int> &task_degrees, const Resources &r, const MachineSpec &m,
                                               bool strided = false);
std::vector<int> view_devices(const MachineView &v, const std::vector<int> &task_degrees, const MachineSpec &m);
// one tensor piece that has to travel between two devices
struct CommunicationEdge {
  int src_device, dst_device;
  double bytes;
};
std::vector<CommunicationEdge> get_tensor_set_movement(const Graph &g, NodeId src, const MachineView &vs, NodeId dst, const MachineView &vd,
                                                       const MachineSpec &m);
double tensor_set_movement_cost_ms(const std::vector<CommunicationEdge> &edges, const MachineSpec &m, const CostEstimator &est);

struct MappingPoint {
  double runtime_ms = 0;
  double memory_bytes = 0;
  std::map<NodeId, MachineView> views;
};
struct MachineMappingResult {
  std::vector<MappingPoint> front;  // Pareto front (size 1 when memory is not tracked); empty = infeasible
  bool feasible() const { return !front.empty(); }
  const MappingPoint &best_runtime() const;
};

// SP decomposition of a (parallel) computation graph with the weight/input pre-processing of the reference
// (get_pcg_series_parallel_decomposition.cc:12-78); falls back to SP-ization when the graph is not SP.
SPTree get_graph_sp_decomposition(const Graph &g, bool *exact = nullptr);

// Results of DP sub-problems, keyed by a structural hash of the sub-problem (subtree content, resources, imposed views).
// One cache may serve every candidate of a search: sub-problems outside the region a substitution rewrote hash the same
// and are not solved again (compiler/machine_mapping/machine_mapping_cache.cc).
struct MachineMappingCache {
  std::map<std::string, std::vector<MappingPoint>> table;
  std::map<std::string, double> movement;  // priced tensor set movements by (producer, view, consumer, view)
  long long hits = 0, misses = 0;
  long long truncated_boundaries = 0;  // series splits whose boundary had more than 256 view combinations
};

// `tree`: any SP decomposition of `pcg`; nodes with more than two children are grouped into pairs internally.
MachineMappingResult get_optimal_machine_mapping(const Graph &pcg, const SPTree &binary_tree, const MachineSpec &m,
                                                 const CostEstimator &est, int max_front = 1, MachineMappingCache *cache = nullptr);

struct SearchResult {
  Graph pcg;
  std::map<NodeId, MachineView> mapping;
  double runtime_ms = 0;
  double memory_bytes = 0;
  Json stats;
};
Graph mapped_pcg_from_pcg_and_mapping(const Graph &pcg, const std::map<NodeId, MachineView> &mapping);

struct UnityConfig {
  double alpha = 1.05;
  int budget = 10;
  int max_num_ops = 100000;
  int max_candidates_per_step = 4000;
  double time_limit_s = 120.0;
  bool single_moves = true;     // one candidate per (rule, match), as the reference does
  bool compound_moves = true;   // plus one candidate per rule: that rule applied wherever it matches
  bool cancel_after_compound = true;
  std::vector<std::vector<int>> families;  // groups of rule indices, each applied exhaustively as one move
  std::vector<int> cleanup_rules;  // indices (into the rule list) of the rules applied exhaustively after a compound move
};
SearchResult evaluate_pcg(const Graph &pcg, const MachineSpec &m, const CostEstimator &est, MachineMappingCache *cache = nullptr);
SearchResult unity_search(const Graph &start, const MachineSpec &m, const CostEstimator &est, const std::vector<Substitution> &rules,
                          const UnityConfig &cfg);
// apply every rule whose name passes `filter` wherever it matches, repeatedly, until nothing applies
Graph apply_rules_exhaustively(const Graph &g, const std::vector<Substitution> &rules, int max_applications = 100000,
                               int max_total_degree = 0);

struct MCMCConfig {
  double temperature = 1.0;
  int num_iterations = 100;
  double substitution_frequency = 0.2;
  unsigned seed = 0;
  bool relative_temperature = false;  // temperature as a fraction of the starting cost instead of milliseconds
};
SearchResult mcmc_search(const Graph &start, const MachineSpec &m, const CostEstimator &est, const std::vector<Substitution> &rules,
                         const MCMCConfig &cfg);

// Metropolis search over any state type (reference: compiler/mcmc/generic_mcmc_algorithm.h).  `sampler(state, rng)` proposes
// a neighbour or nothing; a proposal that costs less is taken, one that costs more with probability
// exp(-(cost - current cost) / temperature); the cheapest state seen is returned.  (The reference measures the increase
// against the best state instead of the current one; against the current one the chain can leave a local minimum and
// still come back.)  One cost evaluation per proposal; `accepted` counts the proposals taken.
template <typename State, typename Sampler, typename Cost, typename Rng>
State run_mcmc(const State &start, Sampler sampler, Cost cost, double temperature, int num_iterations, Rng &rng, int *accepted = nullptr,
               double *best_cost_out = nullptr) {
  std::uniform_real_distribution<double> uni(0.0, 1.0);
  State cur = start, best = start;
  double cur_cost = cost(cur), best_cost = cur_cost;
  int taken = 0;
  for (int it = 0; it < num_iterations; ++it) {
    std::optional<State> cand = sampler(cur, rng);
    if (!cand) continue;
    const double c = cost(*cand);
    const double accept_p = c <= cur_cost ? 1.0 : std::exp(-(c - cur_cost) / std::max(1e-12, temperature));
    if (uni(rng) < accept_p) {
      cur = std::move(*cand);
      cur_cost = c;
      ++taken;
      if (c < best_cost) {
        best = cur;
        best_cost = c;
      }
    }
  }
  if (accepted) *accepted = taken;
  if (best_cost_out) *best_cost_out = best_cost;
  return best;
}

// Machine views with the reference's stride semantics (compiler/machine_mapping/machine_view.cc:65-135,
// allowed_machine_views.cc:51-162), next to the absolute-stride views the mapping search uses (allowed_machine_views above).
// Here a view's stride is relative: the task dims projected onto the same machine dimension (inter-node / intra-node) are
// combined first-dim-fastest, dim k weighing prod_{i<k}(degree_i * stride_i) * stride_k.  `reference_machine_coordinate` maps a
// task coordinate to (node, device); `reference_allowed_machine_views` enumerates every (start, strides, projections) whose
// last task stays inside a machine of num_nodes x gpus_per_node, strides up to ceil(devices / prod(degree_i - 1));
// `absolute_view_from_reference` rewrites such a view with absolute strides so that view_devices resolves it.
std::pair<int, int> reference_machine_coordinate(const MachineView &v, const std::vector<int> &task_degrees, const std::vector<int> &coord);
std::vector<MachineView> reference_allowed_machine_views(const std::vector<int> &task_degrees, int num_nodes, int gpus_per_node);
MachineView absolute_view_from_reference(const MachineView &v, const std::vector<int> &task_degrees);

// Event-driven execution of a task graph (reference: compiler/task_graph_simulator/simulate_task_graph_execution.cc).  Tasks
// 0..n-1 with durations `cost`, precedence `edges` (before, after).  A task whose predecessors have finished starts as soon
// as `allowed(task, in_progress, finished)` says so; ready tasks are offered in index order, again after every start and every
// completion; tasks that end at the same time complete together.  Throws when tasks remain that may never start.
struct TaskProfile {
  int task;
  double start, end;
};
using TaskConstraint = std::function<bool(int, const std::set<int> &, const std::set<int> &)>;
std::vector<TaskProfile> simulate_task_graph_execution(int n, const std::vector<std::pair<int, int>> &edges, const std::vector<double> &cost,
                                                       const TaskConstraint &allowed);

// Simulation of a mapped PCG on that engine: one task per operator (forward; with include_backward also the mirrored backward
// task) that occupies its devices exclusively, one unconstrained task per tensor movement between differing device sets.
// Returns the makespan in ms.
double simulate_task_graph(const Graph &mapped_pcg, const MachineSpec &m, const CostEstimator &est, bool include_backward = false);

}  // namespace ff
