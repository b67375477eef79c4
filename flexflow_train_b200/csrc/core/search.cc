#include "search.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <functional>
#include <limits>
#include <queue>
#include <set>

#include <pybind11/functional.h>

#include "pyjson.h"

namespace ff {

// ---------------------------------------------------------------- cost model
Json CostParams::to_json() const {
  Json j = Json::object();
  j["matmul_tflops"] = matmul_tflops; j["matmul_efficiency"] = matmul_efficiency; j["hbm_gbs"] = hbm_gbs;
  j["nvlink_gbs"] = nvlink_gbs; j["allreduce_bus_gbs"] = allreduce_bus_gbs; j["launch_us"] = launch_us;
  j["collective_latency_us"] = collective_latency_us; j["inter_node_gbs"] = inter_node_gbs;
  j["fused_overlap"] = fused_overlap; j["bytes_per_float"] = bytes_per_float;
  Json mg = Json::object();
  for (auto &kv : measured_gbs) mg[kv.first] = kv.second;
  j["measured_gbs"] = mg;
  return j;
}
double CostParams::collective_gbs(const std::string &kind, int group, double nominal) const {
  double best = nominal;
  int best_size = 0;
  for (auto &kv : measured_gbs) {
    auto at = kv.first.find('@');
    if (at == std::string::npos || kv.first.compare(0, at, kind) != 0) continue;
    int size = std::atoi(kv.first.c_str() + at + 1);
    if (size <= group && size > best_size) {
      best_size = size;
      best = kv.second;
    }
  }
  return best;
}
CostParams CostParams::from_json(const Json &j) {
  CostParams p;
  p.matmul_tflops = j.get_float("matmul_tflops", p.matmul_tflops);
  p.matmul_efficiency = j.get_float("matmul_efficiency", p.matmul_efficiency);
  p.hbm_gbs = j.get_float("hbm_gbs", p.hbm_gbs);
  p.nvlink_gbs = j.get_float("nvlink_gbs", p.nvlink_gbs);
  p.allreduce_bus_gbs = j.get_float("allreduce_bus_gbs", p.allreduce_bus_gbs);
  p.launch_us = j.get_float("launch_us", p.launch_us);
  p.collective_latency_us = j.get_float("collective_latency_us", p.collective_latency_us);
  p.inter_node_gbs = j.get_float("inter_node_gbs", p.inter_node_gbs);
  p.fused_overlap = j.get_float("fused_overlap", p.fused_overlap);
  p.bytes_per_float = (int)j.get_int("bytes_per_float", p.bytes_per_float);
  if (j.contains("measured_gbs")) {
    p.measured_gbs.clear();
    for (auto &kv : j.at("measured_gbs").fields()) p.measured_gbs[kv.first] = kv.second.as_float();
  }
  return p;
}

static double elem_bytes(const PShape &s, const CostParams &p) {
  if (s.dtype == DataType::FLOAT || s.dtype == DataType::HALF || s.dtype == DataType::BFLOAT16) return p.bytes_per_float;
  return dtype_bytes(s.dtype);
}
static double piece_bytes(const PShape &s, const CostParams &p) { return (double)s.piece_elements() * elem_bytes(s, p); }

std::string CostEstimator::op_cost_key(const Node &n, const Graph &g) {
  std::string k = to_string(n.type) + n.attrs.canonical();
  for (auto &e : n.inputs) k += "|" + to_string(e.dst_slot) + ":" + g.shape(e.src).str();
  return k;
}

double CostEstimator::movement_cost_ms(double bytes, bool inter_node) const {
  double bw = inter_node ? params.inter_node_gbs : params.nvlink_gbs;
  return params.collective_latency_us * 1e-3 + bytes / (bw * 1e9) * 1e3;
}

OpCost CostEstimator::op_cost(const Node &n, const Graph &g) const {
  const_cast<CostEstimator *>(this)->num_queries++;
  if (!measured.empty()) {
    auto it = measured.find(op_cost_key(n, g));
    if (it != measured.end()) return it->second;
  }
  const CostParams &p = params;
  OpCost c;
  double in_bytes = 0, out_bytes = 0, weight_bytes = 0;
  for (auto &e : n.inputs) {
    double b = piece_bytes(g.shape(e.src), p);
    if (is_weight_slot(n.type, e.dst_slot)) weight_bytes += b;
    else in_bytes += b;
  }
  for (auto &o : n.outputs) out_bytes += piece_bytes(o.shape, p);
  c.memory_bytes = out_bytes;
  const double flops_per_ms = p.matmul_tflops * p.matmul_efficiency * 1e9;
  const double bytes_per_ms = p.hbm_gbs * 1e6;
  const double launch = p.launch_us * 1e-3;
  auto mem_time = [&](double bytes) { return bytes / bytes_per_ms; };
  auto coll_lat = p.collective_latency_us * 1e-3;
  switch (n.type) {
    case OpType::INPUT:
      return c;
    case OpType::WEIGHT:
      // parameters plus gradient plus fp32 master and Adam moments (2 + 2 + 4 + 4 + 4 bytes per element)
      c.memory_bytes = (double)n.outputs[0].shape.piece_elements() * 16.0;
      return c;
    case OpType::NOOP:
      c.memory_bytes = 0;
      return c;
    case OpType::LINEAR: {
      const PShape &x = g.shape(n.in(Slot::INPUT)->src);
      const PShape &y = n.outputs[0].shape;
      double rows = (double)x.piece_elements() / ((double)x.dims.back().size / x.dims.back().degree);
      double k = (double)x.dims.back().size / x.dims.back().degree;
      double nn = (double)y.dims.back().size / y.dims.back().degree;
      double flops = 2.0 * rows * k * nn;
      c.fwd_ms = std::max(flops / flops_per_ms, mem_time(in_bytes + out_bytes + weight_bytes)) + launch;
      c.bwd_ms = std::max(2.0 * flops / flops_per_ms, mem_time(2 * (in_bytes + out_bytes) + 2 * weight_bytes)) + 2 * launch;
      return c;
    }
    case OpType::BATCHMATMUL: {
      const PShape &a = g.shape(n.in(Slot::LHS_INPUT)->src);
      const PShape &y = n.outputs[0].shape;
      double m = (double)a.dims.back().size / a.dims.back().degree;
      double flops = 2.0 * (double)y.piece_elements() * m;
      c.fwd_ms = std::max(flops / flops_per_ms, mem_time(in_bytes + out_bytes)) + launch;
      c.bwd_ms = 2 * c.fwd_ms;
      return c;
    }
    case OpType::MULTIHEAD_ATTENTION: {
      const PShape &q = g.shape(n.in(Slot::QUERY)->src);
      const PShape &k = g.shape(n.in(Slot::KEY)->src);
      double heads = (double)n.attrs.at("num_heads").as_int() / std::max(1, q.discard_copy_degree);
      double kd = (double)n.attrs.at("kdim").as_int(), vd = (double)n.attrs.at("vdim").as_int();
      double e = (double)n.attrs.at("embed_dim").as_int();
      double b = (double)q.dims[0].size / q.dims[0].degree, sq = (double)q.dims[1].size, sk = (double)k.dims[1].size;
      double dq = (double)q.dims[2].size;
      double proj = 2.0 * b * (sq * dq * heads * kd + 2.0 * sk * dq * heads * (kd + vd) / 2.0 + sq * heads * vd * e);
      double core = 2.0 * b * heads * sq * sk * (kd + vd);
      double score_bytes = b * heads * sq * sk * p.bytes_per_float;
      c.fwd_ms = std::max((proj + core) / flops_per_ms, mem_time(in_bytes + out_bytes + weight_bytes + 4.0 * score_bytes)) + 6 * launch;
      c.bwd_ms = std::max(2.0 * (proj + core) / flops_per_ms, mem_time(2 * (in_bytes + out_bytes) + 2 * weight_bytes + 8.0 * score_bytes)) + 12 * launch;
      c.memory_bytes = out_bytes + score_bytes + b * sq * heads * (2 * kd + 2 * vd) * p.bytes_per_float;
      return c;
    }
    case OpType::CONV2D: {
      const PShape &x = g.shape(n.in(Slot::INPUT)->src);
      const PShape &y = n.outputs[0].shape;
      double ic = (double)x.dims[1].size / x.dims[1].degree;
      double flops = 2.0 * (double)y.piece_elements() * ic * (double)n.attrs.at("kernel_h").as_int() * (double)n.attrs.at("kernel_w").as_int();
      // implicit GEMM on small, odd channel counts reaches a smaller share of the tensor-core peak than Linear
      c.fwd_ms = std::max(flops / (0.5 * flops_per_ms), mem_time(in_bytes + out_bytes + weight_bytes)) + launch;
      c.bwd_ms = 2 * c.fwd_ms;
      return c;
    }
    case OpType::EMBEDDING:
      c.fwd_ms = mem_time(2 * out_bytes) + launch;
      c.bwd_ms = mem_time(3 * out_bytes) + launch;
      return c;
    // ---- parallel operators: collectives over NVLink (degree within one node) ----
    case OpType::REPARTITION: {
      int k = (int)n.attrs.at("repartition_degree").as_int();
      // forward: every rank keeps its slice of data it already holds; backward: all-gather of the gradient
      c.fwd_ms = launch;
      c.bwd_ms = coll_lat + in_bytes * (k - 1.0) / k / (p.collective_gbs("allgather", k, p.nvlink_gbs) * 1e6);
      c.memory_bytes = out_bytes;
      return c;
    }
    case OpType::COMBINE: {
      int k = (int)n.attrs.at("combine_degree").as_int();
      c.fwd_ms = coll_lat + out_bytes * (k - 1.0) / k / (p.collective_gbs("allgather", k, p.nvlink_gbs) * 1e6);
      c.bwd_ms = launch;
      return c;
    }
    case OpType::REPLICATE: {
      int k = (int)n.attrs.at("replicate_degree").as_int();
      // forward is free in SPMD execution (the tensor already lives on every rank); backward sums the
      // replicas' gradients: an all-reduce, overlapped with the rest of backward when it is a weight gradient
      double ar = coll_lat + 2.0 * in_bytes * (k - 1.0) / k / (p.collective_gbs("allreduce", k, p.allreduce_bus_gbs) * 1e6);
      bool weight_grad = g.node(n.inputs[0].src.node).type == OpType::WEIGHT ||
                         (is_parallel_op(g.node(n.inputs[0].src.node).type) && !g.node(n.inputs[0].src.node).inputs.empty() &&
                          g.node(g.node(n.inputs[0].src.node).inputs[0].src.node).type == OpType::WEIGHT);
      c.fwd_ms = 0;
      c.bwd_ms = weight_grad ? ar * (1.0 - p.fused_overlap) : ar;
      c.memory_bytes = 0;
      return c;
    }
    case OpType::REDUCTION: {
      int k = (int)n.attrs.at("reduction_degree").as_int();
      double ar = coll_lat + 2.0 * out_bytes * (k - 1.0) / k / (p.collective_gbs("allreduce", k, p.allreduce_bus_gbs) * 1e6);
      // fused with the producing GEMM (GEMM -> reduce-scatter kernel) most of the transfer hides under the math
      const Node &prod = g.node(n.inputs[0].src.node);
      bool fused = prod.type == OpType::LINEAR || prod.type == OpType::BATCHMATMUL || prod.type == OpType::MULTIHEAD_ATTENTION;
      c.fwd_ms = fused ? ar * (1.0 - p.fused_overlap) + coll_lat : ar;
      c.bwd_ms = 0;
      return c;
    }
    default: {
      // bandwidth-bound operators: forward reads inputs and writes outputs, backward about twice that
      c.fwd_ms = mem_time(in_bytes + out_bytes + weight_bytes) + launch;
      c.bwd_ms = mem_time(2 * in_bytes + 2 * out_bytes) + launch;
      if (n.type == OpType::RESHAPE || n.type == OpType::FLAT) { c.fwd_ms = 0; c.bwd_ms = 0; c.memory_bytes = 0; }
      return c;
    }
  }
}

// ---------------------------------------------------------------- machine views
std::vector<MachineView> allowed_machine_views(const std::vector<int> &task_degrees, const Resources &r, const MachineSpec &m, bool strided) {
  int count = 1;
  for (int d : task_degrees) count *= d;
  std::vector<MachineView> out;
  if (count > r.count) return out;
  const int per_node = m.num_gpus_per_node;
  strided = strided || m.view_enumeration == 1;
  if (m.view_enumeration == 2) {
    // the reference's enumeration over the whole machine, kept where every task lands inside the resource range on its own
    // device; rewritten with absolute strides, which is what view_devices and the rest of the search read
    std::set<MachineView> seen;
    for (auto &v : reference_allowed_machine_views(task_degrees, m.num_nodes, per_node)) {
      MachineView a = absolute_view_from_reference(v, task_degrees);
      auto devs = view_devices(a, task_degrees, m);
      std::set<int> distinct(devs.begin(), devs.end());
      bool inside = distinct.size() == devs.size();
      for (int d : devs) inside = inside && d >= r.start && d < r.start + r.count;
      if (inside && seen.insert(a).second) out.push_back(a);
    }
    return out;
  }
  if (strided && count > 1) {
    // Strided placements inside one node (the reference's MachineView stride, allowed_machine_views.cc:51-162): the
    // tasks sit on every s-th device, s a power of two, so that s interleaved groups tile a block of count * s devices.
    // s = 1 gives the contiguous views below.  On an NVSwitch node all of them cost the same, which is why the mapping
    // search does not ask for them; a machine with a ring or a mesh between its GPUs would.
    for (int s = 2; count * s <= r.count && r.start % per_node + r.count <= per_node; s *= 2) {
      for (int block = r.start; block + count * s <= r.start + r.count; block += count * s) {
        for (int off = 0; off < s; ++off) {
          MachineView v;
          v.start_node = (block + off) / per_node;
          v.start_device = (block + off) % per_node;
          int stride = s;
          std::vector<MachineViewDim> dims(task_degrees.size());
          for (int i = (int)task_degrees.size() - 1; i >= 0; --i) {
            dims[i] = {stride, false};
            stride *= task_degrees[i];
          }
          v.dims = dims;
          out.push_back(v);
        }
      }
    }
  }
  std::vector<MachineView> contiguous;
  for (int start = r.start; start + count <= r.start + r.count; start += count) {
    MachineView v;
    v.start_node = start / per_node;
    v.start_device = start % per_node;
    int stride = 1;
    std::vector<MachineViewDim> dims(task_degrees.size());
    for (int i = (int)task_degrees.size() - 1; i >= 0; --i) {
      // contiguous layout: the last task dim varies fastest; a dim whose stride reaches the node size crosses nodes
      bool inter = stride >= per_node;
      dims[i] = {inter ? stride / per_node : stride, inter};
      stride *= task_degrees[i];
    }
    v.dims = dims;
    contiguous.push_back(v);
  }
  contiguous.insert(contiguous.end(), out.begin(), out.end());   // contiguous views first, then the strided ones
  return contiguous;
}
std::vector<int> view_devices(const MachineView &v, const std::vector<int> &task_degrees, const MachineSpec &m) {
  std::vector<int> devs;
  int n = 1;
  for (int d : task_degrees) n *= d;
  int base = v.start_node * m.num_gpus_per_node + v.start_device;
  for (int t = 0; t < n; ++t) {
    int rem = t, dev = base;
    for (int i = (int)task_degrees.size() - 1; i >= 0; --i) {
      int c = rem % task_degrees[i];
      rem /= task_degrees[i];
      int stride = i < (int)v.dims.size() ? v.dims[i].stride * (v.dims[i].inter_node ? m.num_gpus_per_node : 1) : 1;
      dev += c * stride;
    }
    devs.push_back(dev);
  }
  return devs;
}

// ---------------------------------------------------------------- machine views, reference stride semantics
namespace {
// weight of task dim k among the dims that share its projection: product of (degree * stride) of the earlier ones
std::vector<long long> reference_dim_weights(const MachineView &v, const std::vector<int> &deg) {
  if (v.dims.size() != deg.size()) throw Error("machine view has " + std::to_string(v.dims.size()) + " dims, the task space " + std::to_string(deg.size()));
  std::vector<long long> w(deg.size(), 1);
  long long acc[2] = {1, 1};
  for (size_t k = 0; k < deg.size(); ++k) {
    const int p = v.dims[k].inter_node ? 1 : 0;
    w[k] = acc[p] * v.dims[k].stride;
    acc[p] *= (long long)deg[k] * v.dims[k].stride;
  }
  return w;
}
}  // namespace
std::pair<int, int> reference_machine_coordinate(const MachineView &v, const std::vector<int> &deg, const std::vector<int> &coord) {
  if (coord.size() != deg.size()) throw Error("task coordinate and task space differ in rank");
  auto w = reference_dim_weights(v, deg);
  long long node = v.start_node, dev = v.start_device;
  for (size_t k = 0; k < deg.size(); ++k) {
    if (coord[k] < 0 || coord[k] >= deg[k]) throw Error("task coordinate outside the task space");
    (v.dims[k].inter_node ? node : dev) += w[k] * coord[k];
  }
  return {(int)node, (int)dev};
}
std::vector<MachineView> reference_allowed_machine_views(const std::vector<int> &deg, int num_nodes, int gpus_per_node) {
  long long full = 1;
  for (int d : deg) full *= std::max(d - 1, 0);
  full = std::max(full, 1ll);
  const int total = num_nodes * gpus_per_node;
  const int max_stride = (int)((total + full - 1) / full);
  std::vector<int> last;
  for (int d : deg) last.push_back(d - 1);
  std::vector<MachineView> out;
  const size_t nd = deg.size();
  std::vector<int> stride(nd, 1);
  for (;;) {   // every stride vector in [1, max_stride]^nd
    for (unsigned proj = 0; proj < (1u << nd); ++proj)
      for (int node = 0; node < num_nodes; ++node)
        for (int dev = 0; dev < gpus_per_node; ++dev) {
          MachineView v;
          v.start_node = node;
          v.start_device = dev;
          for (size_t k = 0; k < nd; ++k) v.dims.push_back({stride[k], ((proj >> k) & 1u) != 0});
          auto mx = reference_machine_coordinate(v, deg, last);
          if (mx.first < num_nodes && mx.second < gpus_per_node) out.push_back(v);
        }
    size_t k = 0;
    while (k < nd && ++stride[k] > max_stride) stride[k++] = 1;
    if (k == nd) break;
  }
  return out;
}
MachineView absolute_view_from_reference(const MachineView &v, const std::vector<int> &deg) {
  auto w = reference_dim_weights(v, deg);
  MachineView a = v;
  for (size_t k = 0; k < deg.size(); ++k) a.dims[k].stride = (int)w[k];
  return a;
}

// ---------------------------------------------------------------- tensor set movement
// Which pieces travel between which devices when `src` (placed by view `vs`) feeds `dst` (placed by `vd`): for every
// task of the consumer, the shard of the tensor it reads (operator_tensor_coord) is looked up among the producer's
// tasks; a piece whose producing and consuming tasks sit on different devices is one communication edge
// (compiler/machine_mapping/abstracted_tensor_set_movement -> TensorSetMovement{CommunicationEdge -> bytes}).
static int flat_minimal_task(const std::vector<int> &full, const std::vector<int> &task) {
  int f = 0;
  for (size_t i = 0; i < full.size(); ++i)
    if (full[i] > 1) f = f * full[i] + task[i];
  return f;
}
static void for_each_task(const std::vector<int> &full, const std::function<void(const std::vector<int> &)> &fn) {
  std::vector<int> t(full.size(), 0);
  while (true) {
    fn(t);
    int i = (int)full.size() - 1;
    while (i >= 0 && ++t[i] == full[i]) t[i--] = 0;
    if (i < 0) return;
  }
}
std::vector<CommunicationEdge> get_tensor_set_movement(const Graph &g, NodeId src, const MachineView &vs, NodeId dst, const MachineView &vd,
                                                       const MachineSpec &m) {
  const Node &p = g.node(src), &c = g.node(dst);
  const std::vector<int> fp = operator_full_task_degrees(p, g), fc = operator_full_task_degrees(c, g);
  const std::vector<int> dp = view_devices(vs, operator_task_space(p, g), m), dc = view_devices(vd, operator_task_space(c, g), m);
  std::vector<CommunicationEdge> out;
  std::set<std::tuple<int, int, std::vector<int>>> seen;
  for (auto &e : c.inputs) {
    if (e.src.node != src) continue;
    using Key = std::vector<int>;  // shard..., sum, copy
    auto key_of = [](const TensorCoord &tc) {
      Key k = tc.shard;
      k.push_back(tc.sum_component);
      k.push_back(tc.discard_copy_component);
      return k;
    };
    std::map<Key, int> producer_device;
    for_each_task(fp, [&](const std::vector<int> &t) {
      producer_device[key_of(operator_tensor_coord(p, g, t, e.src.slot, true))] = dp.at((size_t)flat_minimal_task(fp, t));
    });
    const double bytes = (double)g.shape(e.src).piece_bytes();
    for_each_task(fc, [&](const std::vector<int> &t) {
      Key k = key_of(operator_tensor_coord(c, g, t, e.dst_slot, false));
      auto it = producer_device.find(k);
      if (it == producer_device.end()) throw Error("tensor set movement: the consumer reads a piece its producer does not make");
      const int to = dc.at((size_t)flat_minimal_task(fc, t));
      if (it->second != to && seen.insert({it->second, to, k}).second) out.push_back({it->second, to, bytes});
    });
  }
  return out;
}
// max over the point-to-point edges of bytes / bandwidth (lib/local-execution/.../local_cost_estimator.cc:155-179)
double tensor_set_movement_cost_ms(const std::vector<CommunicationEdge> &edges, const MachineSpec &m, const CostEstimator &est) {
  double worst = 0;
  for (auto &e : edges) {
    const bool inter = e.src_device / m.num_gpus_per_node != e.dst_device / m.num_gpus_per_node;
    worst = std::max(worst, est.movement_cost_ms(e.bytes, inter));
  }
  return worst;
}

// ---------------------------------------------------------------- SP decomposition of a graph
static DiGraph graph_digraph(const Graph &g) {
  DiGraph d;
  for (auto &kv : g.nodes()) {
    d.add_node(kv.first);
    for (auto &e : kv.second.inputs) d.add_edge(e.src.node, kv.first);
  }
  return d;
}
SPTree get_graph_sp_decomposition(const Graph &g, bool *exact) {
  DiGraph d = graph_digraph(g);
  if (exact) *exact = true;
  if (auto t = get_series_parallel_decomposition(d)) return *t;
  // weights and inputs, each with its trailing chain of parallel ops, are connected all-to-all to the
  // successors of those chains: this hoists them in front of the computation
  std::set<int> sources, chain_nodes;
  for (auto &kv : g.nodes())
    if (kv.second.type == OpType::WEIGHT || kv.second.type == OpType::INPUT) sources.insert(kv.first);
  std::map<int, int> chain_end;  // source -> last node of its parallel-op chain
  for (int s : sources) {
    int cur = s;
    while (true) {
      auto succ = g.successors(cur);
      if (succ.size() == 1 && is_parallel_op(g.node(succ[0]).type) && g.predecessors(succ[0]).size() == 1) cur = succ[0];
      else break;
    }
    chain_end[s] = cur;
  }
  std::set<int> targets;
  for (auto &kv : chain_end)
    for (int t : g.successors(kv.second)) targets.insert(t);
  DiGraph d2 = d;
  for (auto &kv : chain_end)
    for (int t : targets) d2.add_edge(kv.second, t);
  if (is_acyclic(d2))
    if (auto t = get_series_parallel_decomposition(d2)) return *t;
  if (exact) *exact = false;
  return escribano_sp_ization(is_acyclic(d2) ? d2 : d);
}

// ---------------------------------------------------------------- machine-mapping DP
const MappingPoint &MachineMappingResult::best_runtime() const {
  if (front.empty()) throw Error("machine mapping is infeasible");
  size_t b = 0;
  for (size_t i = 1; i < front.size(); ++i) if (front[i].runtime_ms < front[b].runtime_ms) b = i;
  return front[b];
}

namespace {
using Front = std::vector<MappingPoint>;

void prune(Front &f, int max_front) {
  if (f.empty()) return;
  std::sort(f.begin(), f.end(), [](const MappingPoint &a, const MappingPoint &b) {
    return a.runtime_ms < b.runtime_ms || (a.runtime_ms == b.runtime_ms && a.memory_bytes < b.memory_bytes);
  });
  Front out;
  double best_mem = std::numeric_limits<double>::infinity();
  for (auto &p : f) {
    if (max_front == 1) { out.push_back(p); break; }
    if (p.memory_bytes < best_mem) { out.push_back(p); best_mem = p.memory_bytes; }
    if ((int)out.size() >= max_front) break;
  }
  f.swap(out);
}

// 64-bit mixing for structural hashes
inline uint64_t mix64(uint64_t h, uint64_t v) {
  h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
  h *= 0xBF58476D1CE4E5B9ull;
  return h ^ (h >> 29);
}
inline uint64_t hash_str(const std::string &s) {
  uint64_t h = 1469598103934665603ull;
  for (unsigned char c : s) { h ^= c; h *= 1099511628211ull; }
  return h;
}

// One sub-problem of the DP: a subtree of the binary SP tree with its leaves and a hash of everything inside it that
// the result depends on (operator cost keys, task spaces, the edges between its leaves).  Two subtrees with the same
// hash -- in this graph or in another candidate of the same search whose rewritten region lies elsewhere -- are the same
// sub-problem, which is what lets the cache survive from one candidate to the next
// (compiler/machine_mapping/machine_mapping_cache.cc keys its table by the problem tree in the same way).
struct Sub {
  SPTree::Kind kind = SPTree::Leaf;
  int node = -1;
  int left = -1, right = -1;
  std::vector<int> leaves;  // sorted
  uint64_t hash = 0;
  double work_ms = 0;  // sum of the operators' forward + backward times
};

struct DP {
  const Graph &g;
  const MachineSpec &m;
  const CostEstimator &est;
  int max_front;
  MachineMappingCache &cache;
  std::map<NodeId, OpCost> cost_cache;
  std::map<NodeId, std::vector<int>> task_cache;
  std::map<NodeId, uint64_t> node_hash;
  std::vector<Sub> subs;
  // operators that are not leaves of the tree but ride along with one that is: a weight or input with its chain of
  // parallel operators is placed with (and its time and memory are added to) the operator that consumes it
  std::map<NodeId, std::vector<NodeId>> attached;

  const OpCost &cost(NodeId n) {
    auto it = cost_cache.find(n);
    if (it == cost_cache.end()) {
      OpCost c = est.op_cost(g.node(n), g);
      auto at = attached.find(n);
      if (at != attached.end())
        for (NodeId a : at->second) {
          OpCost ca = est.op_cost(g.node(a), g);
          c.fwd_ms += ca.fwd_ms;
          c.bwd_ms += ca.bwd_ms;
          c.memory_bytes += ca.memory_bytes;
        }
      it = cost_cache.emplace(n, c).first;
    }
    return it->second;
  }
  const std::vector<int> &tasks(NodeId n) {
    auto it = task_cache.find(n);
    if (it == task_cache.end()) it = task_cache.emplace(n, operator_task_space(g.node(n), g)).first;
    return it->second;
  }
  uint64_t hash_of_node(NodeId n) {
    auto it = node_hash.find(n);
    if (it != node_hash.end()) return it->second;
    const Node &nd = g.node(n);
    uint64_t h = mix64(hash_str(CostEstimator::op_cost_key(nd, g)), (uint64_t)n);
    for (auto &o : nd.outputs) h = mix64(h, hash_str(o.shape.str()));
    for (auto &e : nd.inputs) h = mix64(h, ((uint64_t)e.src.node << 8) ^ (uint64_t)e.src.slot);
    auto at = attached.find(n);
    if (at != attached.end())
      for (NodeId a : at->second) h = mix64(h, mix64(hash_str(CostEstimator::op_cost_key(g.node(a), g)), (uint64_t)a));
    return node_hash[n] = h;
  }
  int add_leaf(int node) {
    Sub s;
    s.kind = SPTree::Leaf;
    s.node = node;
    s.leaves = {node};
    s.hash = mix64(0x1111, hash_of_node(node));
    s.work_ms = cost(node).total_ms();
    subs.push_back(std::move(s));
    return (int)subs.size() - 1;
  }
  int add_pair(SPTree::Kind kind, int li, int ri) {
    Sub s;
    s.kind = kind;
    s.left = li;
    s.right = ri;
    const Sub &l = subs[(size_t)li], &r = subs[(size_t)ri];
    s.leaves.resize(l.leaves.size() + r.leaves.size());
    std::merge(l.leaves.begin(), l.leaves.end(), r.leaves.begin(), r.leaves.end(), s.leaves.begin());
    s.hash = mix64(mix64(kind == SPTree::Series ? 0x2222 : 0x3333, l.hash), r.hash);
    s.work_ms = l.work_ms + r.work_ms;
    subs.push_back(std::move(s));
    return (int)subs.size() - 1;
  }
  // Binary grouping of the children [lo, hi) of an n-ary node.  The cut goes where the hash of the two neighbouring
  // children is smallest, so the shape of the grouping depends only on what the children are, never on how many there
  // are or where a rewrite happened: after a substitution every group that does not contain a rewritten operator is
  // the same sub-problem as before (same hash) and comes out of the cache.  Expected depth is logarithmic.
  int group(SPTree::Kind kind, const std::vector<int> &kids, size_t lo, size_t hi) {
    if (hi - lo == 1) return kids[lo];
    size_t cut = lo + 1;
    uint64_t best = ~0ull;
    for (size_t i = lo + 1; i < hi; ++i) {
      const uint64_t pr = mix64(subs[(size_t)kids[i - 1]].hash, subs[(size_t)kids[i]].hash);
      if (pr < best) { best = pr; cut = i; }
    }
    const int l = group(kind, kids, lo, cut), r = group(kind, kids, cut, hi);
    return add_pair(kind, l, r);
  }
  int annotate(const SPTree &t) {
    if (t.kind == SPTree::Leaf) return add_leaf(t.node);
    std::vector<int> kids;
    for (auto &c : t.children) kids.push_back(annotate(c));
    if (t.kind == SPTree::Parallel)  // branches in a canonical order
      std::sort(kids.begin(), kids.end(), [&](int a, int b) { return subs[(size_t)a].hash < subs[(size_t)b].hash; });
    return group(t.kind, kids, 0, kids.size());
  }
  static bool has(const std::vector<int> &sorted, int v) { return std::binary_search(sorted.begin(), sorted.end(), v); }

  // Cost of the tensors on edges a -> b.  Nothing moves when b's devices all hold what a produced (same device set, or a
  // subset of it); otherwise the pieces that travel are worked out from the two operators' shard mappings
  // (get_tensor_set_movement) where both have one, and priced as whole pieces otherwise.  Forward activation and
  // backward gradient both cross the edge.
  double movement(NodeId a, const MachineView &va, NodeId b, const MachineView &vb) {
    std::vector<int> da = view_devices(va, tasks(a), m), db = view_devices(vb, tasks(b), m);
    std::sort(da.begin(), da.end());
    std::sort(db.begin(), db.end());
    if (da == db) return 0.0;
    if (std::includes(da.begin(), da.end(), db.begin(), db.end())) return 0.0;
    std::string key = std::to_string(hash_of_node(a)) + va.str() + ">" + std::to_string(hash_of_node(b)) + vb.str();
    auto it = cache.movement.find(key);
    if (it != cache.movement.end()) return it->second;
    double c;
    try {
      c = 2.0 * tensor_set_movement_cost_ms(get_tensor_set_movement(g, a, va, b, vb, m), m, est);
    } catch (const std::exception &) {
      double bytes = 0;
      for (auto &e : g.node(b).inputs)
        if (e.src.node == a) bytes += (double)g.shape(e.src).piece_bytes();
      bool inter = (da.front() / m.num_gpus_per_node) != (db.front() / m.num_gpus_per_node);
      c = 2.0 * est.movement_cost_ms(bytes, inter);
    }
    return cache.movement[key] = c;
  }

  // Views a boundary layer is tried at inside `r`.  On one node of a switch-connected machine any two placements that
  // differ by a permutation of the devices cost the same, so it is enough to distinguish "at the start of the slice"
  // from "at the start of its second half" (the two sides a resource split can give to parallel branches); machines
  // with several nodes keep every aligned start, because crossing a node boundary changes the bandwidth.
  std::vector<MachineView> boundary_views(NodeId n, const Resources &r) {
    std::vector<MachineView> all = allowed_machine_views(tasks(n), r, m);
    if (m.num_nodes > 1 || all.size() <= 2) return all;
    int count = 1;
    for (int d : tasks(n)) count *= d;
    std::vector<MachineView> out;
    const int half = r.start + r.count / 2;
    for (auto &v : all) {
      const int start = v.start_node * m.num_gpus_per_node + v.start_device;
      if (start == r.start || (start == half && count <= r.count / 2)) out.push_back(v);
    }
    return out.empty() ? all : out;
  }

  Front solve(int si, Resources r, const std::map<NodeId, MachineView> &fixed) {
    const Sub &sub = subs[(size_t)si];
    struct { SPTree::Kind kind; int node; } t{sub.kind, sub.node};
    std::string key = std::to_string(sub.hash) + "@" + std::to_string(r.start) + "+" + std::to_string(r.count) + "/" + std::to_string(max_front);
    for (auto &kv : fixed)
      if (has(sub.leaves, kv.first)) key += ";" + std::to_string(kv.first) + kv.second.str();
    auto it = cache.table.find(key);
    if (it != cache.table.end()) {
      ++cache.hits;
      return it->second;
    }
    ++cache.misses;
    Front res;
    if (t.kind == SPTree::Leaf) {
      const OpCost &c = cost(t.node);
      auto fit = fixed.find(t.node);
      std::vector<MachineView> views;
      if (fit != fixed.end()) {
        // a fixed view must lie inside the resources of this subproblem
        auto devs = view_devices(fit->second, tasks(t.node), m);
        bool inside = true;
        for (int d : devs) if (d < r.start || d >= r.start + r.count) inside = false;
        if (inside) views.push_back(fit->second);
      } else views = allowed_machine_views(tasks(t.node), r, m);
      // on a uniform machine every allowed view costs the same: keep the first (lowest start) only
      if (!views.empty()) {
        MappingPoint p;
        p.runtime_ms = c.total_ms();
        p.memory_bytes = c.memory_bytes;
        p.views[t.node] = views.front();
        res.push_back(p);
      }
    } else if (t.kind == SPTree::Series) {
      const Sub &l = subs[(size_t)sub.left], &rt = subs[(size_t)sub.right];
      // boundary: producers in the left subtree with consumers in the right subtree
      std::vector<std::pair<NodeId, NodeId>> edges;
      for (int b : rt.leaves)
        for (auto &e : g.node(b).inputs)
          if (has(l.leaves, e.src.node)) edges.push_back({e.src.node, b});
      // The transfer cost across the split depends on the views of the boundary layers, so those views are
      // enumerated here and imposed on both sub-problems as constraints (get_optimal_machine_mapping.cc:162-210).
      std::vector<NodeId> boundary;
      for (auto &e : edges) {
        for (NodeId n : {e.first, e.second})
          if (!fixed.count(n) && std::find(boundary.begin(), boundary.end(), n) == boundary.end()) boundary.push_back(n);
      }
      std::vector<std::vector<MachineView>> options;
      size_t combos = 1;
      for (NodeId n : boundary) {
        options.push_back(boundary_views(n, r));
        if (options.back().empty()) { combos = 0; break; }
        combos *= options.back().size();
      }
      if (combos > 256) {  // very wide boundaries: the lowest-start view of each layer (counted, so a caller can tell)
        for (auto &o : options) o.resize(1);
        combos = 1;
        ++cache.truncated_boundaries;
      }
      for (size_t ci = 0; ci < combos; ++ci) {
        std::map<NodeId, MachineView> fx;
        // only constraints on leaves of this subtree matter below
        for (auto &kv : fixed)
          if (has(sub.leaves, kv.first)) fx.insert(kv);
        size_t rem = ci;
        for (size_t bi = 0; bi < boundary.size(); ++bi) {
          fx[boundary[bi]] = options[bi][rem % options[bi].size()];
          rem /= options[bi].size();
        }
        Front fl = solve(sub.left, r, fx), fr = solve(sub.right, r, fx);
        for (auto &a : fl)
          for (auto &b : fr) {
            MappingPoint p;
            double move = 0;
            for (auto &e : edges) move = std::max(move, movement(e.first, a.views.at(e.first), e.second, b.views.at(e.second)));
            p.runtime_ms = a.runtime_ms + b.runtime_ms + move;
            p.memory_bytes = a.memory_bytes + b.memory_bytes;
            p.views = a.views;
            p.views.insert(b.views.begin(), b.views.end());
            res.push_back(p);
          }
      }
    } else {
      // (a) run the branches one after the other on all resources
      Front fl = solve(sub.left, r, fixed), fr = solve(sub.right, r, fixed);
      for (auto &a : fl)
        for (auto &b : fr) {
          MappingPoint p;
          p.runtime_ms = a.runtime_ms + b.runtime_ms;
          p.memory_bytes = a.memory_bytes + b.memory_bytes;
          p.views = a.views;
          p.views.insert(b.views.begin(), b.views.end());
          res.push_back(p);
        }
      // (b) split the resources (power-of-two halves) and run the branches side by side; a branch without work (weights,
      // inputs, a residual connection) gains nothing from devices of its own
      if (r.count >= 2 && r.count % 2 == 0 && subs[(size_t)sub.left].work_ms > 0 && subs[(size_t)sub.right].work_ms > 0) {
        Resources r1{r.start, r.count / 2}, r2{r.start + r.count / 2, r.count / 2};
        for (int swap = 0; swap < 2; ++swap) {
          Front a_ = solve(sub.left, swap ? r2 : r1, fixed), b_ = solve(sub.right, swap ? r1 : r2, fixed);
          for (auto &a : a_)
            for (auto &b : b_) {
              MappingPoint p;
              p.runtime_ms = std::max(a.runtime_ms, b.runtime_ms);
              p.memory_bytes = std::max(a.memory_bytes, b.memory_bytes);
              p.views = a.views;
              p.views.insert(b.views.begin(), b.views.end());
              res.push_back(p);
            }
        }
      }
    }
    prune(res, max_front);
    cache.table[key] = res;
    return res;
  }
};
}  // namespace

MachineMappingResult get_optimal_machine_mapping(const Graph &pcg, const SPTree &binary_tree, const MachineSpec &m, const CostEstimator &est,
                                                 int max_front, MachineMappingCache *cache) {
  MachineMappingCache local;
  DP dp{pcg, m, est, std::max(1, max_front), cache ? *cache : local};
  const int root = dp.annotate(binary_tree);
  MachineMappingResult r;
  r.front = dp.solve(root, Resources{0, m.num_devices()}, {});
  return r;
}

Graph mapped_pcg_from_pcg_and_mapping(const Graph &pcg, const std::map<NodeId, MachineView> &mapping) {
  Graph g = pcg;
  for (auto &kv : mapping)
    if (g.has_node(kv.first)) g.node(kv.first).view = kv.second;
  return g;
}

// Weights and inputs, each with the parallel operators that follow it in a chain, as {chain nodes} -> consumer.
// A chain whose end feeds several operators belongs to the first of them in topological order.
static std::map<NodeId, std::vector<NodeId>> source_chains(const Graph &g) {
  std::map<NodeId, int> topo_pos;
  int i = 0;
  for (NodeId n : g.topological_order()) topo_pos[n] = i++;
  std::map<NodeId, std::vector<NodeId>> by_consumer;
  for (auto &kv : g.nodes()) {
    if (kv.second.type != OpType::WEIGHT && kv.second.type != OpType::INPUT) continue;
    std::vector<NodeId> chain{kv.first};
    NodeId cur = kv.first;
    while (true) {
      auto succ = g.successors(cur);
      if (succ.size() == 1 && is_parallel_op(g.node(succ[0]).type) && g.predecessors(succ[0]).size() == 1) {
        cur = succ[0];
        chain.push_back(cur);
      } else break;
    }
    auto succ = g.successors(cur);
    if (succ.empty()) continue;  // an unused source stays a leaf of its own
    NodeId consumer = succ[0];
    for (NodeId c : succ)
      if (topo_pos[c] < topo_pos[consumer]) consumer = c;
    auto &v = by_consumer[consumer];
    v.insert(v.end(), chain.begin(), chain.end());
  }
  // a consumer that is itself part of a chain cannot happen (chains end where a non-parallel operator or a join begins)
  return by_consumer;
}

SearchResult evaluate_pcg(const Graph &pcg, const MachineSpec &m, const CostEstimator &est, MachineMappingCache *cache) {
  SearchResult r;
  r.pcg = pcg;
  // The tree the DP works on holds the computation only.  Sources (weights, inputs and the parallel operators chained to
  // them) are placed with their consumers: as branches of the SP tree they would nest the whole graph one level deeper
  // per weight, and a rewrite anywhere would change every enclosing sub-problem.
  std::map<NodeId, std::vector<NodeId>> attached = source_chains(pcg);
  std::set<NodeId> riding;
  for (auto &kv : attached) riding.insert(kv.second.begin(), kv.second.end());
  DiGraph d;
  for (auto &kv : pcg.nodes()) {
    if (riding.count(kv.first)) continue;
    d.add_node(kv.first);
    for (auto &e : kv.second.inputs)
      if (!riding.count(e.src.node)) d.add_edge(e.src.node, kv.first);
  }
  SPTree tree;
  if (auto t = get_series_parallel_decomposition(d)) tree = normalize_sp(*t);
  else tree = normalize_sp(escribano_sp_ization(d));
  MachineMappingCache local;
  DP dp{pcg, m, est, 1, cache ? *cache : local};
  dp.attached = attached;
  const int root = dp.annotate(tree);
  Front front = dp.solve(root, Resources{0, m.num_devices()}, {});
  if (front.empty()) {
    r.runtime_ms = std::numeric_limits<double>::infinity();
    return r;
  }
  const MappingPoint &best = front.front();
  r.mapping = best.views;
  r.runtime_ms = best.runtime_ms;
  r.memory_bytes = best.memory_bytes;
  // sources sit on the devices of their consumer: the first allowed view inside the consumer's device range
  for (auto &kv : attached) {
    auto cv = r.mapping.find(kv.first);
    if (cv == r.mapping.end()) continue;
    std::vector<int> devs = view_devices(cv->second, operator_task_space(pcg.node(kv.first), pcg), m);
    const int lo = *std::min_element(devs.begin(), devs.end()), hi = *std::max_element(devs.begin(), devs.end());
    for (NodeId a : kv.second) {
      const std::vector<int> ts = operator_task_space(pcg.node(a), pcg);
      auto vs = allowed_machine_views(ts, Resources{lo, hi - lo + 1}, m);
      if (vs.empty()) vs = allowed_machine_views(ts, Resources{0, m.num_devices()}, m);
      if (!vs.empty()) r.mapping[a] = vs.front();
    }
  }
  return r;
}

static bool within_degree(const Graph &g, int max_total_degree) {
  if (max_total_degree <= 0) return true;
  for (auto &kv : g.nodes())
    for (auto &o : kv.second.outputs)
      if (o.shape.total_degree() > max_total_degree) return false;
  return true;
}
Graph apply_rules_exhaustively(const Graph &g0, const std::vector<Substitution> &rules, int max_applications, int max_total_degree) {
  Graph g = g0;
  int applied = 0;
  bool progress = true;
  while (progress && applied < max_applications) {
    progress = false;
    for (auto &rule : rules) {
      bool again = true;
      while (again && applied < max_applications) {
        again = false;
        for (auto &mt : find_pattern_matches(rule.pattern, g)) {
          auto ng = apply_substitution(g, rule, mt);
          if (ng && within_degree(*ng, max_total_degree)) {
            g = *ng;
            ++applied;
            again = true;
            progress = true;
            break;  // matches are stale after an application
          }
        }
      }
    }
  }
  return g;
}

SearchResult unity_search(const Graph &start, const MachineSpec &m, const CostEstimator &est, const std::vector<Substitution> &rules,
                          const UnityConfig &cfg) {
  auto t0 = std::chrono::steady_clock::now();
  auto elapsed = [&] { return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count(); };
  struct State {
    double cost;
    Graph g;
    bool exempt;  // produced by a compound move: expanded even when outside the alpha band
    bool operator<(const State &o) const { return cost > o.cost; }  // min-heap
  };
  std::priority_queue<State> queue;
  std::set<std::string> seen;
  MachineMappingCache cache;  // shared by every candidate: only the sub-problems around a rewritten region are solved anew
  SearchResult best = evaluate_pcg(start, m, est, &cache);
  queue.push({best.runtime_ms, start, true});
  seen.insert(start.signature());
  long long evaluated = 1, generated = 0;
  int iterations = 0;
  for (; iterations < cfg.budget && !queue.empty(); ++iterations) {
    if (elapsed() > cfg.time_limit_s) break;
    State cur = queue.top();
    queue.pop();
    if (!cur.exempt && cur.cost > cfg.alpha * best.runtime_ms) continue;
    int candidates = 0;
    auto consider = [&](const Graph &ng, bool keep_anyway) {
      ++generated;
      if ((int)ng.num_nodes() > cfg.max_num_ops) return;
      if (!seen.insert(ng.signature()).second) return;
      ++candidates;
      SearchResult r = evaluate_pcg(ng, m, est, &cache);
      ++evaluated;
      if (r.runtime_ms < best.runtime_ms) best = r;
      if (keep_anyway ? std::isfinite(r.runtime_ms) : r.runtime_ms <= cfg.alpha * best.runtime_ms) queue.push({r.runtime_ms, ng, keep_anyway});
    };
    auto cleanup = [&](Graph g) {
      if (!cfg.cancel_after_compound || cfg.cleanup_rules.empty()) return g;
      std::vector<Substitution> cl;
      for (int ci : cfg.cleanup_rules) cl.push_back(rules.at((size_t)ci));
      return apply_rules_exhaustively(g, cl, 100000, m.num_devices());
    };
    // Rule families (for instance every sample-dimension partition rule of one degree): all of a family's rules applied
    // wherever they match, as one move.
    for (auto &fam : cfg.families) {
      if (elapsed() > cfg.time_limit_s) break;
      std::vector<Substitution> rs;
      for (int ri : fam) rs.push_back(rules.at((size_t)ri));
      consider(cleanup(apply_rules_exhaustively(cur.g, rs, 100000, m.num_devices())), true);
    }
    for (auto &rule : rules) {
      if (candidates >= cfg.max_candidates_per_step || elapsed() > cfg.time_limit_s) break;
      auto matches = find_pattern_matches(rule.pattern, cur.g);
      if (matches.empty()) continue;
      // Compound move: the rule applied at every place it matches.  A data- or tensor-parallel plan differs from the
      // serial graph by one rule application per operator, and each of them alone makes the graph slower (a Repartition
      // and a Combine around one operator) until its neighbours follow and the pairs cancel; as one move the whole step
      // is a single candidate, so the search can cross that ridge.  Such a candidate stays in the queue even when it is
      // outside the alpha band: its value shows only after the cancellation rules have been applied to it.
      if (cfg.compound_moves && matches.size() > 1) {
        std::vector<Substitution> one{rule};
        consider(cleanup(apply_rules_exhaustively(cur.g, one, 100000, m.num_devices())), true);
      }
      if (cfg.single_moves)
        for (auto &mt : matches) {
          if (candidates >= cfg.max_candidates_per_step || elapsed() > cfg.time_limit_s) break;
          auto ng = apply_substitution(cur.g, rule, mt);
          if (!ng) continue;
          consider(*ng, false);
        }
    }
  }
  best.stats = Json::object();
  best.stats["iterations"] = iterations;
  best.stats["evaluated"] = evaluated;
  best.stats["generated"] = generated;
  best.stats["seconds"] = elapsed();
  best.stats["cost_queries"] = est.num_queries;
  best.stats["cache_hits"] = cache.hits;
  best.stats["cache_misses"] = cache.misses;
  best.stats["truncated_boundaries"] = cache.truncated_boundaries;
  return best;
}

// ---------------------------------------------------------------- simulator
std::vector<TaskProfile> simulate_task_graph_execution(int n, const std::vector<std::pair<int, int>> &edges, const std::vector<double> &cost,
                                                       const TaskConstraint &allowed) {
  if ((int)cost.size() != n) throw Error("simulate_task_graph_execution: one cost per task is needed");
  std::vector<std::vector<int>> succ(n);
  std::vector<int> missing(n, 0);
  for (auto &e : edges) {
    if (e.first < 0 || e.first >= n || e.second < 0 || e.second >= n) throw Error("simulate_task_graph_execution: edge endpoint out of range");
    succ[e.first].push_back(e.second);
    ++missing[e.second];
  }
  std::set<int> ready, in_progress, finished;
  for (int t = 0; t < n; ++t)
    if (missing[t] == 0) ready.insert(t);
  std::vector<TaskProfile> trace(n, TaskProfile{-1, 0, 0});
  std::multimap<double, int> running;   // end time -> task
  double now = 0;
  while ((int)finished.size() < n) {
    // offer the ready tasks in index order; a start changes what the constraint sees, so go round until nothing starts
    for (bool started = true; started;) {
      started = false;
      for (int t : std::vector<int>(ready.begin(), ready.end())) {
        if (!allowed(t, in_progress, finished)) continue;
        ready.erase(t);
        in_progress.insert(t);
        trace[t] = TaskProfile{t, now, now + cost[t]};
        running.emplace(now + cost[t], t);
        started = true;
      }
    }
    if (running.empty()) throw Error("simulate_task_graph_execution: " + std::to_string(n - (int)finished.size()) + " tasks can never start (cycle, or the constraint refuses them with nothing running)");
    now = running.begin()->first;
    while (!running.empty() && running.begin()->first == now) {
      const int t = running.begin()->second;
      running.erase(running.begin());
      in_progress.erase(t);
      finished.insert(t);
      for (int s2 : succ[t])
        if (--missing[s2] == 0) ready.insert(s2);
    }
  }
  return trace;
}

double simulate_task_graph(const Graph &g, const MachineSpec &m, const CostEstimator &est, bool include_backward) {
  auto devices_of = [&](NodeId n) {
    const Node &nd = g.node(n);
    auto ts = operator_task_space(nd, g);
    MachineView v = nd.view ? *nd.view : MachineView{};
    if (!nd.view) {
      auto vs = allowed_machine_views(ts, Resources{0, m.num_devices()}, m);
      if (!vs.empty()) v = vs.front();
    }
    auto d = view_devices(v, ts, m);
    std::sort(d.begin(), d.end());
    return d;
  };
  auto order = g.topological_order();
  std::map<NodeId, std::vector<int>> devs;
  for (NodeId n : order) devs[n] = devices_of(n);
  auto comm_ms = [&](NodeId a, NodeId b) {   // movement of a's outputs that b consumes, 0 when b's devices already hold them
    const auto &da = devs[a], &db = devs[b];
    if (da == db || std::includes(da.begin(), da.end(), db.begin(), db.end())) return 0.0;
    double bytes = 0;
    for (auto &e : g.node(b).inputs) if (e.src.node == a) bytes += (double)g.shape(e.src).piece_bytes();
    return est.movement_cost_ms(bytes, da.front() / m.num_gpus_per_node != db.front() / m.num_gpus_per_node);
  };
  // tasks: forward operator tasks in topological order, then (optionally) backward operator tasks, then movement tasks
  std::vector<double> cost;
  std::vector<std::vector<int>> task_devs;   // empty = unconstrained (movement)
  std::vector<std::pair<int, int>> edges;
  std::map<NodeId, int> fwd, bwd;
  for (NodeId n : order) {
    fwd[n] = (int)cost.size();
    cost.push_back(est.op_cost(g.node(n), g).fwd_ms);
    task_devs.push_back(devs[n]);
  }
  if (include_backward)
    for (NodeId n : order) {
      bwd[n] = (int)cost.size();
      cost.push_back(est.op_cost(g.node(n), g).bwd_ms);
      task_devs.push_back(devs[n]);
    }
  auto link = [&](int from, int to, double ms) {
    if (ms <= 0) { edges.push_back({from, to}); return; }
    const int c = (int)cost.size();
    cost.push_back(ms);
    task_devs.push_back({});
    edges.push_back({from, c});
    edges.push_back({c, to});
  };
  std::vector<int> sinks;
  for (NodeId n : order) {
    std::set<NodeId> producers;
    for (auto &e : g.node(n).inputs) producers.insert(e.src.node);
    for (NodeId a : producers) {
      const double ms = comm_ms(a, n);
      link(fwd[a], fwd[n], ms);
      if (include_backward) link(bwd[n], bwd[a], ms);   // the gradient goes back over the same pieces
    }
    if (g.successors(n).empty()) sinks.push_back(fwd[n]);
  }
  if (include_backward)   // backward starts when the whole forward pass has finished (the loss needs every output)
    for (NodeId n : order)
      if (g.successors(n).empty())
        for (int s2 : sinks) edges.push_back({s2, bwd[n]});
  auto allowed = [&](int t, const std::set<int> &in_progress, const std::set<int> &) {
    if (task_devs[t].empty()) return true;
    for (int r : in_progress)
      for (int d : task_devs[r])
        if (std::binary_search(task_devs[t].begin(), task_devs[t].end(), d)) return false;
    return true;
  };
  double makespan = 0;
  for (auto &tp : simulate_task_graph_execution((int)cost.size(), edges, cost, allowed)) makespan = std::max(makespan, tp.end);
  return makespan;
}

// ---------------------------------------------------------------- MCMC
SearchResult mcmc_search(const Graph &start, const MachineSpec &m, const CostEstimator &est, const std::vector<Substitution> &rules,
                         const MCMCConfig &cfg) {
  std::mt19937 rng(cfg.seed);
  std::uniform_real_distribution<double> uni(0.0, 1.0);
  auto random_views = [&](const Graph &g) {
    std::map<NodeId, MachineView> mv;
    for (auto &kv : g.nodes()) {
      auto vs = allowed_machine_views(operator_task_space(kv.second, g), Resources{0, m.num_devices()}, m);
      if (vs.empty()) continue;
      mv[kv.first] = vs[rng() % vs.size()];
    }
    return mv;
  };
  auto score = [&](const Graph &g, const std::map<NodeId, MachineView> &mv) {
    return simulate_task_graph(mapped_pcg_from_pcg_and_mapping(g, mv), m, est, true);
  };
  struct State {
    Graph g;
    std::map<NodeId, MachineView> views;
  };
  State init{start, random_views(start)};
  const double start_cost = score(init.g, init.views);
  int substitutions = 0;
  // relative: the temperature is a fraction of the starting cost, so that "a candidate 1 % worse" means the same
  // whether a step takes 3 ms or 300 ms; absolute: exp(-delta / temperature) with delta in ms
  const double temperature = cfg.relative_temperature ? cfg.temperature * std::max(start_cost, 1e-9) : cfg.temperature;
  auto propose = [&](const State &cur, std::mt19937 &) -> std::optional<State> {
    State cand = cur;
    bool changed = false;
    if (uni(rng) < cfg.substitution_frequency && !rules.empty()) {
      // a random rule at a random match; new layers take a random allowed view
      for (int attempt = 0; attempt < 8 && !changed; ++attempt) {
        const Substitution &rule = rules[rng() % rules.size()];
        auto ms = find_pattern_matches(rule.pattern, cur.g);
        if (ms.empty()) continue;
        auto ng = apply_substitution(cur.g, rule, ms[rng() % ms.size()]);
        if (!ng) continue;
        cand.g = *ng;
        for (auto &kv : cand.g.nodes())
          if (!cand.views.count(kv.first)) {
            auto vs = allowed_machine_views(operator_task_space(kv.second, cand.g), Resources{0, m.num_devices()}, m);
            if (!vs.empty()) cand.views[kv.first] = vs[rng() % vs.size()];
          }
        for (auto itv = cand.views.begin(); itv != cand.views.end();)
          itv = cand.g.has_node(itv->first) ? std::next(itv) : cand.views.erase(itv);
        changed = true;
        ++substitutions;
      }
    }
    if (!changed) {
      // mutate the view of one layer
      auto ids = cand.g.node_ids();
      NodeId n = ids[rng() % ids.size()];
      auto vs = allowed_machine_views(operator_task_space(cand.g.node(n), cand.g), Resources{0, m.num_devices()}, m);
      if (vs.empty()) return std::nullopt;
      cand.views[n] = vs[rng() % vs.size()];
    }
    return cand;
  };
  int accepted = 0;
  double best_cost = start_cost;
  State found = run_mcmc(init, propose, [&](const State &st) { return score(st.g, st.views); }, temperature, cfg.num_iterations, rng, &accepted,
                         &best_cost);
  SearchResult best;
  best.pcg = found.g;
  best.mapping = found.views;
  best.runtime_ms = best_cost;
  best.stats = Json::object();
  best.stats["iterations"] = cfg.num_iterations;
  best.stats["accepted"] = accepted;
  best.stats["substitutions"] = substitutions;
  return best;
}

// ---------------------------------------------------------------- python bindings
static py::dict result_to_py(const SearchResult &r) {
  py::dict d;
  d["pcg"] = r.pcg;
  d["mapped_pcg"] = mapped_pcg_from_pcg_and_mapping(r.pcg, r.mapping);
  py::dict mv;
  for (auto &kv : r.mapping) mv[py::int_(kv.first)] = json_to_py(kv.second.to_json());
  d["mapping"] = mv;
  d["runtime_ms"] = r.runtime_ms;
  d["memory_bytes"] = r.memory_bytes;
  d["stats"] = json_to_py(r.stats);
  return d;
}

void bind_search(py::module &m) {
  py::class_<CostEstimator>(m, "CostEstimator")
      .def(py::init([](const MachineSpec &ms, py::object params) {
             CostParams p = params.is_none() ? CostParams() : CostParams::from_json(json_from_py(params));
             p.nvlink_gbs = params.is_none() ? ms.intra_node_bandwidth : p.nvlink_gbs;
             return CostEstimator(p, ms);
           }),
           py::arg("machine"), py::arg("params") = py::none())
      .def("params", [](const CostEstimator &e) { return json_to_py(e.params.to_json()); })
      .def("op_cost", [](const CostEstimator &e, const Graph &g, NodeId n) {
        OpCost c = e.op_cost(g.node(n), g);
        py::dict d;
        d["fwd_ms"] = c.fwd_ms; d["bwd_ms"] = c.bwd_ms; d["memory_bytes"] = c.memory_bytes;
        return d;
      })
      .def("op_cost_key", [](const CostEstimator &, const Graph &g, NodeId n) { return CostEstimator::op_cost_key(g.node(n), g); })
      .def("set_measured", [](CostEstimator &e, const std::string &key, double fwd, double bwd, double mem) { e.measured[key] = OpCost{fwd, bwd, mem}; })
      .def("num_measured", [](const CostEstimator &e) { return e.measured.size(); })
      .def("movement_cost_ms", &CostEstimator::movement_cost_ms)
      .def_readonly("num_queries", &CostEstimator::num_queries);
  m.def("allowed_machine_views", [](std::vector<int> task, int start, int count, const MachineSpec &ms, bool strided) {
    py::list l;
    for (auto &v : allowed_machine_views(task, Resources{start, count}, ms, strided)) l.append(json_to_py(v.to_json()));
    return l;
  }, py::arg("task_degrees"), py::arg("start"), py::arg("count"), py::arg("machine"), py::arg("strided") = false);
  m.def("get_tensor_set_movement", [](const Graph &g, NodeId src, py::object vs, NodeId dst, py::object vd, const MachineSpec &ms) {
    py::list out;
    for (auto &e : get_tensor_set_movement(g, src, MachineView::from_json(json_from_py(vs)), dst, MachineView::from_json(json_from_py(vd)), ms)) {
      py::dict d;
      d["src"] = e.src_device;
      d["dst"] = e.dst_device;
      d["bytes"] = e.bytes;
      out.append(d);
    }
    return out;
  });
  m.def("tensor_set_movement_cost_ms", [](const Graph &g, NodeId src, py::object vs, NodeId dst, py::object vd, const MachineSpec &ms,
                                          const CostEstimator &est) {
    return tensor_set_movement_cost_ms(get_tensor_set_movement(g, src, MachineView::from_json(json_from_py(vs)), dst,
                                                               MachineView::from_json(json_from_py(vd)), ms), ms, est);
  });
  m.def("reference_machine_coordinate", [](py::object view, std::vector<int> task, std::vector<int> coord) {
    return reference_machine_coordinate(MachineView::from_json(json_from_py(view)), task, coord);
  }, py::arg("view"), py::arg("task_degrees"), py::arg("coord"), "(node, device) of a task under the reference's relative-stride view semantics");
  m.def("reference_allowed_machine_views", [](std::vector<int> task, int num_nodes, int gpus_per_node) {
    py::list l;
    for (auto &v : reference_allowed_machine_views(task, num_nodes, gpus_per_node)) l.append(json_to_py(v.to_json()));
    return l;
  }, py::arg("task_degrees"), py::arg("num_nodes"), py::arg("gpus_per_node"));
  m.def("absolute_view_from_reference", [](py::object view, std::vector<int> task) {
    return json_to_py(absolute_view_from_reference(MachineView::from_json(json_from_py(view)), task).to_json());
  });
  m.def("view_devices", [](py::object view, std::vector<int> task, const MachineSpec &ms) {
    return view_devices(MachineView::from_json(json_from_py(view)), task, ms);
  });
  m.def("get_graph_sp_decomposition", [](const Graph &g) {
    bool exact = true;
    SPTree t = get_graph_sp_decomposition(g, &exact);
    return py::make_tuple(sp_to_py(t), exact);
  });
  m.def("get_optimal_machine_mapping", [](const Graph &g, py::object tree, const MachineSpec &ms, const CostEstimator &est, int max_front) {
    SPTree t = tree.is_none() ? balanced_binary_sp_tree(get_graph_sp_decomposition(g)) : sp_from_py(tree);
    auto r = get_optimal_machine_mapping(g, t, ms, est, max_front);
    py::list pts;
    for (auto &p : r.front) {
      py::dict d;
      d["runtime_ms"] = p.runtime_ms;
      d["memory_bytes"] = p.memory_bytes;
      py::dict mv;
      for (auto &kv : p.views) mv[py::int_(kv.first)] = json_to_py(kv.second.to_json());
      d["views"] = mv;
      pts.append(d);
    }
    return pts;
  }, py::arg("pcg"), py::arg("tree") = py::none(), py::arg("machine") = MachineSpec(), py::arg("estimator") = CostEstimator(),
        py::arg("max_front") = 1);
  m.def("evaluate_pcg", [](const Graph &g, const MachineSpec &ms, const CostEstimator &est) { return result_to_py(evaluate_pcg(g, ms, est)); });
  m.def("apply_rules_exhaustively", [](const Graph &g, std::vector<Substitution> rules, int max_app, int max_deg) {
    return apply_rules_exhaustively(g, rules, max_app, max_deg);
  }, py::arg("graph"), py::arg("rules"), py::arg("max_applications") = 100000, py::arg("max_total_degree") = 0);
  m.def("unity_search", [](const Graph &g, const MachineSpec &ms, const CostEstimator &est, std::vector<Substitution> rules, double alpha,
                           int budget, int max_num_ops, double time_limit_s, bool compound_moves, bool single_moves,
                           std::vector<std::vector<int>> families) {
    UnityConfig c;
    c.families = families;
    c.alpha = alpha; c.budget = budget; c.max_num_ops = max_num_ops; c.time_limit_s = time_limit_s;
    c.compound_moves = compound_moves; c.single_moves = single_moves;
    // rules that only remove parallel operators (a Combine meeting a Repartition and the like) tidy up after a compound move
    for (size_t i = 0; i < rules.size(); ++i)
      if (rules[i].name.rfind("cancel_", 0) == 0) c.cleanup_rules.push_back((int)i);
    py::gil_scoped_release rel;
    SearchResult r = unity_search(g, ms, est, rules, c);
    py::gil_scoped_acquire acq;
    return result_to_py(r);
  }, py::arg("pcg"), py::arg("machine"), py::arg("estimator"), py::arg("rules"), py::arg("alpha") = 1.05, py::arg("budget") = 10,
        py::arg("max_num_ops") = 100000, py::arg("time_limit_s") = 120.0, py::arg("compound_moves") = true, py::arg("single_moves") = true,
        py::arg("families") = std::vector<std::vector<int>>());
  m.def("mcmc_search", [](const Graph &g, const MachineSpec &ms, const CostEstimator &est, std::vector<Substitution> rules, double temperature,
                          int iters, double sub_freq, unsigned seed, bool relative) {
    MCMCConfig c;
    c.temperature = temperature; c.num_iterations = iters; c.substitution_frequency = sub_freq; c.seed = seed;
    c.relative_temperature = relative;
    return result_to_py(mcmc_search(g, ms, est, rules, c));
  }, py::arg("pcg"), py::arg("machine"), py::arg("estimator"), py::arg("rules"), py::arg("temperature") = 1.0, py::arg("num_iterations") = 100,
        py::arg("substitution_frequency") = 0.2, py::arg("seed") = 0, py::arg("relative_temperature") = false);
  m.def("run_mcmc",
        [](py::object start, std::function<py::object(py::object, double)> sampler, std::function<double(py::object)> cost, double temperature,
           int num_iterations, unsigned seed) {
          std::mt19937 rng(seed);
          std::uniform_real_distribution<double> uni(0.0, 1.0);
          int accepted = 0;
          double best_cost = 0;
          auto propose = [&](const py::object &st, std::mt19937 &r) -> std::optional<py::object> {
            py::object o = sampler(st, uni(r));
            if (o.is_none()) return std::nullopt;
            return o;
          };
          py::object best = run_mcmc(start, propose, cost, temperature, num_iterations, rng, &accepted, &best_cost);
          return py::make_tuple(best, best_cost, accepted);
        },
        py::arg("start"), py::arg("sampler"), py::arg("cost"), py::arg("temperature") = 1.0, py::arg("num_iterations") = 100, py::arg("seed") = 0,
        "Metropolis search over Python states: sampler(state, u) -> state or None (u uniform in [0, 1) from the seeded generator), "
        "cost(state) -> float; returns (best state, its cost, proposals accepted)");
  m.def("simulate_task_graph_execution",
        [](int n, const std::vector<std::pair<int, int>> &edges, const std::vector<double> &cost, const TaskConstraint &allowed) {
          std::vector<std::tuple<int, double, double>> out;
          for (auto &tp : simulate_task_graph_execution(n, edges, cost, allowed)) out.emplace_back(tp.task, tp.start, tp.end);
          return out;
        },
        py::arg("num_tasks"), py::arg("edges"), py::arg("cost"), py::arg("allowed"),
        "event-driven execution of a task graph; allowed(task, in_progress, finished) -> bool; returns [(task, start, end)]");
  m.def("simulate_task_graph", &simulate_task_graph, py::arg("mapped_pcg"), py::arg("machine"), py::arg("estimator"),
        py::arg("include_backward") = false);
  m.def("mapped_pcg_from_pcg_and_mapping", [](const Graph &g, py::dict mapping) {
    std::map<NodeId, MachineView> mv;
    for (auto kv : mapping) mv[kv.first.cast<int>()] = MachineView::from_json(json_from_py(kv.second));
    return mapped_pcg_from_pcg_and_mapping(g, mv);
  });
}

}  // namespace ff
