// bindings.cc -- the pybind11 module `_ffcore`: Python surface of the C++ compiler core.
#include <pybind11/functional.h>

#include "builder.h"
#include "models.h"
#include "pyjson.h"

namespace ff {
void bind_substitutions(py::module &m);
void bind_search(py::module &m);
void bind_lowering(py::module &m);
void bind_utils(py::module &m);
void bind_dataflow(py::module &m);
void bind_containers(py::module &m);
}  // namespace ff

using namespace ff;

static py::dict node_to_py(NodeId id, const Node &n) {
  py::dict d;
  d["id"] = id;
  d["type"] = to_string(n.type);
  d["attrs"] = json_to_py(n.attrs);
  d["name"] = n.name;
  py::list ins, outs;
  for (auto &e : n.inputs) ins.append(py::make_tuple(to_string(e.dst_slot), value_to_py(e.src)));
  for (auto &o : n.outputs) outs.append(py::make_tuple(to_string(o.slot), o.shape, o.create_grad));
  d["inputs"] = ins;
  d["outputs"] = outs;
  d["view"] = n.view ? json_to_py(n.view->to_json()) : py::none();
  return d;
}

static SlotShapes slot_shapes_from_py(const py::handle &o) {
  SlotShapes r;
  for (auto item : o) {
    auto t = item.cast<py::tuple>();
    r.push_back({slot_from_string(t[0].cast<std::string>()), t[1].cast<PShape>()});
  }
  return r;
}
static py::list slot_shapes_to_py(const SlotShapes &s) {
  py::list l;
  for (auto &p : s) l.append(py::make_tuple(to_string(p.first), p.second));
  return l;
}

template <typename F>
static auto vfn(F f) {
  return f;
}

PYBIND11_MODULE(_ffcore, m) {
  m.doc() = "C++ compiler core: IR, shape inference, builders, model zoo, graph algorithms, substitutions, search";
  py::register_exception<ff::Error>(m, "CoreError");

  py::class_<PShape>(m, "ParallelTensorShape")
      .def(py::init([](std::vector<int64_t> sizes, const std::string &dtype, std::vector<int> degrees, int sum, int copy) {
             PShape s = PShape::make(sizes, datatype_from_string(dtype));
             if (!degrees.empty()) {
               if (degrees.size() != sizes.size()) throw Error("degrees rank mismatch");
               for (size_t i = 0; i < sizes.size(); ++i) s.dims[i].degree = degrees[i];
             }
             s.sum_degree = sum;
             s.discard_copy_degree = copy;
             return s;
           }),
           py::arg("sizes"), py::arg("dtype") = "FLOAT", py::arg("degrees") = std::vector<int>{}, py::arg("sum_degree") = 1,
           py::arg("discard_copy_degree") = 1)
      .def_property_readonly("sizes", &PShape::sizes)
      .def_property_readonly("degrees", &PShape::degrees)
      .def_property_readonly("piece_sizes", &PShape::piece_sizes)
      .def_readonly("sum_degree", &PShape::sum_degree)
      .def_readonly("discard_copy_degree", &PShape::discard_copy_degree)
      .def_property_readonly("dtype", [](const PShape &s) { return to_string(s.dtype); })
      .def_property_readonly("num_elements", &PShape::num_elements)
      .def_property_readonly("piece_bytes", &PShape::piece_bytes)
      .def_property_readonly("total_degree", &PShape::total_degree)
      .def("reduced", &PShape::reduced)
      .def("to_json", [](const PShape &s, bool parallel) { return json_to_py(parallel ? s.to_json_parallel() : s.to_json_plain()); },
           py::arg("parallel") = true)
      .def_static("from_json", [](py::object o) { return PShape::from_json(json_from_py(o)); })
      .def("__eq__", [](const PShape &a, const PShape &b) { return a == b; })
      .def("__repr__", &PShape::str);

  py::class_<MachineSpec>(m, "MachineSpecification")
      .def(py::init([](int nodes, int gpus, int cpus, double inter_bw, double intra_bw) {
             MachineSpec s;
             s.num_nodes = nodes; s.num_gpus_per_node = gpus; s.num_cpus_per_node = cpus;
             s.inter_node_bandwidth = inter_bw; s.intra_node_bandwidth = intra_bw;
             return s;
           }),
           py::arg("num_nodes") = 1, py::arg("num_gpus_per_node") = 1, py::arg("num_cpus_per_node") = 1,
           py::arg("inter_node_bandwidth") = 25.0, py::arg("intra_node_bandwidth") = 770.0)
      .def_readwrite("view_enumeration", &MachineSpec::view_enumeration)
      .def_readwrite("num_nodes", &MachineSpec::num_nodes)
      .def_readwrite("num_gpus_per_node", &MachineSpec::num_gpus_per_node)
      .def_readwrite("num_cpus_per_node", &MachineSpec::num_cpus_per_node)
      .def_readwrite("inter_node_bandwidth", &MachineSpec::inter_node_bandwidth)
      .def_readwrite("intra_node_bandwidth", &MachineSpec::intra_node_bandwidth)
      .def_property_readonly("num_devices", &MachineSpec::num_devices)
      .def("to_json", [](const MachineSpec &s) { return json_to_py(s.to_json()); })
      .def_static("from_json", [](py::object o) { return MachineSpec::from_json(json_from_py(o)); });

  py::class_<Graph>(m, "Graph")
      .def(py::init<>())
      .def("add_node",
           [](Graph &g, const std::string &type, py::object attrs, const std::string &name, py::object inputs, py::object outputs) {
             std::vector<InEdge> ins;
             for (auto item : inputs) {
               auto t = item.cast<py::tuple>();
               ins.push_back({slot_from_string(t[0].cast<std::string>()), value_from_py(t[1])});
             }
             std::vector<OutValue> outs;
             for (auto item : outputs) {
               auto t = item.cast<py::tuple>();
               outs.push_back({slot_from_string(t[0].cast<std::string>()), t[1].cast<PShape>(), t.size() > 2 ? t[2].cast<bool>() : true});
             }
             return g.add_node(optype_from_string(type), json_from_py(attrs), name, ins, outs);
           },
           py::arg("type"), py::arg("attrs"), py::arg("name") = "", py::arg("inputs") = py::list(), py::arg("outputs") = py::list())
      .def("remove_node", &Graph::remove_node)
      .def("node", [](const Graph &g, NodeId n) { return node_to_py(n, g.node(n)); })
      .def("node_type", [](const Graph &g, NodeId n) { return to_string(g.node(n).type); })
      .def("node_ids", &Graph::node_ids)
      .def("nodes", [](const Graph &g) {
        py::list l;
        for (auto &kv : g.nodes()) l.append(node_to_py(kv.first, kv.second));
        return l;
      })
      .def("__len__", &Graph::num_nodes)
      .def("topological_order", &Graph::topological_order)
      .def("shape", [](const Graph &g, py::object v) { return g.shape(value_from_py(v)); })
      .def("consumers", [](const Graph &g, py::object v) {
        py::list l;
        for (auto &c : g.consumers(value_from_py(v))) l.append(py::make_tuple(c.first, to_string(c.second)));
        return l;
      })
      .def("successors", &Graph::successors)
      .def("predecessors", &Graph::predecessors)
      .def("sink_values", [](const Graph &g) {
        py::list l;
        for (auto &v : g.sink_values()) l.append(value_to_py(v));
        return l;
      })
      .def("set_view", [](Graph &g, NodeId n, py::object v) {
        if (v.is_none()) g.node(n).view.reset();
        else g.node(n).view = MachineView::from_json(json_from_py(v));
      })
      .def("is_mapped", &Graph::is_mapped)
      .def("signature", &Graph::signature)
      // graph queries of the reference's computation_graph.h / parallel_computation_graph.h
      .def("get_layer_by_name", [](const Graph &g, const std::string &name) {
        std::vector<NodeId> found;
        for (auto &kv : g.nodes())
          if (kv.second.name == name) found.push_back(kv.first);
        if (found.size() != 1) throw Error("get_layer_by_name: " + std::to_string(found.size()) + " layers are named \"" + name + "\"");
        return found[0];
      })
      .def("get_incoming_tensors", [](const Graph &g, NodeId n) {
        py::list l;
        for (auto &e : g.node(n).inputs) l.append(py::make_tuple(to_string(e.dst_slot), py::make_tuple(e.src.node, to_string(e.src.slot))));
        return l;
      }, "(slot, value) of every operand, in slot order")
      .def("get_incoming_inputs", [](const Graph &g, NodeId n) {
        py::list l;
        for (auto &e : g.node(n).inputs)
          if (!is_weight_slot(g.node(n).type, e.dst_slot)) l.append(py::make_tuple(e.src.node, to_string(e.src.slot)));
        return l;
      }, "operands that are activations (the operator's incoming tensor role INPUT)")
      .def("get_incoming_weights", [](const Graph &g, NodeId n) {
        py::list l;
        for (auto &e : g.node(n).inputs)
          if (is_weight_slot(g.node(n).type, e.dst_slot)) l.append(py::make_tuple(e.src.node, to_string(e.src.slot)));
        return l;
      }, "operands that are parameters (role WEIGHT)")
      .def("get_outgoing_tensors", [](const Graph &g, NodeId n) {
        py::list l;
        for (auto &o : g.node(n).outputs) l.append(py::make_tuple(n, to_string(o.slot)));
        return l;
      })
      .def("get_all_tensors", [](const Graph &g) {
        py::list l;
        for (auto &v : g.all_values()) l.append(py::make_tuple(v.node, to_string(v.slot)));
        return l;
      })
      .def("get_source_layer", [](const Graph &g, py::object v) { return value_from_py(v).node; })
      .def("without_layer_names", [](const Graph &g) {
        Graph r = g;
        for (NodeId n : r.node_ids()) r.node(n).name.clear();
        return r;
      }, "a copy whose layers have no names (names do not take part in `signature`, so it is isomorphic to the original)")
      .def("is_isomorphic_to", [](const Graph &a, const Graph &b) { return a.num_nodes() == b.num_nodes() && a.signature() == b.signature(); },
           "same operators with the same attributes and shapes wired the same way, whatever the node ids and names")
      .def("get_subgraph_incoming_edges", [](const Graph &g, std::set<NodeId> sub) {
        py::list l;
        for (NodeId n : sub)
          for (auto &e : g.node(n).inputs)
            if (!sub.count(e.src.node)) l.append(py::make_tuple(py::make_tuple(e.src.node, to_string(e.src.slot)), py::make_tuple(n, to_string(e.dst_slot))));
        return l;
      })
      .def("get_subgraph_outgoing_edges", [](const Graph &g, std::set<NodeId> sub) {
        py::list l;
        for (NodeId n : sub)
          for (auto &o : g.node(n).outputs)
            for (auto &c2 : g.consumers(ValueRef{n, o.slot}))
              if (!sub.count(c2.first)) l.append(py::make_tuple(py::make_tuple(n, to_string(o.slot)), py::make_tuple(c2.first, to_string(c2.second))));
        return l;
      })
      .def("get_subgraph_successors", [](const Graph &g, std::set<NodeId> sub) {
        std::set<NodeId> r;
        for (NodeId n : sub)
          for (NodeId s2 : g.successors(n))
            if (!sub.count(s2)) r.insert(s2);
        return r;
      })
      .def("as_dot", &Graph::as_dot)
      .def("copy", [](const Graph &g) { return Graph(g); })
      .def("to_v1", [](const Graph &g, bool parallel) { return json_to_py(graph_to_v1(g, parallel)); }, py::arg("parallel") = false)
      .def("to_v1_string", [](const Graph &g, bool parallel, int indent) { return graph_to_v1(g, parallel).dump(indent); },
           py::arg("parallel") = false, py::arg("indent") = -1)
      .def_static("from_v1", [](py::object o) {
        if (py::isinstance<py::str>(o)) return graph_from_v1(Json::parse(o.cast<std::string>()));
        return graph_from_v1(json_from_py(o));
      })
      .def("digraph", [](const Graph &g) {
        DiGraph d;
        for (auto &kv : g.nodes()) {
          d.add_node(kv.first);
          for (auto &e : kv.second.inputs) d.add_edge(e.src.node, kv.first);
        }
        return d;
      });

  m.def("infer_shapes", [](const std::string &type, py::object attrs, py::object inputs) {
    Inferred r = infer_shapes(optype_from_string(type), json_from_py(attrs), slot_shapes_from_py(inputs));
    py::dict d;
    d["weights"] = slot_shapes_to_py(r.weights);
    d["outputs"] = slot_shapes_to_py(r.outputs);
    return d;
  });
  m.def("is_weight_slot", [](const std::string &t, const std::string &s) { return is_weight_slot(optype_from_string(t), slot_from_string(s)); });
  m.def("is_parallel_op", [](const std::string &t) { return is_parallel_op(optype_from_string(t)); });
  m.def("operator_task_space", [](const Graph &g, NodeId n) { return operator_task_space(g.node(n), g); });
  m.def("operator_full_task_degrees", [](const Graph &g, NodeId n) { return operator_full_task_degrees(g.node(n), g); });
  m.def("operator_tensor_coord", [](const Graph &g, NodeId n, const std::vector<int> &task, const std::string &slot, bool is_output) {
    TensorCoord c = operator_tensor_coord(g.node(n), g, task, slot_from_string(slot), is_output);
    py::dict d;
    d["shard"] = c.shard;
    d["sum"] = c.sum_component;
    d["discard_copy"] = c.discard_copy_component;
    return d;
  }, py::arg("graph"), py::arg("node"), py::arg("task"), py::arg("slot") = "OUTPUT", py::arg("is_output") = true);
  m.def("operator_types", []() {
    std::vector<std::string> r;
#define X(n) r.push_back(#n);
    FF_OPTYPES(X)
#undef X
    return r;
  });
  m.def("slot_names", []() {
    std::vector<std::string> r;
#define X(n) r.push_back(#n);
    FF_SLOTS(X)
#undef X
    return r;
  });
  m.def("pcg_from_computation_graph", &pcg_from_computation_graph);
  m.def("json_roundtrip", [](const std::string &s) { return Json::parse(s).dump(); });

  // ---- builder
  auto V2 = [](const V &v) { return value_to_py(v); };
  auto VL = [](const std::vector<V> &vs) {
    py::list l;
    for (auto &v : vs) l.append(value_to_py(v));
    return l;
  };
  auto optinit = [](py::object o) -> OptInit { return o.is_none() ? OptInit() : OptInit(json_from_py(o)); };
  auto optstr = [](py::object o) -> std::optional<std::string> { return o.is_none() ? std::nullopt : std::optional<std::string>(o.cast<std::string>()); };
  auto optint = [](py::object o) -> std::optional<int64_t> { return o.is_none() ? std::nullopt : std::optional<int64_t>(o.cast<int64_t>()); };
  py::class_<GraphBuilder>(m, "GraphBuilder")
      .def(py::init<bool>(), py::arg("parallel") = false)
      .def_readwrite("graph", &GraphBuilder::graph)
      .def_property_readonly("parallel", &GraphBuilder::parallel)
      .def("shape", [](GraphBuilder &b, py::object v) { return b.shape(value_from_py(v)); })
      .def("create_input", [=](GraphBuilder &b, std::vector<int64_t> dims, const std::string &dt, bool grad, const std::string &name) {
        return V2(b.create_input(dims, datatype_from_string(dt), grad, name));
      }, py::arg("dims"), py::arg("dtype") = "FLOAT", py::arg("create_grad") = false, py::arg("name") = "")
      .def("create_weight", [=](GraphBuilder &b, std::vector<int64_t> dims, const std::string &dt, py::object init, bool grad, const std::string &name) {
        return V2(b.create_weight(dims, datatype_from_string(dt), optinit(init), grad, name));
      }, py::arg("dims"), py::arg("dtype") = "FLOAT", py::arg("initializer") = py::none(), py::arg("create_grad") = true, py::arg("name") = "")
      .def("add_layer", [=](GraphBuilder &b, const std::string &type, py::object attrs, py::object inputs, const std::string &name) {
        std::vector<std::pair<Slot, V>> ins;
        for (auto item : inputs) {
          auto t = item.cast<py::tuple>();
          ins.push_back({slot_from_string(t[0].cast<std::string>()), value_from_py(t[1])});
        }
        return VL(b.add_layer(optype_from_string(type), json_from_py(attrs), ins, name));
      }, py::arg("type"), py::arg("attrs"), py::arg("inputs"), py::arg("name") = "")
      .def("unary", [=](GraphBuilder &b, const std::string &op, py::object x, py::object scalar, const std::string &name) {
        std::optional<double> s = scalar.is_none() ? std::nullopt : std::optional<double>(scalar.cast<double>());
        return V2(b.unary(optype_from_string(op), value_from_py(x), s, name));
      }, py::arg("op"), py::arg("x"), py::arg("scalar") = py::none(), py::arg("name") = "")
      .def("binary", [=](GraphBuilder &b, const std::string &op, py::object x, py::object y, const std::string &name) {
        return V2(b.binary(optype_from_string(op), value_from_py(x), value_from_py(y), name));
      }, py::arg("op"), py::arg("x"), py::arg("y"), py::arg("name") = "")
      .def("dense", [=](GraphBuilder &b, py::object x, int64_t out, py::object act, bool bias, py::object wi, py::object bi, const std::string &name) {
        return V2(b.dense(value_from_py(x), out, optstr(act), bias, optinit(wi), optinit(bi), name));
      }, py::arg("x"), py::arg("out_channels"), py::arg("activation") = py::none(), py::arg("use_bias") = true,
           py::arg("projection_initializer") = py::none(), py::arg("bias_initializer") = py::none(), py::arg("name") = "")
      .def("conv2d", [=](GraphBuilder &b, py::object x, int64_t out, int kh, int kw, int sh, int sw, int ph, int pw, py::object act, int groups,
                         bool bias, py::object ki, py::object bi, const std::string &name) {
        return V2(b.conv2d(value_from_py(x), out, kh, kw, sh, sw, ph, pw, optstr(act), groups, bias, optinit(ki), optinit(bi), name));
      }, py::arg("x"), py::arg("out_channels"), py::arg("kernel_h"), py::arg("kernel_w"), py::arg("stride_h") = 1, py::arg("stride_w") = 1,
           py::arg("padding_h") = 0, py::arg("padding_w") = 0, py::arg("activation") = py::none(), py::arg("groups") = 1,
           py::arg("use_bias") = true, py::arg("kernel_initializer") = py::none(), py::arg("bias_initializer") = py::none(), py::arg("name") = "")
      .def("pool2d", [=](GraphBuilder &b, py::object x, int kh, int kw, int sh, int sw, int ph, int pw, const std::string &type, py::object act,
                         const std::string &name) {
        return V2(b.pool2d(value_from_py(x), kh, kw, sh, sw, ph, pw, type, optstr(act), name));
      }, py::arg("x"), py::arg("kernel_h"), py::arg("kernel_w"), py::arg("stride_h"), py::arg("stride_w"), py::arg("padding_h") = 0,
           py::arg("padding_w") = 0, py::arg("pool_type") = "MAX", py::arg("activation") = py::none(), py::arg("name") = "")
      .def("adaptive_pool2d", [=](GraphBuilder &b, py::object x, int oh, int ow, const std::string &type, const std::string &name) {
        return V2(b.adaptive_pool2d(value_from_py(x), oh, ow, type, name));
      }, py::arg("x"), py::arg("output_h"), py::arg("output_w"), py::arg("pool_type") = "AVG", py::arg("name") = "")
      .def("batch_norm", [=](GraphBuilder &b, py::object x, bool affine, py::object act, double eps, py::object mom, const std::string &name) {
        std::optional<double> mm = mom.is_none() ? std::nullopt : std::optional<double>(mom.cast<double>());
        return V2(b.batch_norm(value_from_py(x), affine, optstr(act), eps, mm, name));
      }, py::arg("x"), py::arg("affine") = true, py::arg("activation") = py::none(), py::arg("eps") = 1e-5, py::arg("momentum") = 0.1,
           py::arg("name") = "")
      .def("layer_norm", [=](GraphBuilder &b, py::object x, std::vector<int> axes, bool affine, double eps, const std::string &name) {
        return V2(b.layer_norm(value_from_py(x), axes, affine, eps, name));
      }, py::arg("x"), py::arg("axes") = std::vector<int>{-1}, py::arg("elementwise_affine") = true, py::arg("eps") = 1e-5, py::arg("name") = "")
      .def("embedding", [=](GraphBuilder &b, py::object x, int64_t n, int64_t d, const std::string &aggr, const std::string &dt, py::object init,
                            const std::string &name) {
        return V2(b.embedding(value_from_py(x), n, d, aggr, datatype_from_string(dt), optinit(init), name));
      }, py::arg("x"), py::arg("num_entries"), py::arg("out_dim"), py::arg("aggr") = "SUM", py::arg("dtype") = "FLOAT",
           py::arg("initializer") = py::none(), py::arg("name") = "")
      .def("multihead_attention", [=](GraphBuilder &b, py::object q, py::object k, py::object v, int64_t embed, int64_t heads, py::object kdim,
                                      py::object vdim, double dropout, bool bias, bool abkv, bool aza, py::object init, const std::string &name) {
        return V2(b.multihead_attention(value_from_py(q), value_from_py(k), value_from_py(v), embed, heads, optint(kdim), optint(vdim), dropout,
                                        bias, abkv, aza, optinit(init), name));
      }, py::arg("query"), py::arg("key"), py::arg("value"), py::arg("embed_dim"), py::arg("num_heads"), py::arg("kdim") = py::none(),
           py::arg("vdim") = py::none(), py::arg("dropout") = 0.0, py::arg("bias") = false, py::arg("add_bias_kv") = false,
           py::arg("add_zero_attn") = false, py::arg("initializer") = py::none(), py::arg("name") = "")
      .def("batch_matmul", [=](GraphBuilder &b, py::object x, py::object y, const std::string &name) {
        return V2(b.batch_matmul(value_from_py(x), value_from_py(y), name));
      }, py::arg("a"), py::arg("b"), py::arg("name") = "")
      .def("dropout", [=](GraphBuilder &b, py::object x, double rate, uint64_t seed, const std::string &name) {
        return V2(b.dropout(value_from_py(x), rate, seed, name));
      }, py::arg("x"), py::arg("rate"), py::arg("seed") = 0, py::arg("name") = "")
      .def("softmax", [=](GraphBuilder &b, py::object x, int dim, const std::string &name) { return V2(b.softmax(value_from_py(x), dim, name)); },
           py::arg("x"), py::arg("dim") = -1, py::arg("name") = "")
      .def("cast", [=](GraphBuilder &b, py::object x, const std::string &dt, const std::string &name) {
        return V2(b.cast(value_from_py(x), datatype_from_string(dt), name));
      }, py::arg("x"), py::arg("dtype"), py::arg("name") = "")
      .def("concat", [=](GraphBuilder &b, py::object xs, int axis, const std::string &name) {
        std::vector<V> vs;
        for (auto x : xs) vs.push_back(value_from_py(x));
        return V2(b.concat(vs, axis, name));
      }, py::arg("tensors"), py::arg("axis"), py::arg("name") = "")
      .def("split", [=](GraphBuilder &b, py::object x, std::vector<int64_t> sizes, int axis, const std::string &name) {
        return VL(b.split(value_from_py(x), sizes, axis, name));
      }, py::arg("x"), py::arg("sizes"), py::arg("axis"), py::arg("name") = "")
      .def("flat", [=](GraphBuilder &b, py::object x, int s, int e, const std::string &name) { return V2(b.flat(value_from_py(x), s, e, name)); },
           py::arg("x"), py::arg("start_dim") = 1, py::arg("end_dim") = -1, py::arg("name") = "")
      .def("transpose", [=](GraphBuilder &b, py::object x, std::vector<int> perm, const std::string &name) {
        return V2(b.transpose(value_from_py(x), perm, name));
      }, py::arg("x"), py::arg("perm"), py::arg("name") = "")
      .def("reshape", [=](GraphBuilder &b, py::object x, std::vector<int64_t> dims, const std::string &name) {
        return V2(b.reshape(value_from_py(x), dims, name));
      }, py::arg("x"), py::arg("shape"), py::arg("name") = "")
      .def("reverse", [=](GraphBuilder &b, py::object x, int axis, const std::string &name) { return V2(b.reverse(value_from_py(x), axis, name)); },
           py::arg("x"), py::arg("axis"), py::arg("name") = "")
      .def("gather", [=](GraphBuilder &b, py::object x, py::object idx, int dim, const std::string &name) {
        return V2(b.gather(value_from_py(x), value_from_py(idx), dim, name));
      }, py::arg("x"), py::arg("index"), py::arg("dim"), py::arg("name") = "")
      .def("top_k", [=](GraphBuilder &b, py::object x, int k, bool sorted, const std::string &name) {
        return VL(b.top_k(value_from_py(x), k, sorted, name));
      }, py::arg("x"), py::arg("k"), py::arg("sorted") = true, py::arg("name") = "")
      .def("reduce", [=](GraphBuilder &b, const std::string &op, py::object x, std::vector<int> axes, bool keep, const std::string &name) {
        return V2(b.reduce(optype_from_string(op), value_from_py(x), axes, keep, name));
      }, py::arg("op"), py::arg("x"), py::arg("axes"), py::arg("keepdims") = false, py::arg("name") = "")
      .def("broadcast", [=](GraphBuilder &b, py::object x, std::vector<int64_t> target, const std::string &name) {
        return V2(b.broadcast(value_from_py(x), target, name));
      }, py::arg("x"), py::arg("target_dims"), py::arg("name") = "")
      .def("noop", [=](GraphBuilder &b, py::object x, const std::string &name) { return V2(b.noop(value_from_py(x), name)); }, py::arg("x"),
           py::arg("name") = "")
      .def("parallel_partition", [=](GraphBuilder &b, py::object x, int dim, int deg, const std::string &name) {
        return V2(b.parallel_partition(value_from_py(x), dim, deg, name));
      }, py::arg("x"), py::arg("dim"), py::arg("degree"), py::arg("name") = "")
      .def("parallel_combine", [=](GraphBuilder &b, py::object x, int dim, int deg, const std::string &name) {
        return V2(b.parallel_combine(value_from_py(x), dim, deg, name));
      }, py::arg("x"), py::arg("dim"), py::arg("degree"), py::arg("name") = "")
      .def("parallel_replicate", [=](GraphBuilder &b, py::object x, int deg, const std::string &name) {
        return V2(b.parallel_replicate(value_from_py(x), deg, name));
      }, py::arg("x"), py::arg("degree"), py::arg("name") = "")
      .def("parallel_reduce", [=](GraphBuilder &b, py::object x, int deg, const std::string &name) {
        return V2(b.parallel_reduce(value_from_py(x), deg, name));
      }, py::arg("x"), py::arg("degree"), py::arg("name") = "");

  // ---- models
  m.def("model_names", &model_names);
  m.def("default_model_config", [](const std::string &n) { return json_to_py(default_model_config(n)); });
  m.def("tensor_dims_has_dim", &tensor_dims_has_dim);
  m.def("tensor_dims_is_broadcastable_to", &tensor_dims_is_broadcastable_to, py::arg("curr"), py::arg("goal"));
  m.def("get_broadcast_target_dims", &get_broadcast_target_dims);
  m.def("get_tensor_dims_coord_set", &get_tensor_dims_coord_set);
  m.def("tensor_dims_drop_dims", &tensor_dims_drop_dims, py::arg("dims"), py::arg("should_drop"));
  m.def("build_model", [](const std::string &n, py::object cfg) { return build_model(n, json_from_py(cfg)); }, py::arg("name"),
        py::arg("config") = py::none());

  // ---- graph algorithms
  py::class_<DiGraph>(m, "DiGraph")
      .def(py::init<>())
      .def(py::init([](std::vector<int> nodes, std::vector<std::pair<int, int>> edges) {
        DiGraph g;
        for (int n : nodes) g.add_node(n);
        for (auto &e : edges) g.add_edge(e.first, e.second);
        return g;
      }), py::arg("nodes"), py::arg("edges"))
      .def("add_node", &DiGraph::add_node)
      .def("add_edge", &DiGraph::add_edge)
      .def("nodes", &DiGraph::nodes)
      .def("edges", &DiGraph::edges)
      .def("successors", [](const DiGraph &g, int n) { return std::vector<int>(g.successors(n).begin(), g.successors(n).end()); })
      .def("predecessors", [](const DiGraph &g, int n) { return std::vector<int>(g.predecessors(n).begin(), g.predecessors(n).end()); })
      .def("sources", &DiGraph::sources)
      .def("sinks", &DiGraph::sinks);
  m.def("is_acyclic", &is_acyclic);
  m.def("topological_ordering", &topological_ordering);
  m.def("transitive_closure", &transitive_closure);
  m.def("transitive_reduction", &transitive_reduction);
  m.def("get_dominators", &get_dominators);
  m.def("get_post_dominators", &get_post_dominators);
  m.def("get_imm_dominator", &get_imm_dominator);
  m.def("flipped", &flipped);
  m.def("get_strict_dominators", &get_strict_dominators);
  m.def("get_imm_dominators_map", &get_imm_dominators_map);
  m.def("get_imm_post_dominator", &get_imm_post_dominator);
  m.def("get_imm_post_dominators_map", &get_imm_post_dominators_map);
  m.def("calculate_topo_rank", &calculate_topo_rank);
  m.def("get_node_with_greatest_topo_rank", &get_node_with_greatest_topo_rank);
  m.def("get_topological_ordering_from_starting_node", &get_topological_ordering_from_starting_node);
  m.def("get_edge_topological_ordering", &get_edge_topological_ordering);
  m.def("is_tree", &is_tree);
  m.def("get_edges_from_subgraph_to_subgraph", &get_edges_from_subgraph_to_subgraph);
  m.def("get_subgraph_outgoing_edges", &get_subgraph_outgoing_edges);
  m.def("get_subgraph_successors", &get_subgraph_successors);
  m.def("apply_contraction", &apply_contraction);
  m.def("contract_node", &contract_node);
  m.def("is_complete_bipartite_digraph", &is_complete_bipartite_digraph);
  m.def("digraph_as_dot", &digraph_as_dot);
  m.def("get_weakly_connected_components", &get_weakly_connected_components);
  m.def("get_longest_path_lengths_from_root", &get_longest_path_lengths_from_root);
  m.def("get_descendants", &get_descendants);
  m.def("get_ancestors", &get_ancestors);
  m.def("get_lowest_common_ancestor", &get_lowest_common_ancestor);
  m.def("is_2_terminal_dag", &is_2_terminal_dag);
  m.def("get_series_parallel_decomposition", [](const DiGraph &g) -> py::object {
    auto t = get_series_parallel_decomposition(g);
    if (!t) return py::none();
    return sp_to_py(*t);
  });
  m.def("sp_normalize", [](py::object t) {
    // a tree without a single node has no normal form (normalize_sp_decomposition.h refuses it as well)
    SPTree n = normalize_sp(sp_from_py(t));
    if (n.kind != SPTree::Leaf && n.children.empty()) throw std::runtime_error("sp_normalize: the decomposition holds no node");
    return sp_to_py(n);
  });
  m.def("sp_balanced_binary", [](py::object t) { return sp_to_py(balanced_binary_sp_tree(sp_from_py(t))); });
  m.def("sp_left_associative_binary", [](py::object t) { return sp_to_py(left_associative_binary_sp_tree(sp_from_py(t))); });
  m.def("sp_right_associative_binary", [](py::object t) { return sp_to_py(right_associative_binary_sp_tree(sp_from_py(t))); });
  m.def("sp_to_json", [](py::object t) { return json_to_py(sp_to_json(sp_from_py(t))); });
  m.def("sp_from_json", [](py::object j) { return sp_to_py(sp_from_json(json_from_py(j))); });
  m.def("sp_nodes", [](py::object t) { return sp_nodes(sp_from_py(t)); });
  m.def("sp_work_cost", [](py::object t, std::map<int, double> cost) {
    return sp_work_cost(sp_from_py(t), [&](int n) { auto it = cost.find(n); return it == cost.end() ? 1.0 : it->second; });
  }, py::arg("tree"), py::arg("cost") = std::map<int, double>{});
  m.def("sp_critical_path_cost", [](py::object t, std::map<int, double> cost) {
    return sp_critical_path_cost(sp_from_py(t), [&](int n) { auto it = cost.find(n); return it == cost.end() ? 1.0 : it->second; });
  }, py::arg("tree"), py::arg("cost") = std::map<int, double>{});
  m.def("digraph_from_sp", [](py::object t) { return digraph_from_sp(sp_from_py(t)); });
  m.def("naive_stratum_sync_sp_ization", [](const DiGraph &g) { return sp_to_py(naive_stratum_sync_sp_ization(g)); });
  m.def("work_duplicating_sp_ization", [](const DiGraph &g, bool coalesce) { return sp_to_py(work_duplicating_sp_ization(g, coalesce)); },
        py::arg("g"), py::arg("coalesce") = false);
  m.def("sp_ancestors", [](py::object t, int node) { return sp_ancestors(sp_from_py(t), node); }, py::arg("tree"), py::arg("node"));
  m.def("bridge_out_nodes", [](const DiGraph &g, std::set<int> nodes) {
    return bridge_out_nodes(g, [&](int n) { return nodes.count(n) > 0; });
  }, py::arg("g"), py::arg("nodes"));
  m.def("escribano_sp_ization", [](const DiGraph &g) { return sp_to_py(escribano_sp_ization(g)); });
  m.def("flexible_sp_ization", [](const DiGraph &g, std::map<int, double> cost) {
    return sp_to_py(flexible_sp_ization(g, [&](int n) { auto it = cost.find(n); return it == cost.end() ? 1.0 : it->second; }));
  }, py::arg("g"), py::arg("cost") = std::map<int, double>{});
  m.def("sp_preserves_dependencies", [](py::object t, const DiGraph &g) { return sp_preserves_dependencies(sp_from_py(t), g); });

  bind_substitutions(m);
  bind_search(m);
  bind_lowering(m);
  bind_utils(m);
  bind_dataflow(m);
  bind_containers(m);
}
