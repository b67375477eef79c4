#include "dataflow.h"

#include <functional>

#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

namespace py = pybind11;

namespace ff {

// ---------------------------------------------------------------------------------------------- isomorphism
// A graph cannot be given chosen node ids (add_node numbers them), so a permutation is realised by inserting the nodes in an
// order in which the ids come out right where that is possible; where it is not (the new ids would break "producers first"),
// the nodes are inserted in topological order and `assigned` reports the ids they got.
OpenDataflowGraph permute_node_ids(const OpenDataflowGraphView &g, const std::map<int, int> &new_of_old, std::map<int, int> *assigned) {
  std::set<int> seen;
  for (int n : g.get_nodes()) {
    auto it = new_of_old.find(n);
    if (it == new_of_old.end()) throw std::invalid_argument("permute_node_ids: node " + std::to_string(n) + " has no new id");
    if (!seen.insert(it->second).second) throw std::invalid_argument("permute_node_ids: two nodes map to the same id");
  }
  OpenDataflowGraph out;
  std::map<int, int> in_map;
  for (auto &gi : g.get_graph_inputs()) in_map[gi.idx] = out.add_input().idx;
  std::map<int, int> got;
  for (int n : g.topological_ordering()) {
    std::vector<OpenDataflowValue> ins;
    for (auto &v : g.get_inputs(n)) {
      if (std::holds_alternative<DataflowOutput>(v)) {
        const DataflowOutput &o = std::get<DataflowOutput>(v);
        ins.push_back(DataflowOutput{got.at(o.node), o.idx});
      } else {
        ins.push_back(DataflowGraphInput{in_map.at(std::get<DataflowGraphInput>(v).idx)});
      }
    }
    got[n] = out.add_node(ins, (int)g.get_outputs(n).size()).node;
  }
  if (assigned) *assigned = got;
  return out;
}
OpenDataflowGraph permute_input_ids(const OpenDataflowGraphView &g, const std::map<int, int> &new_of_old) {
  std::vector<std::pair<int, int>> by_new;   // (new id, old id)
  std::set<int> seen;
  for (auto &gi : g.get_graph_inputs()) {
    auto it = new_of_old.find(gi.idx);
    if (it == new_of_old.end()) throw std::invalid_argument("permute_input_ids: input " + std::to_string(gi.idx) + " has no new id");
    if (!seen.insert(it->second).second) throw std::invalid_argument("permute_input_ids: two inputs map to the same id");
    by_new.push_back({it->second, gi.idx});
  }
  std::sort(by_new.begin(), by_new.end());
  OpenDataflowGraph out;
  std::map<int, int> in_map;   // old id -> id in `out` (inputs are created in the order of their new ids)
  for (auto &p : by_new) in_map[p.second] = out.add_input().idx;
  std::map<int, int> got;
  for (int n : g.topological_ordering()) {
    std::vector<OpenDataflowValue> ins;
    for (auto &v : g.get_inputs(n)) {
      if (std::holds_alternative<DataflowOutput>(v)) {
        const DataflowOutput &o = std::get<DataflowOutput>(v);
        ins.push_back(DataflowOutput{got.at(o.node), o.idx});
      } else {
        ins.push_back(DataflowGraphInput{in_map.at(std::get<DataflowGraphInput>(v).idx)});
      }
    }
    got[n] = out.add_node(ins, (int)g.get_outputs(n).size()).node;
  }
  return out;
}
bool is_isomorphic_under(const OpenDataflowGraphView &a, const OpenDataflowGraphView &b, const std::map<int, int> &node_map,
                         const std::map<int, int> &input_map) {
  if (a.get_nodes().size() != b.get_nodes().size() || a.get_graph_inputs().size() != b.get_graph_inputs().size()) return false;
  std::set<int> img;
  for (int n : a.get_nodes()) {
    auto it = node_map.find(n);
    if (it == node_map.end() || !b.has_node(it->second) || !img.insert(it->second).second) return false;
    if (a.get_outputs(n).size() != b.get_outputs(it->second).size()) return false;
    const auto &ia = a.get_inputs(n);
    const auto &ib = b.get_inputs(it->second);
    if (ia.size() != ib.size()) return false;
    for (size_t i = 0; i < ia.size(); ++i) {
      if (ia[i].index() != ib[i].index()) return false;
      if (std::holds_alternative<DataflowOutput>(ia[i])) {
        const DataflowOutput &x = std::get<DataflowOutput>(ia[i]), &y = std::get<DataflowOutput>(ib[i]);
        auto m = node_map.find(x.node);
        if (m == node_map.end() || m->second != y.node || x.idx != y.idx) return false;
      } else {
        auto m = input_map.find(std::get<DataflowGraphInput>(ia[i]).idx);
        if (m == input_map.end() || m->second != std::get<DataflowGraphInput>(ib[i]).idx) return false;
      }
    }
  }
  return true;
}
std::string open_dataflow_graph_as_dot(const OpenDataflowGraphView &g) {
  std::ostringstream o;
  o << "digraph {\n";
  for (auto &gi : g.get_graph_inputs()) o << "  i" << gi.idx << " [shape=box, label=\"input " << gi.idx << "\"];\n";
  for (int n : g.get_nodes()) o << "  n" << n << " [label=\"" << n << "\"];\n";
  for (int n : g.get_nodes()) {
    const auto &ins = g.get_inputs(n);
    for (size_t i = 0; i < ins.size(); ++i) {
      if (std::holds_alternative<DataflowOutput>(ins[i])) {
        const DataflowOutput &x = std::get<DataflowOutput>(ins[i]);
        o << "  n" << x.node << " -> n" << n << " [label=\"" << x.idx << " -> " << i << "\"];\n";
      } else {
        o << "  i" << std::get<DataflowGraphInput>(ins[i]).idx << " -> n" << n << " [label=\"-> " << i << "\"];\n";
      }
    }
  }
  o << "}\n";
  return o.str();
}

std::optional<std::map<int, int>> find_dataflow_isomorphism(const OpenDataflowGraphView &a, const OpenDataflowGraphView &b) {
  const std::vector<int> na = a.topological_ordering(), nb = b.topological_ordering();
  if (na.size() != nb.size() || a.get_graph_inputs().size() != b.get_graph_inputs().size()) return std::nullopt;
  std::map<int, int> node_map, input_map;
  std::set<int> used_nodes, used_inputs;
  // a's nodes are matched in a's topological order, so every operand's producer is matched before its consumer
  std::function<bool(size_t)> rec = [&](size_t i) -> bool {
    if (i == na.size()) return true;
    const int x = na[i];
    const auto &xin = a.get_inputs(x);
    for (int y : nb) {
      if (used_nodes.count(y)) continue;
      const auto &yin = b.get_inputs(y);
      if (xin.size() != yin.size() || a.get_outputs(x).size() != b.get_outputs(y).size()) continue;
      std::vector<std::pair<int, int>> new_inputs;  // graph-input bindings made for this candidate
      bool ok = true;
      for (size_t k = 0; k < xin.size() && ok; ++k) {
        if (xin[k].index() != yin[k].index()) { ok = false; break; }
        if (std::holds_alternative<DataflowOutput>(xin[k])) {
          const DataflowOutput &ox = std::get<DataflowOutput>(xin[k]), &oy = std::get<DataflowOutput>(yin[k]);
          auto it = node_map.find(ox.node);
          ok = it != node_map.end() && it->second == oy.node && ox.idx == oy.idx;
        } else {
          const int gx = std::get<DataflowGraphInput>(xin[k]).idx, gy = std::get<DataflowGraphInput>(yin[k]).idx;
          auto it = input_map.find(gx);
          if (it != input_map.end()) ok = it->second == gy;
          else if (used_inputs.count(gy)) ok = false;
          else {
            input_map[gx] = gy;
            used_inputs.insert(gy);
            new_inputs.push_back({gx, gy});
          }
        }
      }
      if (ok) {
        node_map[x] = y;
        used_nodes.insert(y);
        if (rec(i + 1)) return true;
        node_map.erase(x);
        used_nodes.erase(y);
      }
      for (auto &p : new_inputs) {
        input_map.erase(p.first);
        used_inputs.erase(p.second);
      }
    }
    return false;
  };
  if (!rec(0)) return std::nullopt;
  return node_map;
}

// ---------------------------------------------------------------------------------------------- command lines
CLISpec empty_cli_spec() { return CLISpec{}; }
CLIArgumentKey cli_add_flag(CLISpec &cli, const CLIFlagSpec &spec) {
  cli.flags.push_back(spec);
  return CLIFlagKey{(int)cli.flags.size() - 1};
}
CLIArgumentKey cli_add_help_flag(CLISpec &cli) { return cli_add_flag(cli, CLIFlagSpec{"help", 'h', "show this help message and exit"}); }
CLIArgumentKey cli_add_positional_argument(CLISpec &cli, const CLIPositionalArgumentSpec &spec) {
  cli.positional_arguments.push_back(spec);
  return CLIPositionalArgumentKey{(int)cli.positional_arguments.size() - 1};
}
std::vector<CLIFlagKey> cli_get_flag_keys(const CLISpec &cli) {
  std::vector<CLIFlagKey> r;
  for (size_t i = 0; i < cli.flags.size(); ++i) r.push_back({(int)i});
  return r;
}
CLIParseOutcome cli_parse(const CLISpec &cli, const std::vector<std::string> &args) {
  CLIParseResult res;
  for (auto k : cli_get_flag_keys(cli)) res.flags[k] = false;
  size_t used = 0;
  for (size_t i = 1; i < args.size(); ++i) {
    const std::string &arg = args[i];
    if (!arg.empty() && arg[0] == '-' && arg.size() > 1) {
      bool found = false;
      for (size_t f = 0; f < cli.flags.size(); ++f) {
        const CLIFlagSpec &fs = cli.flags[f];
        if (arg == "--" + fs.long_flag || (fs.short_flag && arg == std::string("-") + *fs.short_flag)) {
          res.flags[CLIFlagKey{(int)f}] = true;
          found = true;
        }
      }
      if (!found) return {std::nullopt, "Encountered unknown flag " + arg};
      continue;
    }
    if (used >= cli.positional_arguments.size())
      return {std::nullopt, "Too many positional arguments: expected " + std::to_string(cli.positional_arguments.size())};
    const CLIPositionalArgumentSpec &ps = cli.positional_arguments[used];
    if (ps.choices && std::find(ps.choices->begin(), ps.choices->end(), arg) == ps.choices->end())
      return {std::nullopt, "Invalid option for positional argument \"" + ps.name + "\": \"" + arg + "\""};
    res.positional_arguments[CLIPositionalArgumentKey{(int)used}] = arg;
    ++used;
  }
  // a help request is answered even when the positional arguments are missing
  bool help = false;
  for (size_t f = 0; f < cli.flags.size(); ++f)
    if (cli.flags[f].long_flag == "help" && res.flags[CLIFlagKey{(int)f}]) help = true;
  if (!help && used != cli.positional_arguments.size())
    return {std::nullopt, "Not enough positional arguments: found " + std::to_string(used) + ", expected " +
                              std::to_string(cli.positional_arguments.size())};
  return {res, ""};
}
bool cli_get_flag(const CLIParseResult &r, const CLIArgumentKey &k) { return r.flags.at(std::get<CLIFlagKey>(k)); }
std::string cli_get_argument(const CLIParseResult &r, const CLIArgumentKey &k) {
  return r.positional_arguments.at(std::get<CLIPositionalArgumentKey>(k));
}
std::string cli_get_help_message(const std::string &program_name, const CLISpec &cli) {
  auto pos_text = [](const CLIPositionalArgumentSpec &p) {
    if (!p.choices) return p.name;
    std::string s = "{";
    for (size_t i = 0; i < p.choices->size(); ++i) s += (i ? "," : "") + (*p.choices)[i];
    return s + "}";
  };
  auto flag_text = [](const CLIFlagSpec &f) {
    return (f.short_flag ? std::string("-") + *f.short_flag + ", " : std::string()) + "--" + f.long_flag;
  };
  std::ostringstream o;
  o << "usage: " << program_name;
  for (auto &f : cli.flags) o << " [" << (f.short_flag ? std::string("-") + *f.short_flag : "--" + f.long_flag) << "]";
  for (auto &p : cli.positional_arguments) o << " " << pos_text(p);
  o << "\n";
  size_t width = 0;
  for (auto &p : cli.positional_arguments) width = std::max(width, pos_text(p).size());
  for (auto &f : cli.flags) width = std::max(width, flag_text(f).size());
  width = std::min<size_t>(width, 20);
  auto row = [&](const std::string &key, const std::optional<std::string> &desc) {
    if (!desc) return "  " + key;
    if (key.size() > width) return "  " + key + "\n" + std::string(24, ' ') + *desc;
    return "  " + key + std::string(width - key.size() + 2, ' ') + *desc;
  };
  if (!cli.positional_arguments.empty()) {
    o << "\npositional arguments:\n";
    for (auto &p : cli.positional_arguments) o << row(pos_text(p), p.description) << "\n";
  }
  if (!cli.flags.empty()) {
    o << "\noptions:\n";
    for (auto &f : cli.flags) o << row(flag_text(f), f.description) << "\n";
  }
  return o.str();
}

}  // namespace ff

// ---------------------------------------------------------------------------------------------- python bindings
using namespace ff;

static py::object value_to_py(const OpenDataflowValue &v) {
  if (std::holds_alternative<DataflowOutput>(v)) {
    const DataflowOutput &o = std::get<DataflowOutput>(v);
    return py::make_tuple(o.node, o.idx);
  }
  return py::make_tuple("input", std::get<DataflowGraphInput>(v).idx);
}
static OpenDataflowValue value_from_py_df(const py::handle &h) {
  py::tuple t = h.cast<py::tuple>();
  if (py::isinstance<py::str>(t[0])) return DataflowGraphInput{t[1].cast<int>()};
  return DataflowOutput{t[0].cast<int>(), t[1].cast<int>()};
}

namespace ff {
void bind_dataflow(py::module &root) {
  py::module m = root.def_submodule("dataflow", "dataflow graph family and declarative command lines");
  // values are (node, output index) tuples; graph inputs are ("input", index) tuples
  py::class_<OpenDataflowGraphView>(m, "OpenDataflowGraphView")
      .def("get_nodes", &OpenDataflowGraphView::get_nodes)
      .def("has_node", &OpenDataflowGraphView::has_node)
      .def("get_outputs", [](const OpenDataflowGraphView &g, int n) {
        py::list l;
        for (auto &o : g.get_outputs(n)) l.append(py::make_tuple(o.node, o.idx));
        return l;
      })
      .def("get_inputs", [](const OpenDataflowGraphView &g, int n) {
        py::list l;
        for (auto &v : g.get_inputs(n)) l.append(value_to_py(v));
        return l;
      })
      .def("get_graph_inputs", [](const OpenDataflowGraphView &g) {
        py::list l;
        for (auto &i : g.get_graph_inputs()) l.append(py::make_tuple("input", i.idx));
        return l;
      })
      .def("query_edges", [](const OpenDataflowGraphView &g, std::optional<std::set<int>> src, std::optional<std::set<int>> dst) {
        DataflowEdgeQuery q;
        q.src_nodes = src;
        q.dst_nodes = dst;
        py::list l;
        for (auto &e : g.query_edges(q)) l.append(py::make_tuple(py::make_tuple(e.src.node, e.src.idx), py::make_tuple(e.dst.node, e.dst.idx)));
        return l;
      }, py::arg("src_nodes") = py::none(), py::arg("dst_nodes") = py::none())
      .def("get_uses", [](const OpenDataflowGraphView &g, py::object v) {
        py::list l;
        for (auto &u : g.get_uses(value_from_py_df(v))) l.append(py::make_tuple(u.node, u.idx));
        return l;
      })
      .def("get_unused_outputs", [](const OpenDataflowGraphView &g) {
        py::list l;
        for (auto &o : g.get_unused_outputs()) l.append(py::make_tuple(o.node, o.idx));
        return l;
      })
      .def("topological_ordering", &OpenDataflowGraphView::topological_ordering)
      .def("as_digraph", &OpenDataflowGraphView::as_digraph)
      .def("is_closed", &OpenDataflowGraphView::is_closed)
      .def("use_count", &OpenDataflowGraphView::use_count);
  py::class_<OpenDataflowGraph, OpenDataflowGraphView>(m, "OpenDataflowGraph")
      .def(py::init<>())
      .def("add_input", [](OpenDataflowGraph &g) { return py::make_tuple("input", g.add_input().idx); })
      .def("add_node", [](OpenDataflowGraph &g, py::list inputs, int num_outputs) {
        std::vector<OpenDataflowValue> v;
        for (auto h : inputs) v.push_back(value_from_py_df(h));
        NodeAddedResult r = g.add_node(v, num_outputs);
        py::list outs;
        for (auto &o : r.outputs) outs.append(py::make_tuple(o.node, o.idx));
        return py::make_tuple(r.node, outs);
      })
      .def("copy", [](const OpenDataflowGraph &g) { return OpenDataflowGraph(g); })
      .def("view", [](const OpenDataflowGraph &g) { return OpenDataflowGraphView(g); })
      .def_static("materialize", &OpenDataflowGraph::materialize);
  m.def("get_open_subgraph", [](const OpenDataflowGraphView &g, std::set<int> nodes) {
    OpenSubgraphResult r = get_open_subgraph(g, nodes);
    py::list ins;
    for (auto &p : r.input_of) ins.append(py::make_tuple(py::make_tuple("input", p.first.idx), value_to_py(p.second)));
    return py::make_tuple(r.graph, r.node_of, ins);
  });
  m.def("find_dataflow_isomorphism", &find_dataflow_isomorphism);
  auto edges_to_py = [](const std::set<DataflowEdge> &es) {
    py::list l;
    for (auto &e : es) l.append(py::make_tuple(py::make_tuple(e.src.node, e.src.idx), py::make_tuple(e.dst.node, e.dst.idx)));
    return l;
  };
  m.def("get_source_nodes", &get_source_nodes);
  m.def("get_unused_open_dataflow_graph_inputs", [](const OpenDataflowGraphView &g) {
    std::set<int> r;
    for (auto &gi : get_unused_open_dataflow_graph_inputs(g)) r.insert(gi.idx);
    return r;
  });
  m.def("get_dataflow_edges_from_node_to_node", [=](const OpenDataflowGraphView &g, int a, int b) { return edges_to_py(get_dataflow_edges_from_node_to_node(g, a, b)); });
  m.def("get_subgraph_inputs", [](const OpenDataflowGraphView &g, std::set<int> nodes) {
    py::list l;
    for (auto &v : get_subgraph_inputs(g, nodes)) l.append(value_to_py(v));
    return l;
  });
  m.def("get_subgraph_incoming_edges", [=](const OpenDataflowGraphView &g, std::set<int> nodes) { return edges_to_py(get_subgraph_incoming_edges(g, nodes)); });
  m.def("get_subgraph_outgoing_edges", [=](const OpenDataflowGraphView &g, std::set<int> nodes) { return edges_to_py(get_subgraph_outgoing_dataflow_edges(g, nodes)); });
  m.def("permute_node_ids", [](const OpenDataflowGraphView &g, std::map<int, int> new_of_old) {
    std::map<int, int> got;
    OpenDataflowGraph r = permute_node_ids(g, new_of_old, &got);
    return py::make_tuple(r, got);
  });
  m.def("permute_input_ids", &permute_input_ids);
  m.def("is_isomorphic_under", &is_isomorphic_under, py::arg("a"), py::arg("b"), py::arg("node_map"), py::arg("input_map") = std::map<int, int>{});
  m.def("open_dataflow_graph_as_dot", &open_dataflow_graph_as_dot);

  // named slots and labels, instantiated for what Python can hold: string slots, object labels
  using KG = KwargDataflowGraph<std::string>;
  py::class_<KG>(m, "KwargDataflowGraph")
      .def(py::init<>())
      .def("add_node", [](KG &g, std::map<std::string, std::pair<int, std::string>> inputs, std::vector<std::string> outs) {
        std::map<std::string, KG::Output> in;
        for (auto &kv : inputs) in[kv.first] = KG::Output{kv.second.first, kv.second.second};
        KG::Added a = g.add_node(in, outs);
        std::map<std::string, std::pair<int, std::string>> o;
        for (auto &kv : a.outputs) o[kv.first] = {kv.second.node, kv.second.slot};
        return py::make_tuple(a.node, o);
      })
      .def("get_nodes", &KG::get_nodes)
      .def("get_inputs", [](const KG &g, int n) {
        std::map<std::string, std::pair<int, std::string>> o;
        for (auto &kv : g.get_inputs(n)) o[kv.first] = {kv.second.node, kv.second.slot};
        return o;
      })
      .def("get_output_slots", &KG::get_output_slots)
      .def("positional", [](const KG &g) { return g.positional(); });
  using LG = LabelledOpenDataflowGraph<py::object, py::object>;
  py::class_<LG>(m, "LabelledOpenDataflowGraph")
      .def(py::init<>())
      .def("add_input", [](LG &g, py::object l) { return py::make_tuple("input", g.add_input(l).idx); })
      .def("add_node", [](LG &g, py::object label, py::list inputs, std::vector<py::object> out_labels) {
        std::vector<OpenDataflowValue> v;
        for (auto h : inputs) v.push_back(value_from_py_df(h));
        NodeAddedResult r = g.add_node(label, v, out_labels);
        py::list outs;
        for (auto &o : r.outputs) outs.append(py::make_tuple(o.node, o.idx));
        return py::make_tuple(r.node, outs);
      })
      .def("node_label", [](const LG &g, int n) { return g.at(n); })
      .def("value_label", [](const LG &g, py::object v) { return g.at(value_from_py_df(v)); })
      .def("raw", [](const LG &g) { return g.raw(); })
      .def("rewrite_node_labels", [](const LG &g, py::function f) {
        return g.rewrite_node_labels([&](int n, const py::object &l) { return py::object(f(n, l)); });
      });

  // command lines
  py::class_<CLISpec>(m, "CLISpec").def(py::init<>());
  py::class_<CLIParseResult>(m, "CLIParseResult");
  m.def("empty_cli_spec", &empty_cli_spec);
  m.def("cli_add_help_flag", [](CLISpec &c) { return py::make_tuple("flag", std::get<CLIFlagKey>(cli_add_help_flag(c)).raw_idx); });
  m.def("cli_add_flag", [](CLISpec &c, std::string long_flag, std::optional<std::string> short_flag, std::optional<std::string> desc) {
    std::optional<char> sf;
    if (short_flag && !short_flag->empty()) sf = (*short_flag)[0];
    return py::make_tuple("flag", std::get<CLIFlagKey>(cli_add_flag(c, CLIFlagSpec{long_flag, sf, desc})).raw_idx);
  }, py::arg("spec"), py::arg("long_flag"), py::arg("short_flag") = py::none(), py::arg("description") = py::none());
  m.def("cli_add_positional_argument", [](CLISpec &c, std::string name, std::optional<std::vector<std::string>> choices,
                                          std::optional<std::string> desc) {
    return py::make_tuple("positional",
                          std::get<CLIPositionalArgumentKey>(cli_add_positional_argument(c, CLIPositionalArgumentSpec{name, choices, desc})).raw_idx);
  }, py::arg("spec"), py::arg("name"), py::arg("choices") = py::none(), py::arg("description") = py::none());
  m.def("cli_parse", [](const CLISpec &c, std::vector<std::string> args) -> py::object {
    CLIParseOutcome o = cli_parse(c, args);
    if (!o.ok()) throw py::value_error(o.error);
    return py::cast(*o.result);
  });
  m.def("cli_get_flag", [](const CLIParseResult &r, py::tuple key) { return r.flags.at(CLIFlagKey{key[1].cast<int>()}); });
  m.def("cli_get_argument", [](const CLIParseResult &r, py::tuple key) -> py::object {
    auto it = r.positional_arguments.find(CLIPositionalArgumentKey{key[1].cast<int>()});
    if (it == r.positional_arguments.end()) return py::none();
    return py::str(it->second);
  });
  m.def("cli_get_help_message", &cli_get_help_message);
}
}  // namespace ff
