// lowering.cc -- from a (mapped) parallel computation graph to the list of task invocations a training
// iteration executes.
//
// Counterpart of the reference's dynamic open dataflow graph and its passes
// (lib/task-spec/include/task-spec/dynamic_graph/*.h): make_dynamic_open_dataflow_graph_from_{cg,mapped_pcg},
// perform_pass_expansion (pass_expansion.cc:114), perform_loss_insertion (loss_insertion.cc:16),
// perform_update_insertion (update_insertion.cc:106), perform_copy_insertion (copy_insertion.cc:83,153),
// perform_shard_expansion (shard_expansion.cc:89,140) and perform_machine_slicing (machine_slicing.cc:21).
//
// An invocation is {task, node, op_type, shard, device, inputs[], outputs[]}; a value reference is
// {node, slot, role, shard} with role in {FWD, GRAD, OPT:<slot>, LABEL}.  The passes are pure functions over
// the invocation list (a JSON array), applied in the order the reference applies them; the result is what
// each rank's executor runs, in list order.
#include <algorithm>
#include <set>

#include <cmath>
#include "pyjson.h"
#include "search.h"

namespace ff {

namespace {

Json value_ref(NodeId node, Slot slot, const std::string &role) {
  Json v = Json::object();
  v["node"] = node;
  v["slot"] = to_string(slot);
  v["role"] = role;
  v["shard"] = Json();
  return v;
}
Json invocation(const std::string &task, NodeId node, const Node &n) {
  Json j = Json::object();
  j["task"] = task;
  j["node"] = node;
  j["op_type"] = to_string(n.type);
  j["name"] = n.name;
  j["shard"] = Json();
  j["device"] = Json();
  j["inputs"] = Json::array();
  j["outputs"] = Json::array();
  return j;
}
// Pass-state predicates, checked at pass boundaries (the reference asserts no_part_of_graph_is_* before a pass and
// graph_is_fully_* after it, e.g. lib/task-spec/src/task-spec/dynamic_graph/shard_expansion.cc:142,149): a pass
// applied twice, or in the wrong order, is a programming error that should fail at once, not produce a plan with
// duplicated backward tasks.
int count_task(const Json &list, const std::string &task) {
  int n = 0;
  for (auto &inv : list.items())
    if (inv.at("task").as_string() == task) ++n;
  return n;
}
bool no_part_is_pass_expanded(const Json &list) { return count_task(list, "BWD") == 0; }
bool no_part_has_loss(const Json &list) { return count_task(list, "LOSS") == 0; }
bool no_part_has_updates(const Json &list) { return count_task(list, "UPD") == 0; }
bool no_part_has_copies(const Json &list) { return count_task(list, "COPY") == 0; }
bool no_part_is_shard_expanded(const Json &list) {
  for (auto &inv : list.items())
    if (!inv.at("shard").is_null() || !inv.at("device").is_null()) return false;
  return true;
}
bool fully_shard_expanded(const Json &list) {
  for (auto &inv : list.items())
    if (inv.at("shard").is_null() || inv.at("device").is_null()) return false;
  return true;
}
void require_state(bool ok, const char *pass, const char *what) {
  if (!ok) throw Error(std::string(pass) + ": " + what);
}

bool is_float(DataType d) { return d == DataType::FLOAT || d == DataType::HALF || d == DataType::DOUBLE || d == DataType::BFLOAT16; }

std::map<ValueRef, bool> grad_values(const Graph &g) {
  std::map<ValueRef, bool> req;
  for (NodeId n : g.topological_order()) {
    const Node &nd = g.node(n);
    bool r = nd.type == OpType::WEIGHT;
    if (nd.type != OpType::WEIGHT && nd.type != OpType::INPUT)
      for (auto &e : nd.inputs) r = r || req[e.src];
    for (auto &o : nd.outputs) req[{n, o.slot}] = r && is_float(o.shape.dtype) && o.create_grad;
  }
  return req;
}

}  // namespace

// one FWD invocation per operator, in topological order
Json make_dynamic_graph(const Graph &g) {
  Json list = Json::array();
  for (NodeId n : g.topological_order()) {
    const Node &nd = g.node(n);
    Json inv = invocation("FWD", n, nd);
    for (auto &e : nd.inputs) {
      Json v = value_ref(e.src.node, e.src.slot, "FWD");
      v["as"] = to_string(e.dst_slot);
      inv["inputs"].push_back(v);
    }
    for (auto &o : nd.outputs) inv["outputs"].push_back(value_ref(n, o.slot, "FWD"));
    list.push_back(inv);
  }
  return list;
}

// every operator that propagates a gradient gets a BWD twin, appended in reverse topological order
Json perform_pass_expansion(const Graph &g, const Json &list) {
  require_state(no_part_is_pass_expanded(list), "pass expansion", "the graph already has backward tasks");
  require_state(no_part_is_shard_expanded(list), "pass expansion", "the graph is already shard-expanded");
  Json out = list;
  auto req = grad_values(g);
  auto order = g.topological_order();
  for (auto it = order.rbegin(); it != order.rend(); ++it) {
    const Node &nd = g.node(*it);
    if (nd.type == OpType::INPUT || nd.type == OpType::WEIGHT) continue;
    bool any_out = false, any_in = false;
    for (auto &o : nd.outputs) any_out = any_out || req[{*it, o.slot}];
    for (auto &e : nd.inputs) any_in = any_in || req[e.src];
    if (!any_out || !any_in) continue;
    Json inv = invocation("BWD", *it, nd);
    for (auto &o : nd.outputs) {
      if (req[{*it, o.slot}]) inv["inputs"].push_back(value_ref(*it, o.slot, "GRAD"));
      inv["inputs"].push_back(value_ref(*it, o.slot, "FWD"));
    }
    for (auto &e : nd.inputs) {
      Json v = value_ref(e.src.node, e.src.slot, "FWD");
      v["as"] = to_string(e.dst_slot);
      inv["inputs"].push_back(v);
      if (req[e.src]) {
        Json gv = value_ref(e.src.node, e.src.slot, "GRAD");
        gv["as"] = to_string(e.dst_slot);
        inv["outputs"].push_back(gv);
      }
    }
    out.push_back(inv);
  }
  return out;
}

// LOSS consumes the logit and the label and produces the logit's gradient; it sits between the last FWD and the first BWD
Json perform_loss_insertion(const Graph &g, const Json &list, const ValueRef &logit, const Json &loss_attrs) {
  require_state(no_part_has_loss(list), "loss insertion", "the graph already has a loss task");
  require_state(no_part_is_shard_expanded(list), "loss insertion", "the graph is already shard-expanded");
  Json out = Json::array();
  Json loss = Json::object();
  loss["task"] = "LOSS";
  loss["node"] = logit.node;
  loss["op_type"] = "LOSS";
  loss["name"] = loss_attrs.get_string("type", "sparse_categorical_crossentropy");
  loss["attrs"] = loss_attrs;
  loss["shard"] = Json();
  loss["device"] = Json();
  loss["inputs"] = Json::array();
  loss["outputs"] = Json::array();
  loss["inputs"].push_back(value_ref(logit.node, logit.slot, "FWD"));
  loss["inputs"].push_back(value_ref(logit.node, logit.slot, "LABEL"));
  loss["outputs"].push_back(value_ref(logit.node, logit.slot, "GRAD"));
  bool placed = false;
  for (auto &inv : list.items()) {
    if (!placed && inv.at("task").as_string() == "BWD") { out.push_back(loss); placed = true; }
    out.push_back(inv);
  }
  if (!placed) out.push_back(loss);
  return out;
}

// one UPD invocation per trainable weight, with the optimizer's state slots (SGD: momentum; Adam: m, v)
Json perform_update_insertion(const Graph &g, const Json &list, const Json &optimizer_attrs) {
  require_state(no_part_has_updates(list), "update insertion", "the graph already has update tasks");
  require_state(no_part_is_shard_expanded(list), "update insertion", "the graph is already shard-expanded");
  Json out = list;
  std::string kind = optimizer_attrs.get_string("type", "sgd");
  std::vector<std::string> slots;
  if (kind == "adam") slots = {"OPT:m", "OPT:v"};
  else if (optimizer_attrs.get_float("momentum", 0.0) > 0) slots = {"OPT:momentum"};
  for (NodeId n : g.topological_order()) {
    const Node &nd = g.node(n);
    if (nd.type != OpType::WEIGHT || !nd.outputs[0].create_grad) continue;
    Json inv = invocation("UPD", n, nd);
    inv["attrs"] = optimizer_attrs;
    inv["inputs"].push_back(value_ref(n, Slot::OUTPUT, "FWD"));
    inv["inputs"].push_back(value_ref(n, Slot::OUTPUT, "GRAD"));
    for (auto &s : slots) inv["inputs"].push_back(value_ref(n, Slot::OUTPUT, s));
    inv["outputs"].push_back(value_ref(n, Slot::OUTPUT, "FWD"));
    for (auto &s : slots) inv["outputs"].push_back(value_ref(n, Slot::OUTPUT, s));
    out.push_back(inv);
  }
  return out;
}

static std::vector<int> devices_of(const Graph &g, NodeId n, const MachineSpec &m) {
  const Node &nd = g.node(n);
  auto ts = operator_task_space(nd, g);
  MachineView v = nd.view ? *nd.view : MachineView{};
  if (!nd.view) {
    auto vs = allowed_machine_views(ts, Resources{0, m.num_devices()}, m);
    if (!vs.empty()) v = vs.front();
  }
  return view_devices(v, ts, m);
}

// where a consumer's devices differ from its producer's, a COPY invocation moves the value (and, in the
// backward direction, its gradient)
Json perform_copy_insertion(const Graph &g, const Json &list, const MachineSpec &m) {
  require_state(no_part_has_copies(list), "copy insertion", "the graph already has copy tasks");
  require_state(no_part_is_shard_expanded(list), "copy insertion", "copies are inserted before shard expansion");
  Json out = Json::array();
  for (auto &inv : list.items()) {
    const std::string task = inv.at("task").as_string();
    if (task == "FWD") {
      NodeId n = (NodeId)inv.at("node").as_int();
      auto dn = devices_of(g, n, m);
      std::sort(dn.begin(), dn.end());
      for (auto &e : g.node(n).inputs) {
        auto dp = devices_of(g, e.src.node, m);
        std::sort(dp.begin(), dp.end());
        if (dp == dn || std::includes(dp.begin(), dp.end(), dn.begin(), dn.end())) continue;
        Json cp = Json::object();
        cp["task"] = "COPY";
        cp["node"] = n;
        cp["op_type"] = "COPY";
        cp["name"] = "";
        cp["shard"] = Json();
        cp["device"] = Json();
        cp["src_devices"] = Json::from_ints(dp);
        cp["dst_devices"] = Json::from_ints(dn);
        cp["inputs"] = Json::array();
        cp["outputs"] = Json::array();
        cp["inputs"].push_back(value_ref(e.src.node, e.src.slot, "FWD"));
        Json o = value_ref(e.src.node, e.src.slot, "FWD");
        o["copy_for"] = n;
        cp["outputs"].push_back(o);
        out.push_back(cp);
      }
    } else if (task == "BWD") {
      // the mirror image: the gradient of one of this operator's outputs is produced by a consumer's backward task on
      // the consumer's devices and has to reach this operator's devices first
      NodeId n = (NodeId)inv.at("node").as_int();
      auto dn = devices_of(g, n, m);
      std::sort(dn.begin(), dn.end());
      std::set<std::pair<NodeId, int>> done;   // (consumer, output slot): one copy per consumer and value
      for (auto &in : inv.at("inputs").items()) {
        if (in.at("role").as_string() != "GRAD") continue;
        const Slot slot = slot_from_string(in.at("slot").as_string());
        for (NodeId cons : g.successors(n)) {
          bool reads = false;
          for (auto &e : g.node(cons).inputs) reads = reads || (e.src.node == n && e.src.slot == slot);
          if (!reads || !done.insert({cons, (int)slot}).second) continue;
          auto dc = devices_of(g, cons, m);
          std::sort(dc.begin(), dc.end());
          if (dc == dn || std::includes(dc.begin(), dc.end(), dn.begin(), dn.end())) continue;
          Json cp = Json::object();
          cp["task"] = "COPY";
          cp["node"] = n;
          cp["op_type"] = "COPY";
          cp["name"] = "";
          cp["shard"] = Json();
          cp["device"] = Json();
          cp["src_devices"] = Json::from_ints(dc);
          cp["dst_devices"] = Json::from_ints(dn);
          cp["inputs"] = Json::array();
          cp["outputs"] = Json::array();
          cp["inputs"].push_back(value_ref(n, slot, "GRAD"));
          Json o = value_ref(n, slot, "GRAD");
          o["copy_for"] = n;
          o["copy_from"] = cons;
          cp["outputs"].push_back(o);
          out.push_back(cp);
        }
      }
    }
    out.push_back(inv);
  }
  return out;
}

// one invocation per shard of the operator's task space, bound to the device its machine view assigns
Json perform_shard_expansion(const Graph &g, const Json &list, const MachineSpec &m) {
  require_state(no_part_is_shard_expanded(list), "shard expansion", "the graph is already shard-expanded");
  Json out = Json::array();
  for (auto &inv : list.items()) {
    NodeId n = (NodeId)inv.at("node").as_int();
    std::vector<int> devs;
    if (inv.at("task").as_string() == "COPY") devs = inv.at("dst_devices").is_array() ? std::vector<int>() : std::vector<int>();
    if (inv.at("task").as_string() == "COPY") {
      for (auto v : inv.at("dst_devices").as_ints()) devs.push_back((int)v);
    } else {
      devs = devices_of(g, n, m);
    }
    if (devs.empty()) devs.push_back(0);
    for (size_t s = 0; s < devs.size(); ++s) {
      Json x = inv;
      x["shard"] = (long long)s;
      x["num_shards"] = (long long)devs.size();
      x["device"] = devs[s];
      out.push_back(x);
    }
  }
  require_state(fully_shard_expanded(out), "shard expansion", "a task was left without shard or device");
  return out;
}

Json perform_machine_slicing(const Json &list, int device) {
  require_state(fully_shard_expanded(list), "machine slicing", "the graph must be shard-expanded first");
  Json out = Json::array();
  for (auto &inv : list.items())
    if (inv.at("device").as_int() == device) out.push_back(inv);
  return out;
}

// the full pipeline of create_pcg_instance (pcg_instance.cc:90-109)
Json lower_training_graph(const Graph &g, const MachineSpec &m, const std::optional<ValueRef> &logit, const Json &loss_attrs,
                          const Json &optimizer_attrs, bool distributed) {
  Json l = make_dynamic_graph(g);
  l = perform_pass_expansion(g, l);
  if (logit) l = perform_loss_insertion(g, l, *logit, loss_attrs);
  l = perform_update_insertion(g, l, optimizer_attrs);
  if (distributed) {
    l = perform_copy_insertion(g, l, m);
    l = perform_shard_expansion(g, l, m);
  }
  return l;
}

// Optimizer attributes (lib/pcg/include/pcg/optimizers/{sgd,adam}_optimizer_attrs.dtg.toml) and the per-iteration
// schedule of Adam's bias correction (lib/pcg/src/pcg/optimizer_attrs.cc:7-25): beta_t and beta2_t are the running
// powers of beta1 and beta2, alpha_t = alpha * sqrt(1 - beta2_t) / (1 - beta_t) the step size of that iteration.
Json make_sgd_optimizer_attrs(double lr, double momentum, bool nesterov, double weight_decay) {
  if (lr < 0 || momentum < 0 || weight_decay < 0) throw Error("sgd optimizer: negative hyper-parameter");
  Json a = Json::object();
  a["type"] = "sgd";
  a["lr"] = lr;
  a["momentum"] = momentum;
  a["nesterov"] = nesterov;
  a["weight_decay"] = weight_decay;
  return a;
}
Json make_adam_optimizer_attrs(double alpha, double beta1, double beta2, double weight_decay, double epsilon) {
  if (alpha < 0 || beta1 < 0 || beta1 >= 1 || beta2 < 0 || beta2 >= 1 || epsilon <= 0) throw Error("adam optimizer: hyper-parameter out of range");
  Json a = Json::object();
  a["type"] = "adam";
  a["alpha"] = alpha;
  a["beta1"] = beta1;
  a["beta2"] = beta2;
  a["weight_decay"] = weight_decay;
  a["epsilon"] = epsilon;
  a["alpha_t"] = alpha;   // before the first iteration
  a["beta_t"] = 1.0;
  a["beta2_t"] = 1.0;
  return a;
}
Json get_optimizer_attrs_for_next_iter(const Json &old) {
  const std::string type = old.get_string("type", "sgd");
  if (type == "sgd") return old;  // nothing changes between iterations
  if (type != "adam") throw Error("unknown optimizer type " + type);
  Json a = old;
  const double beta_t = old.at("beta_t").as_float() * old.at("beta1").as_float();
  const double beta2_t = old.at("beta2_t").as_float() * old.at("beta2").as_float();
  a["beta_t"] = beta_t;
  a["beta2_t"] = beta2_t;
  a["alpha_t"] = old.at("alpha").as_float() * std::sqrt(1.0 - beta2_t) / (1.0 - beta_t);
  return a;
}

void bind_lowering(py::module &m) {
  m.def("make_sgd_optimizer_attrs", [](double lr, double momentum, bool nesterov, double wd) {
    return json_to_py(make_sgd_optimizer_attrs(lr, momentum, nesterov, wd));
  }, py::arg("lr"), py::arg("momentum") = 0.0, py::arg("nesterov") = false, py::arg("weight_decay") = 0.0);
  m.def("make_adam_optimizer_attrs", [](double alpha, double b1, double b2, double wd, double eps) {
    return json_to_py(make_adam_optimizer_attrs(alpha, b1, b2, wd, eps));
  }, py::arg("alpha") = 1e-3, py::arg("beta1") = 0.9, py::arg("beta2") = 0.999, py::arg("weight_decay") = 0.0, py::arg("epsilon") = 1e-8);
  m.def("get_optimizer_attrs_for_next_iter", [](py::object a) { return json_to_py(get_optimizer_attrs_for_next_iter(json_from_py(a))); });
  m.def("make_dynamic_graph", [](const Graph &g) { return json_to_py(make_dynamic_graph(g)); });
  m.def("perform_pass_expansion", [](const Graph &g, py::object l) { return json_to_py(perform_pass_expansion(g, json_from_py(l))); });
  m.def("perform_loss_insertion", [](const Graph &g, py::object l, py::object logit, py::object attrs) {
    return json_to_py(perform_loss_insertion(g, json_from_py(l), value_from_py(logit), json_from_py(attrs)));
  });
  m.def("perform_update_insertion", [](const Graph &g, py::object l, py::object attrs) {
    return json_to_py(perform_update_insertion(g, json_from_py(l), json_from_py(attrs)));
  });
  m.def("perform_copy_insertion", [](const Graph &g, py::object l, const MachineSpec &ms) {
    return json_to_py(perform_copy_insertion(g, json_from_py(l), ms));
  });
  m.def("perform_shard_expansion", [](const Graph &g, py::object l, const MachineSpec &ms) {
    return json_to_py(perform_shard_expansion(g, json_from_py(l), ms));
  });
  m.def("perform_machine_slicing", [](py::object l, int device) { return json_to_py(perform_machine_slicing(json_from_py(l), device)); });
  m.def("lower_training_graph", [](const Graph &g, const MachineSpec &ms, py::object logit, py::object loss_attrs, py::object opt_attrs,
                                   bool distributed) {
    std::optional<ValueRef> lv;
    if (!logit.is_none()) lv = value_from_py(logit);
    return json_to_py(lower_training_graph(g, ms, lv, json_from_py(loss_attrs), json_from_py(opt_attrs), distributed));
  }, py::arg("graph"), py::arg("machine"), py::arg("logit") = py::none(), py::arg("loss_attrs") = py::dict(),
        py::arg("optimizer_attrs") = py::dict(), py::arg("distributed") = false);
}

}  // namespace ff
