// pyjson.h -- conversions between Python objects and ff::Json / core value types for the pybind11 module.
#pragma once
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "graph_algos.h"
#include "ir.h"

namespace py = pybind11;

namespace ff {

inline Json json_from_py(const py::handle &o) {
  if (o.is_none()) return Json();
  if (py::isinstance<py::bool_>(o)) return Json(o.cast<bool>());
  if (py::isinstance<py::int_>(o)) return Json(o.cast<long long>());
  if (py::isinstance<py::float_>(o)) return Json(o.cast<double>());
  if (py::isinstance<py::str>(o)) return Json(o.cast<std::string>());
  if (py::isinstance<py::dict>(o)) {
    Json j = Json::object();
    for (auto kv : o.cast<py::dict>()) j[py::str(kv.first).cast<std::string>()] = json_from_py(kv.second);
    return j;
  }
  if (py::isinstance<py::list>(o) || py::isinstance<py::tuple>(o) || py::isinstance<py::set>(o)) {
    Json j = Json::array();
    for (auto x : o) j.push_back(json_from_py(x));
    return j;
  }
  // numpy scalars and the like
  if (py::hasattr(o, "item")) return json_from_py(o.attr("item")());
  throw std::runtime_error("cannot convert Python object of type " + py::str(o.get_type()).cast<std::string>() + " to JSON");
}

inline py::object json_to_py(const Json &j) {
  switch (j.kind()) {
    case Json::Null: return py::none();
    case Json::Bool: return py::bool_(j.as_bool());
    case Json::Int: return py::int_(j.as_int());
    case Json::Float: return py::float_(j.as_float());
    case Json::String: return py::str(j.as_string());
    case Json::Array: {
      py::list l;
      for (auto &x : j.items()) l.append(json_to_py(x));
      return std::move(l);
    }
    default: {
      py::dict d;
      for (auto &kv : j.fields()) d[py::str(kv.first)] = json_to_py(kv.second);
      return std::move(d);
    }
  }
}

inline ValueRef value_from_py(const py::handle &o) {
  auto t = o.cast<py::tuple>();
  if (t.size() != 2) throw std::runtime_error("a value is a (node_id, slot_name) pair");
  return ValueRef{t[0].cast<int>(), slot_from_string(t[1].cast<std::string>())};
}
inline py::tuple value_to_py(const ValueRef &v) { return py::make_tuple(v.node, to_string(v.slot)); }

inline py::object sp_to_py(const SPTree &t) {
  if (t.kind == SPTree::Leaf) return py::int_(t.node);
  py::list cs;
  for (auto &c : t.children) cs.append(sp_to_py(c));
  return py::make_tuple(t.kind == SPTree::Series ? "S" : "P", cs);
}
inline SPTree sp_from_py(const py::handle &o) {
  if (py::isinstance<py::int_>(o)) return SPTree::leaf(o.cast<int>());
  auto t = o.cast<py::tuple>();
  std::string k = t[0].cast<std::string>();
  SPTree r;
  r.kind = (k == "S") ? SPTree::Series : SPTree::Parallel;
  for (auto c : t[1]) r.children.push_back(sp_from_py(c));
  return r;
}

}  // namespace ff
