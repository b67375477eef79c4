// shape_inference.cc -- (parallel) shape inference for every operator.
//
// For each operator the rule maps the parallel shapes of its data inputs to
// the parallel shapes of its outputs and of the weights it expects.  A plain
// tensor shape is the special case in which all degrees are 1, so the same
// code serves computation graphs and parallel computation graphs.  The degree
// algebra follows lib/op-attrs/src/op-attrs/ops/*.cc of the reference:
//   * sharding a contracted dimension produces partial sums (sum_degree),
//   * replicated inputs (discard_copy_degree) shard the weight's output
//     dimension and so the output's channel dimension,
//   * the other input degrees replicate the weights.
#include <algorithm>
#include <numeric>

#include "ir.h"

namespace ff {

const PShape *find_slot(const SlotShapes &s, Slot slot) {
  for (auto &p : s) if (p.first == slot) return &p.second;
  return nullptr;
}
static const PShape &need(const SlotShapes &s, Slot slot, const char *op) {
  const PShape *p = find_slot(s, slot);
  if (!p) throw Error(std::string(op) + ": missing input slot " + to_string(slot));
  return *p;
}
static PShape with_degrees(const std::vector<int64_t> &sizes, const std::vector<int> &deg, int sum, int copy,
                           DataType dt) {
  PShape p;
  for (size_t i = 0; i < sizes.size(); ++i) {
    if (deg[i] < 1 || sizes[i] % deg[i] != 0)
      throw Error("degree " + std::to_string(deg[i]) + " does not divide dim of size " + std::to_string(sizes[i]));
    p.dims.push_back({sizes[i], deg[i]});
  }
  p.sum_degree = sum;
  p.discard_copy_degree = copy;
  p.dtype = dt;
  return p;
}
static int prod(const std::vector<int> &v, size_t from, size_t to) {
  int r = 1;
  for (size_t i = from; i < to; ++i) r *= v[i];
  return r;
}
static void require(bool c, const std::string &msg) {
  if (!c) throw Error(msg);
}
static PShape shape_from_attr(const Json &a) { return PShape::from_json(a); }

bool is_weight_slot(OpType type, Slot s) {
  switch (type) {
    case OpType::LINEAR: return s == Slot::WEIGHT || s == Slot::BIAS;
    case OpType::CONV2D: return s == Slot::FILTER || s == Slot::BIAS;
    case OpType::EMBEDDING: return s == Slot::WEIGHT;
    case OpType::MULTIHEAD_ATTENTION: return s == Slot::WEIGHT || s == Slot::INPUT_BIAS || s == Slot::OUTPUT_BIAS;
    case OpType::LAYERNORM:
    case OpType::BATCHNORM: return s == Slot::GAMMA || s == Slot::BETA;
    default: return false;
  }
}

static Json init_obj(const std::string &type, Json value) {
  Json j = Json::object();
  j["type"] = type;
  j["value"] = std::move(value);
  return j;
}
Json default_initializer(OpType type, Slot s, const Json &attrs, const SlotShapes &inputs) {
  // Linear / Conv2D: Kaiming-normal-like projection and U(-1/sqrt(fan_in), 1/sqrt(fan_in)) bias,
  // chosen by the reference to match PyTorch (lib/op-attrs/src/op-attrs/ops/linear.cc:234-287,
  // conv_2d.cc:204-253).  Embedding: N(0,1) (embedding.cc:117-134).  Norm scales: 1 / 0.
  auto uniform = [](double lo, double hi) {
    Json v = Json::object();
    v["seed"] = 0;
    v["min_val"] = lo;
    v["max_val"] = hi;
    return init_obj("uniform", v);
  };
  auto constant = [](double c) {
    Json v = Json::object();
    Json val = Json::object();
    val["type"] = "float";
    val["value"] = c;
    v["value"] = val;
    return init_obj("constant", v);
  };
  if (type == OpType::LINEAR || type == OpType::CONV2D) {
    const PShape &in = inputs.at(0).second;
    double fan_in;
    if (type == OpType::LINEAR) fan_in = (double)in.dims.back().size;
    else fan_in = (double)in.dims.at(1).size / attrs.get_int("groups", 1) * attrs.at("kernel_h").as_int() * attrs.at("kernel_w").as_int();
    double bound = 1.0 / std::sqrt(fan_in);
    if (s == Slot::BIAS) return uniform(-bound, bound);
    // the projection: KaimingNormalAttrs{a = sqrt(5), FAN_IN, LEAKY_RELU, seed 0} (linear.cc:253-259)
    Json v = Json::object();
    v["a"] = (double)std::sqrt(5.0f);
    v["mode"] = "FAN_IN";
    v["nonlinearity"] = "LEAKY_RELU";
    v["seed"] = 0;
    return init_obj("kaiming_normal", v);
  }
  if (type == OpType::EMBEDDING) {
    Json v = Json::object();
    v["seed"] = 0;
    v["mean"] = 0.0;
    v["stddev"] = 1.0;
    return init_obj("normal", v);
  }
  if (type == OpType::MULTIHEAD_ATTENTION) {
    if (s != Slot::WEIGHT) return init_obj("zero", Json::object());
    Json v = Json::object();
    v["seed"] = 0;
    return init_obj("glorot_uniform", v);
  }
  if (s == Slot::GAMMA) return constant(1.0);
  return init_obj("zero", Json::object());
}

static int64_t conv_out(int64_t in, int64_t k, int64_t stride, int64_t pad) { return (in + 2 * pad - k) / stride + 1; }

Inferred infer_shapes(OpType type, const Json &a, const SlotShapes &in) {
  Inferred r;
  auto out = [&](Slot s, PShape p) { r.outputs.push_back({s, std::move(p)}); };
  auto weight = [&](Slot s, PShape p) { r.weights.push_back({s, std::move(p)}); };

  if (type == OpType::INPUT || type == OpType::WEIGHT) {
    out(Slot::OUTPUT, shape_from_attr(a.at("tensor_shape")));
    return r;
  }
  if (type == OpType::NOOP || type == OpType::IDENTITY && false) {
    out(Slot::OUTPUT, need(in, Slot::INPUT, "noop"));
    return r;
  }
  if (is_element_unary(type) || type == OpType::DROPOUT) {
    const PShape &x = need(in, Slot::INPUT, "element_unary");
    require(x.sum_degree == 1, to_string(type) + ": expected sum degree 1 (a nonlinear op cannot be applied to partial sums)");
    require(x.discard_copy_degree == 1, to_string(type) + ": expected discard-copy degree 1");
    out(Slot::OUTPUT, x);
    return r;
  }
  if (is_element_binary(type)) {
    const PShape &l = need(in, Slot::LHS_INPUT, "element_binary");
    const PShape &rh = need(in, Slot::RHS_INPUT, "element_binary");
    require(l.ndim() == rh.ndim() || rh.ndim() <= l.ndim(), "element_binary: rank mismatch");
    PShape o = l;
    if (l.sizes() != rh.sizes()) {
      // trailing-dims broadcast of the rhs (bias-like) or size-1 dims
      int off = l.ndim() - rh.ndim();
      for (int i = 0; i < rh.ndim(); ++i) {
        int64_t ls = l.dims[off + i].size, rs = rh.dims[i].size;
        require(ls == rs || rs == 1 || ls == 1, "element_binary: shapes " + l.str() + " and " + rh.str() + " do not broadcast");
        if (ls == 1) o.dims[off + i] = rh.dims[i];
      }
    } else {
      require(l.degrees() == rh.degrees(), "element_binary: operand shard degrees differ: " + l.str() + " vs " + rh.str());
    }
    require(l.sum_degree == rh.sum_degree && l.discard_copy_degree == rh.discard_copy_degree,
            "element_binary: replica degrees differ");
    if (type != OpType::EW_ADD && type != OpType::EW_SUB)
      require(l.sum_degree == 1, "element_binary: only add/sub distribute over partial sums");
    if (type == OpType::EW_EQUAL || type == OpType::EW_GREATER || type == OpType::EW_LESS) o.dtype = DataType::BOOL;
    out(Slot::OUTPUT, o);
    return r;
  }
  switch (type) {
    case OpType::LINEAR: {
      const PShape &x = need(in, Slot::INPUT, "linear");
      require(x.ndim() >= 1, "linear: input needs at least one dim");
      int64_t oc = a.at("out_channels").as_int();
      auto deg = x.degrees();
      int n = x.ndim();
      int k = deg[n - 1];
      int others = prod(deg, 0, n - 1);
      auto sizes = x.sizes();
      int64_t ic = sizes[n - 1];
      sizes[n - 1] = oc;
      auto odeg = deg;
      odeg[n - 1] = x.discard_copy_degree;
      out(Slot::OUTPUT, with_degrees(sizes, odeg, x.sum_degree * k, 1, x.dtype));
      weight(Slot::WEIGHT, with_degrees({oc, ic}, {x.discard_copy_degree, k}, 1, x.sum_degree * others, x.dtype));
      if (a.get_bool("use_bias", true))
        weight(Slot::BIAS, with_degrees({oc}, {x.discard_copy_degree}, x.sum_degree * k, others, x.dtype));
      return r;
    }
    case OpType::BATCHMATMUL: {
      const PShape &l = need(in, Slot::LHS_INPUT, "batch_matmul");
      const PShape &rh = need(in, Slot::RHS_INPUT, "batch_matmul");
      require(l.ndim() == rh.ndim() && l.ndim() >= 2, "batch_matmul: operands need equal rank >= 2");
      int n = l.ndim();
      require(l.dims[n - 1].size == rh.dims[n - 2].size, "batch_matmul: inner dims differ: " + l.str() + " x " + rh.str());
      require(l.dims[n - 1].degree == rh.dims[n - 2].degree, "batch_matmul: inner degrees differ");
      for (int i = 0; i < n - 2; ++i)
        require(l.dims[i] == rh.dims[i], "batch_matmul: batch dims differ");
      // lhs' p-dim is replicated over rhs' p shards and vice versa
      require(l.discard_copy_degree == rh.dims[n - 1].degree && rh.discard_copy_degree == l.dims[n - 2].degree,
              "batch_matmul: each operand must be replicated across the other's free-dim shards");
      require(l.sum_degree == 1 && rh.sum_degree == 1, "batch_matmul: operands must not be partial sums");
      auto sizes = l.sizes();
      sizes[n - 1] = rh.dims[n - 1].size;
      auto deg = l.degrees();
      deg[n - 1] = rh.dims[n - 1].degree;
      out(Slot::OUTPUT, with_degrees(sizes, deg, l.dims[n - 1].degree, 1, l.dtype));
      return r;
    }
    case OpType::CONV2D: {
      const PShape &x = need(in, Slot::INPUT, "conv2d");
      require(x.ndim() == 4, "conv2d: input must be NCHW");
      int64_t oc = a.at("out_channels").as_int(), kh = a.at("kernel_h").as_int(), kw = a.at("kernel_w").as_int();
      int64_t sh = a.at("stride_h").as_int(), sw = a.at("stride_w").as_int();
      int64_t ph = a.at("padding_h").as_int(), pw = a.at("padding_w").as_int();
      int64_t groups = a.get_int("groups", 1);
      require(groups >= 1, "conv2d: groups must be positive");
      require(x.dims[2].degree == 1 && x.dims[3].degree == 1, "conv2d: spatial dims cannot be sharded");
      int nd = x.dims[0].degree, cd = x.dims[1].degree;
      int64_t ic = x.dims[1].size;
      // (the reference's shape inference asserts groups == 1, lib/op-attrs/src/op-attrs/ops/conv_2d.cc; grouped
      // convolutions are accepted here as long as the channel dims stay whole)
      require(groups == 1 || (ic % groups == 0 && oc % groups == 0), "conv2d: groups must divide input and output channels");
      require(groups == 1 || (cd == 1 && x.discard_copy_degree == 1), "conv2d: channels of a grouped convolution cannot be sharded");
      int64_t oh = conv_out(x.dims[2].size, kh, sh, ph), ow = conv_out(x.dims[3].size, kw, sw, pw);
      require(oh > 0 && ow > 0, "conv2d: kernel larger than padded input");
      out(Slot::OUTPUT, with_degrees({x.dims[0].size, oc, oh, ow}, {nd, x.discard_copy_degree, 1, 1}, x.sum_degree * cd, 1, x.dtype));
      weight(Slot::FILTER, with_degrees({oc, ic / groups, kh, kw}, {x.discard_copy_degree, cd, 1, 1}, 1, x.sum_degree * nd, x.dtype));
      if (a.get_bool("use_bias", true))
        weight(Slot::BIAS, with_degrees({oc}, {x.discard_copy_degree}, x.sum_degree * cd, nd, x.dtype));
      return r;
    }
    case OpType::POOL2D: {
      const PShape &x = need(in, Slot::INPUT, "pool2d");
      require(x.ndim() == 4, "pool2d: input must be NCHW");
      require(x.dims[2].degree == 1 && x.dims[3].degree == 1, "pool2d: spatial dims cannot be sharded");
      bool avg = a.get_string("pool_type", "MAX") == "AVG";
      require(x.sum_degree == 1 || (avg && a.get("activation", Json()).is_null()),
              "pool2d: partial sums only pass through average pooling without activation");
      int64_t oh = conv_out(x.dims[2].size, a.at("kernel_h").as_int(), a.at("stride_h").as_int(), a.at("padding_h").as_int());
      int64_t ow = conv_out(x.dims[3].size, a.at("kernel_w").as_int(), a.at("stride_w").as_int(), a.at("padding_w").as_int());
      require(oh > 0 && ow > 0, "pool2d: kernel larger than padded input");
      out(Slot::OUTPUT, with_degrees({x.dims[0].size, x.dims[1].size, oh, ow}, {x.dims[0].degree, x.dims[1].degree, 1, 1},
                                     x.sum_degree, x.discard_copy_degree, x.dtype));
      return r;
    }
    case OpType::BATCHNORM: {
      const PShape &x = need(in, Slot::INPUT, "batch_norm");
      require(x.ndim() >= 2, "batch_norm: input needs a channel dim");
      require(x.sum_degree == 1 && x.discard_copy_degree == 1, "batch_norm: expected sum and discard-copy degree 1");
      for (int i = 2; i < x.ndim(); ++i) require(x.dims[i].degree == 1, "batch_norm: spatial dims cannot be sharded");
      // The reference also forbids sharding the sample dim (batch_norm.cc:121-152); here a
      // sharded sample dim is accepted and means per-shard batch statistics.
      out(Slot::OUTPUT, x);
      if (a.get_bool("affine", true)) {
        int64_t c = x.dims[1].size;
        weight(Slot::GAMMA, with_degrees({c}, {x.dims[1].degree}, 1, x.dims[0].degree, x.dtype));
        weight(Slot::BETA, with_degrees({c}, {x.dims[1].degree}, 1, x.dims[0].degree, x.dtype));
      }
      return r;
    }
    case OpType::LAYERNORM: {
      const PShape &x = need(in, Slot::INPUT, "layer_norm");
      require(x.sum_degree == 1 && x.discard_copy_degree == 1, "layer_norm: expected sum and discard-copy degree 1");
      std::vector<int> axes;
      for (auto v : a.at("axes").as_ints()) axes.push_back(x.norm_dim((int)v));
      std::sort(axes.begin(), axes.end());
      int copy = 1;
      for (int i = 0; i < x.ndim(); ++i) {
        bool normed = std::find(axes.begin(), axes.end(), i) != axes.end();
        if (normed) require(x.dims[i].degree == 1, "layer_norm: normalised dims cannot be sharded");
        else copy *= x.dims[i].degree;
      }
      out(Slot::OUTPUT, x);
      if (a.get_bool("elementwise_affine", true)) {
        // scale/shift cover the normalised dims (PyTorch semantics)
        std::vector<int64_t> ws;
        std::vector<int> wd;
        for (int ax : axes) { ws.push_back(x.dims[ax].size); wd.push_back(1); }
        weight(Slot::GAMMA, with_degrees(ws, wd, 1, copy, x.dtype));
        weight(Slot::BETA, with_degrees(ws, wd, 1, copy, x.dtype));
      }
      return r;
    }
    case OpType::EMBEDDING: {
      const PShape &x = need(in, Slot::INPUT, "embedding");
      require(x.dtype == DataType::INT32 || x.dtype == DataType::INT64, "embedding: indices must be int32/int64");
      require(x.ndim() >= 1, "embedding: input needs a bag dim");
      int64_t oc = a.at("out_channels").as_int(), ne = a.at("num_entries").as_int();
      DataType dt = datatype_from_string(a.get_string("data_type", "FLOAT"));
      auto sizes = x.sizes();
      auto deg = x.degrees();
      int n = x.ndim();
      int bag_deg = deg[n - 1];
      sizes[n - 1] = oc;
      deg[n - 1] = x.discard_copy_degree;
      out(Slot::OUTPUT, with_degrees(sizes, deg, bag_deg * x.sum_degree, 1, dt));
      weight(Slot::WEIGHT, with_degrees({ne, oc}, {1, x.discard_copy_degree}, 1, prod(x.degrees(), 0, n), dt));
      return r;
    }
    case OpType::MULTIHEAD_ATTENTION: {
      const PShape &q = need(in, Slot::QUERY, "attention");
      const PShape &k = need(in, Slot::KEY, "attention");
      const PShape &v = need(in, Slot::VALUE, "attention");
      require(q.ndim() == 3 && k.ndim() == 3 && v.ndim() == 3, "attention: q/k/v must be [batch, seq, feature]");
      require(q.dims[0].size == k.dims[0].size && k.dims[0].size == v.dims[0].size, "attention: batch sizes differ");
      require(k.dims[1].size == v.dims[1].size, "attention: key/value sequence lengths differ");
      require(q.dims[1].degree == 1 && k.dims[1].degree == 1 && v.dims[1].degree == 1, "attention: sequence dim cannot be sharded");
      require(q.dims[2].degree == 1 && k.dims[2].degree == 1 && v.dims[2].degree == 1, "attention: feature dim cannot be sharded");
      require(q.dims[0].degree == k.dims[0].degree && k.dims[0].degree == v.dims[0].degree, "attention: batch degrees differ");
      require(q.discard_copy_degree == k.discard_copy_degree && k.discard_copy_degree == v.discard_copy_degree,
              "attention: q/k/v replication degrees differ");
      require(q.sum_degree == 1 && k.sum_degree == 1 && v.sum_degree == 1, "attention: inputs must not be partial sums");
      int64_t embed = a.at("embed_dim").as_int(), heads = a.at("num_heads").as_int();
      int64_t kdim = a.at("kdim").as_int(), vdim = a.at("vdim").as_int();
      int hd = q.discard_copy_degree;  // replicated inputs -> heads are sharded
      require(heads % hd == 0, "attention: head-parallel degree must divide num_heads");
      int bd = q.dims[0].degree;
      out(Slot::OUTPUT, with_degrees({q.dims[0].size, q.dims[1].size, embed}, {bd, 1, 1}, hd, 1, q.dtype));
      int64_t per_head = q.dims[2].size * kdim + k.dims[2].size * kdim + v.dims[2].size * vdim + vdim * embed;
      weight(Slot::WEIGHT, with_degrees({per_head, heads}, {1, hd}, 1, bd, q.dtype));
      if (a.get_bool("bias", false)) {
        weight(Slot::INPUT_BIAS, with_degrees({(kdim + kdim + vdim) * heads}, {hd}, 1, bd, q.dtype));
        weight(Slot::OUTPUT_BIAS, with_degrees({embed}, {1}, hd, bd, q.dtype));
      }
      return r;
    }
    case OpType::SOFTMAX: {
      const PShape &x = need(in, Slot::INPUT, "softmax");
      require(x.sum_degree == 1 && x.discard_copy_degree == 1, "softmax: expected sum and discard-copy degree 1");
      int d = x.norm_dim((int)a.get_int("dim", -1));
      require(x.dims[d].degree == 1, "softmax: the softmax dim cannot be sharded");
      out(Slot::OUTPUT, x);
      return r;
    }
    case OpType::CONCAT: {
      int n = (int)a.at("num_inputs").as_int();
      const PShape &x0 = need(in, input_slot_n(0), "concat");
      int ax = x0.norm_dim((int)a.at("axis").as_int());
      PShape o = x0;
      require(x0.dims[ax].degree == 1, "concat: the concat axis cannot be sharded");
      for (int i = 1; i < n; ++i) {
        const PShape &xi = need(in, input_slot_n(i), "concat");
        require(xi.ndim() == x0.ndim(), "concat: rank mismatch");
        require(xi.sum_degree == x0.sum_degree && xi.discard_copy_degree == x0.discard_copy_degree, "concat: replica degrees differ");
        for (int d = 0; d < x0.ndim(); ++d) {
          if (d == ax) continue;
          require(xi.dims[d] == x0.dims[d], "concat: non-axis dims differ: " + xi.str() + " vs " + x0.str());
        }
        require(xi.dims[ax].degree == 1, "concat: the concat axis cannot be sharded");
        o.dims[ax].size += xi.dims[ax].size;
      }
      out(Slot::OUTPUT, o);
      return r;
    }
    case OpType::SPLIT: {
      const PShape &x = need(in, Slot::INPUT, "split");
      int ax = x.norm_dim((int)a.at("axis").as_int());
      require(x.dims[ax].degree == 1, "split: the split axis cannot be sharded");
      auto splits = a.at("splits").as_ints();
      int64_t total = 0;
      for (auto s : splits) total += s;
      require(total == x.dims[ax].size, "split: sizes do not add up to the axis extent");
      for (size_t i = 0; i < splits.size(); ++i) {
        PShape o = x;
        o.dims[ax].size = splits[i];
        out(output_slot_n((int)i), o);
      }
      return r;
    }
    case OpType::FLAT: {
      const PShape &x = need(in, Slot::INPUT, "flat");
      int s = x.norm_dim((int)a.get_int("start_dim", 1)), e = x.norm_dim((int)a.get_int("end_dim", -1));
      require(s <= e, "flat: start_dim after end_dim");
      PShape o;
      o.dtype = x.dtype;
      o.sum_degree = x.sum_degree;
      o.discard_copy_degree = x.discard_copy_degree;
      for (int i = 0; i < s; ++i) o.dims.push_back(x.dims[i]);
      ShardDim f{1, 1};
      for (int i = s; i <= e; ++i) { f.size *= x.dims[i].size; f.degree *= x.dims[i].degree; }
      o.dims.push_back(f);
      for (int i = e + 1; i < x.ndim(); ++i) o.dims.push_back(x.dims[i]);
      out(Slot::OUTPUT, o);
      return r;
    }
    case OpType::TRANSPOSE: {
      const PShape &x = need(in, Slot::INPUT, "transpose");
      auto perm = a.at("permutation").as_ints();
      require((int)perm.size() == x.ndim(), "transpose: permutation rank mismatch");
      PShape o = x;
      for (int i = 0; i < x.ndim(); ++i) o.dims[i] = x.dims[x.norm_dim((int)perm[i])];
      out(Slot::OUTPUT, o);
      return r;
    }
    case OpType::RESHAPE: {
      const PShape &x = need(in, Slot::INPUT, "reshape");
      PShape o = shape_from_attr(a.at("shape"));
      require(o.num_elements() == x.num_elements(), "reshape: element counts differ");
      o.dtype = x.dtype;
      // leading dims that keep their size keep their degree; everything else must be unsharded
      int keep = 0;
      while (keep < o.ndim() && keep < x.ndim() && o.dims[keep].size == x.dims[keep].size) {
        o.dims[keep].degree = x.dims[keep].degree;
        ++keep;
      }
      for (int i = keep; i < x.ndim(); ++i) require(x.dims[i].degree == 1, "reshape: reshaped dims cannot be sharded");
      o.sum_degree = x.sum_degree;
      o.discard_copy_degree = x.discard_copy_degree;
      out(Slot::OUTPUT, o);
      return r;
    }
    case OpType::REVERSE: {
      const PShape &x = need(in, Slot::INPUT, "reverse");
      int ax = x.norm_dim((int)a.at("axis").as_int());
      require(x.dims[ax].degree == 1, "reverse: the reversed axis cannot be sharded");
      out(Slot::OUTPUT, x);
      return r;
    }
    case OpType::CAST: {
      PShape o = need(in, Slot::INPUT, "cast");
      o.dtype = datatype_from_string(a.at("dtype").as_string());
      out(Slot::OUTPUT, o);
      return r;
    }
    case OpType::GATHER: {
      const PShape &x = need(in, Slot::INPUT, "gather");
      const PShape &idx = need(in, Slot::INDEX, "gather");
      require(idx.dtype == DataType::INT32 || idx.dtype == DataType::INT64, "gather: index must be int32/int64");
      require(x.ndim() == idx.ndim(), "gather: rank mismatch");
      int d = x.norm_dim((int)a.at("dim").as_int());
      for (int i = 0; i < x.ndim(); ++i) {
        if (i != d) require(idx.dims[i].size <= x.dims[i].size, "gather: index dims exceed input dims");
      }
      require(x.is_unparallel() && idx.is_unparallel(), "gather: parallel gather is not supported");
      PShape o = idx;
      o.dtype = x.dtype;
      out(Slot::OUTPUT, o);
      return r;
    }
    case OpType::TOPK: {
      const PShape &x = need(in, Slot::INPUT, "topk");
      int64_t k = a.at("k").as_int();
      require(x.dims.back().degree == 1, "topk: last dim cannot be sharded");
      require(k <= x.dims.back().size, "topk: k exceeds the last dim");
      PShape v = x;
      v.dims.back().size = k;
      PShape i = v;
      i.dtype = DataType::INT32;
      out(Slot::OUTPUT, v);
      out(Slot::INDEX, i);
      return r;
    }
    case OpType::REDUCE_SUM: case OpType::REDUCE_MEAN: case OpType::REDUCE_MAX: case OpType::REDUCE_MIN:
    case OpType::REDUCE_PROD: case OpType::MEAN: case OpType::REDUCE_ARGMAX: case OpType::REDUCE_ARGMIN: {
      const PShape &x = need(in, Slot::INPUT, "reduce");
      std::vector<int> axes;
      for (auto v : a.at("axes").as_ints()) axes.push_back(x.norm_dim((int)v));
      bool keep = a.get_bool("keepdims", false);
      PShape o;
      o.dtype = x.dtype;
      o.sum_degree = x.sum_degree;
      o.discard_copy_degree = x.discard_copy_degree;
      for (int i = 0; i < x.ndim(); ++i) {
        bool red = std::find(axes.begin(), axes.end(), i) != axes.end();
        if (red) {
          require(x.dims[i].degree == 1, "reduce: reduced dims cannot be sharded");
          if (keep) o.dims.push_back({1, 1});
        } else o.dims.push_back(x.dims[i]);
      }
      if (o.dims.empty()) o.dims.push_back({1, 1});
      out(Slot::OUTPUT, o);
      return r;
    }
    case OpType::BROADCAST: {
      const PShape &x = need(in, Slot::INPUT, "broadcast");
      auto target = a.at("target_dims").contains("ff_ordered") ? a.at("target_dims").at("ff_ordered").as_ints() : a.at("target_dims").as_ints();
      require((int)target.size() >= x.ndim(), "broadcast: target rank below input rank");
      require(x.is_unparallel(), "broadcast: parallel broadcast is not supported");
      int off = (int)target.size() - x.ndim();
      for (int i = 0; i < x.ndim(); ++i)
        require(x.dims[i].size == target[off + i] || x.dims[i].size == 1, "broadcast: dims do not broadcast");
      out(Slot::OUTPUT, PShape::make(std::vector<int64_t>(target.begin(), target.end()), x.dtype));
      return r;
    }
    // ---- the four parallel operators (lib/op-attrs/src/op-attrs/ops/{repartition,combine,replicate,reduction}.cc)
    case OpType::REPARTITION: {
      PShape o = need(in, Slot::INPUT, "repartition");
      int d = o.norm_dim((int)a.at("repartition_dim").as_int());
      int deg = (int)a.at("repartition_degree").as_int();
      require(deg >= 1, "repartition: degree must be positive");
      o.dims[d].degree *= deg;
      require(o.dims[d].size % o.dims[d].degree == 0, "repartition: degree does not divide the dim");
      out(Slot::OUTPUT, o);
      return r;
    }
    case OpType::COMBINE: {
      PShape o = need(in, Slot::INPUT, "combine");
      int d = o.norm_dim((int)a.at("combine_dim").as_int());
      int deg = (int)a.at("combine_degree").as_int();
      require(deg >= 1 && o.dims[d].degree % deg == 0, "combine: degree must divide the dim's shard degree");
      o.dims[d].degree /= deg;
      out(Slot::OUTPUT, o);
      return r;
    }
    case OpType::REPLICATE: {
      PShape o = need(in, Slot::INPUT, "replicate");
      int deg = (int)a.at("replicate_degree").as_int();
      require(deg >= 1, "replicate: degree must be positive");
      o.discard_copy_degree *= deg;
      out(Slot::OUTPUT, o);
      return r;
    }
    case OpType::REDUCTION: {
      PShape o = need(in, Slot::INPUT, "reduction");
      int deg = (int)a.at("reduction_degree").as_int();
      require(deg >= 1 && o.sum_degree % deg == 0, "reduction: degree must divide the sum degree");
      o.sum_degree /= deg;
      out(Slot::OUTPUT, o);
      return r;
    }
    case OpType::NOOP: {
      out(Slot::OUTPUT, need(in, Slot::INPUT, "noop"));
      return r;
    }
    default:
      throw Error("shape inference: operator " + to_string(type) + " is not supported");
  }
}

// ---------------------------------------------------------------- task spaces
std::vector<int> operator_full_task_degrees(const Node &n, const Graph &g) {
  // The task grid of an operator is the shard grid of its (first) output plus its sum and
  // discard-copy replicas: each task produces one piece of the output.  For parallel ops
  // whose output is *less* parallel than the input (Combine, Reduction) the input grid is used.
  const PShape *s = &n.outputs.at(0).shape;
  if ((n.type == OpType::COMBINE || n.type == OpType::REDUCTION) && !n.inputs.empty())
    s = &g.shape(n.inputs[0].src);
  std::vector<int> d = s->degrees();
  d.push_back(s->sum_degree);
  d.push_back(s->discard_copy_degree);
  return d;
}
// Task coordinate (one entry per full task degree: output shard dims..., sum, discard-copy) -> the shard coordinate of
// one of the operator's tensors.  The Linear rules follow the degree algebra of its shape inference: the task's sum
// component enumerates (input sum replica, input-channel shard), the output-channel shard is the input's discard-copy
// replica, and a weight piece is replicated over (input sum replica, flattened batch shard).
static bool is_elementwise_unary(OpType t) {
  switch (t) {
    case OpType::RELU: case OpType::SIGMOID: case OpType::TANH: case OpType::GELU: case OpType::ELU: case OpType::EXP:
    case OpType::IDENTITY: case OpType::NOOP: case OpType::RSQRT: case OpType::SIN: case OpType::COS: case OpType::POW:
    case OpType::SCALAR_MULTIPLY: case OpType::SCALAR_ADD: case OpType::SCALAR_SUB: case OpType::SCALAR_TRUE_DIV:
    case OpType::DROPOUT: case OpType::CAST:
    // row-wise operators whose normalised dim is unsharded (their shape inference requires that) map like element-wise ones
    case OpType::SOFTMAX: case OpType::LAYERNORM:
      return true;
    default: return false;
  }
}
static bool is_elementwise_binary(OpType t) {
  return t == OpType::EW_ADD || t == OpType::EW_SUB || t == OpType::EW_MUL || t == OpType::EW_DIV || t == OpType::EW_MAX ||
         t == OpType::EW_MIN;
}
TensorCoord operator_tensor_coord(const Node &n, const Graph &g, const std::vector<int> &task, Slot slot, bool is_output) {
  const std::vector<int> full = operator_full_task_degrees(n, g);
  if (task.size() != full.size()) throw Error("task coordinate has " + std::to_string(task.size()) + " components, the task space " + std::to_string(full.size()));
  for (size_t i = 0; i < task.size(); ++i)
    if (task[i] < 0 || task[i] >= full[i]) throw Error("task coordinate outside the task space");
  const int nd = (int)task.size() - 2;
  TensorCoord same;
  same.shard.assign(task.begin(), task.begin() + nd);
  same.sum_component = task[nd];
  same.discard_copy_component = task[nd + 1];
  auto input_shape = [&](Slot s) -> const PShape & {
    const InEdge *e = n.in(s);
    if (!e) throw Error("operator has no input in slot " + to_string(s));
    return g.shape(e->src);
  };
  if (n.type == OpType::INPUT || n.type == OpType::WEIGHT) {
    if (!is_output) throw Error("source operators have no inputs");
    return same;
  }
  if (is_elementwise_unary(n.type)) return same;
  if (is_elementwise_binary(n.type)) {
    if (!is_output && input_shape(slot).degrees() != n.outputs.at(0).shape.degrees())
      throw Error("shard mapping of a broadcasting binary operator");
    return same;
  }
  if (n.type == OpType::TRANSPOSE) {
    if (is_output) return same;
    auto perm = n.attrs.at("permutation").as_ints();
    TensorCoord c = same;
    for (int i = 0; i < nd; ++i) c.shard[(size_t)perm[i]] = task[i];  // output dim i is input dim perm[i]
    return c;
  }
  if (n.type == OpType::LINEAR) {
    if (is_output) return same;
    const PShape &x = input_shape(Slot::INPUT);
    const int k = x.dims.back().degree;
    const int kk = task[nd] % k, s = task[nd] / k, o = task[nd - 1];
    auto xdeg = x.degrees();
    int flat_batch = 0;
    for (int i = 0; i < nd - 1; ++i) flat_batch = flat_batch * xdeg[i] + task[i];
    int others = 1;
    for (int i = 0; i < nd - 1; ++i) others *= xdeg[i];
    TensorCoord c;
    if (slot == Slot::INPUT) {
      c.shard.assign(task.begin(), task.begin() + nd - 1);
      c.shard.push_back(kk);
      c.sum_component = s;
      c.discard_copy_component = o;
    } else if (slot == Slot::WEIGHT) {
      c.shard = {o, kk};
      c.sum_component = 0;
      c.discard_copy_component = s * others + flat_batch;
    } else if (slot == Slot::BIAS) {
      // the bias is either a partial-sum tensor (one term per task sum component, as the degree algebra has it) or,
      // as the generated rules feed it, replicated to every task; either way only sum component 0 may add it
      const PShape &bs = input_shape(Slot::BIAS);
      c.shard = {o};
      if (bs.sum_degree > 1) {
        c.sum_component = task[nd] % bs.sum_degree;
        c.discard_copy_component = flat_batch % bs.discard_copy_degree;
      } else {
        c.sum_component = 0;
        c.discard_copy_component = (task[nd] * others + flat_batch) % bs.discard_copy_degree;
      }
    } else {
      throw Error("linear has no slot " + to_string(slot));
    }
    return c;
  }
  // parallel operators: the task grid is the more parallel side (see operator_full_task_degrees)
  if (n.type == OpType::REPARTITION || n.type == OpType::COMBINE) {
    const bool rep = n.type == OpType::REPARTITION;
    const PShape &ref = rep ? n.outputs.at(0).shape : input_shape(Slot::INPUT);
    const int dim = ref.norm_dim((int)n.attrs.at(rep ? "repartition_dim" : "combine_dim").as_int());
    const int k = (int)n.attrs.at(rep ? "repartition_degree" : "combine_degree").as_int();
    if (is_output == rep) return same;        // the side the task grid was taken from
    TensorCoord c = same;
    c.shard[(size_t)dim] = task[dim] / k;     // k consecutive fine shards make one coarse shard
    return c;
  }
  if (n.type == OpType::REPLICATE) {
    if (is_output) return same;
    TensorCoord c = same;
    c.discard_copy_component = task[nd + 1] / (int)n.attrs.at("replicate_degree").as_int();
    return c;
  }
  if (n.type == OpType::REDUCTION) {
    if (!is_output) return same;
    TensorCoord c = same;
    c.sum_component = task[nd] / (int)n.attrs.at("reduction_degree").as_int();
    return c;
  }
  throw Error("no operator-to-tensor shard mapping for " + to_string(n.type));
}

std::vector<int> operator_task_space(const Node &n, const Graph &g) {
  std::vector<int> r;
  for (int d : operator_full_task_degrees(n, g)) if (d > 1) r.push_back(d);
  return r;
}

}  // namespace ff
