// models.cc -- model zoo: computation-graph builders with the reference's default configs
// (lib/models/src/models/{transformer,bert,inception_v3,dlrm,candle_uno,split_test}) plus the
// token-id variants used for training benchmarks (embedding front end + language-model head).
#include "models.h"

#include <cmath>

namespace ff {

static Json cfg_defaults(const Json &user, Json defaults) {
  if (user.is_object())
    for (auto &kv : user.fields()) defaults[kv.first] = kv.second;
  return defaults;
}
static Json normal_init(double stddev, long long seed = 0) {
  Json v = Json::object();
  v["seed"] = seed;
  v["mean"] = 0.0;
  v["stddev"] = stddev;
  Json j = Json::object();
  j["type"] = "normal";
  j["value"] = v;
  return j;
}
static Json uniform_init(double lo, double hi, long long seed = 0) {
  Json v = Json::object();
  v["seed"] = seed;
  v["min_val"] = lo;
  v["max_val"] = hi;
  Json j = Json::object();
  j["type"] = "uniform";
  j["value"] = v;
  return j;
}
static Json zero_init() {
  Json j = Json::object();
  j["type"] = "zero";
  j["value"] = Json::object();
  return j;
}
static Json truncated_normal_init(double stddev) {
  Json v = Json::object();
  v["seed"] = 0;
  v["mean"] = 0.0;
  v["stddev"] = stddev;
  v["min_cutoff"] = -2 * stddev;
  v["max_cutoff"] = 2 * stddev;
  Json j = Json::object();
  j["type"] = "truncated_normal";
  j["value"] = v;
  return j;
}
static Json glorot_normal_init() {
  Json v = Json::object();
  v["seed"] = 0;
  Json j = Json::object();
  j["type"] = "glorot_normal";
  j["value"] = v;
  return j;
}

// ---------------------------------------------------------------- Transformer
Json default_transformer_config() {
  Json c = Json::object();
  c["num_features"] = 512; c["sequence_length"] = 512; c["batch_size"] = 64; c["dim_feedforward"] = 2048;
  c["num_heads"] = 8; c["num_encoder_layers"] = 6; c["num_decoder_layers"] = 6; c["dropout"] = 0.1;
  c["layer_norm_eps"] = 1e-5; c["vocab_size"] = 64;
  return c;
}
namespace {
struct TCfg {
  int64_t d, seq, batch, ffn, heads, enc, dec, vocab, kdim, vdim;
  double dropout, eps;
};
TCfg read_tcfg(const Json &c) {
  TCfg t;
  t.d = c.at("num_features").as_int(); t.seq = c.at("sequence_length").as_int(); t.batch = c.at("batch_size").as_int();
  t.ffn = c.at("dim_feedforward").as_int(); t.heads = c.at("num_heads").as_int();
  t.enc = c.at("num_encoder_layers").as_int(); t.dec = c.at("num_decoder_layers").as_int();
  t.vocab = c.at("vocab_size").as_int(); t.dropout = c.at("dropout").as_float(); t.eps = c.at("layer_norm_eps").as_float();
  // the reference derives the per-head key/value width from dim_feedforward (transformer.cc:36-37)
  t.kdim = c.get_int("kdim", t.ffn / t.heads);
  t.vdim = c.get_int("vdim", t.ffn / t.heads);
  return t;
}
V maybe_dropout(GraphBuilder &b, V x, double p) { return p > 0 ? b.dropout(x, p) : x; }
V ffn(GraphBuilder &b, const TCfg &c, V x, const std::string &act, const std::string &p, const OptInit &wi = std::nullopt,
      const OptInit &bi = std::nullopt) {
  V h = b.dense(x, c.ffn, act, true, wi, bi, p + "ffn1");
  h = maybe_dropout(b, h, c.dropout);
  h = b.dense(h, c.d, std::nullopt, true, wi, bi, p + "ffn2");
  return maybe_dropout(b, h, c.dropout);
}
V encoder_layer(GraphBuilder &b, const TCfg &c, V x, const std::string &p) {
  V a = b.multihead_attention(x, x, x, c.d, c.heads, c.kdim, c.vdim, c.dropout, false, false, false, std::nullopt, p + "attn");
  V n = b.layer_norm(b.add(a, x), {-1}, true, c.eps, p + "ln1");
  V f = ffn(b, c, n, "RELU", p);
  return b.layer_norm(b.add(n, f), {-1}, true, c.eps, p + "ln2");
}
V decoder_layer(GraphBuilder &b, const TCfg &c, V x, std::optional<V> enc, const std::string &p) {
  V a = b.multihead_attention(x, x, x, c.d, c.heads, c.kdim, c.vdim, c.dropout, false, false, false, std::nullopt, p + "self_attn");
  V n = b.layer_norm(b.add(x, a), {-1}, true, c.eps, p + "ln1");
  if (enc) {
    V m = b.multihead_attention(n, *enc, *enc, c.d, c.heads, c.kdim, c.vdim, c.dropout, false, false, false, std::nullopt, p + "cross_attn");
    n = b.layer_norm(b.add(n, m), {-1}, true, c.eps, p + "ln2");
  }
  V f = ffn(b, c, n, "RELU", p);
  return b.layer_norm(b.add(n, f), {-1}, true, c.eps, p + "ln3");
}
}  // namespace

Graph build_transformer(const Json &user) {
  Json cfg = cfg_defaults(user, default_transformer_config());
  TCfg c = read_tcfg(cfg);
  GraphBuilder b;
  V input = b.create_input({c.batch, c.seq, c.d}, DataType::FLOAT, true, "input");
  V target = b.create_input({c.batch, c.seq, c.d}, DataType::FLOAT, true, "target");
  V e = input;
  for (int i = 0; i < c.enc; ++i) e = encoder_layer(b, c, e, "enc" + std::to_string(i) + ".");
  V d = target;
  for (int i = 0; i < c.dec; ++i) d = decoder_layer(b, c, d, e, "dec" + std::to_string(i) + ".");
  b.softmax(b.dense(d, c.vocab, "RELU", true, std::nullopt, std::nullopt, "lm_head"), -1, "out_prob");
  return b.graph;
}

// Decoder-only language model on token ids: embedding -> N x (self-attention, FFN; post-LN as in the
// encoder-decoder builder above) -> vocabulary projection -> softmax.  Head width is d_model / heads.
Json default_transformer_lm_config() {
  Json c = Json::object();
  c["num_features"] = 2048; c["sequence_length"] = 1024; c["batch_size"] = 32; c["dim_feedforward"] = 8192;
  c["num_heads"] = 16; c["num_encoder_layers"] = 0; c["num_decoder_layers"] = 24; c["dropout"] = 0.1;
  c["layer_norm_eps"] = 1e-5; c["vocab_size"] = 32000; c["init_std"] = 0.02; c["data_type"] = "FLOAT";
  return c;
}
Graph build_transformer_lm(const Json &user) {
  Json cfg = cfg_defaults(user, default_transformer_lm_config());
  if (!cfg.contains("kdim")) cfg["kdim"] = cfg.at("num_features").as_int() / cfg.at("num_heads").as_int();
  if (!cfg.contains("vdim")) cfg["vdim"] = cfg.at("kdim");
  TCfg c = read_tcfg(cfg);
  double std = cfg.get_float("init_std", 0.02);
  DataType dt = datatype_from_string(cfg.get_string("data_type", "FLOAT"));
  GraphBuilder b;
  V ids = b.create_input({c.batch, c.seq, 1}, DataType::INT32, false, "input_ids");
  V x = b.embedding(ids, c.vocab, c.d, "SUM", dt, normal_init(std), "tok_emb");
  for (int i = 0; i < c.dec; ++i) {
    std::string p = "layer" + std::to_string(i) + ".";
    V a = b.multihead_attention(x, x, x, c.d, c.heads, c.kdim, c.vdim, c.dropout, false, false, false, normal_init(std), p + "attn");
    V n = b.layer_norm(b.add(x, a), {-1}, true, c.eps, p + "ln1");
    V f = ffn(b, c, n, "RELU", p, normal_init(std), zero_init());
    x = b.layer_norm(b.add(n, f), {-1}, true, c.eps, p + "ln2");
  }
  V logits = b.dense(x, c.vocab, std::nullopt, false, normal_init(std), std::nullopt, "lm_head");
  b.softmax(logits, -1, "out_prob");
  return b.graph;
}

// ---------------------------------------------------------------- BERT
Json default_bert_config() {
  Json c = Json::object();
  c["vocab_size"] = 30522; c["hidden_size"] = 768; c["num_encoder_layers"] = 12; c["num_heads"] = 12;
  c["dim_feedforward"] = 3072; c["hidden_act"] = "GELU"; c["hidden_dropout_prob"] = 0.1;
  c["attention_probs_dropout_prob"] = 0.1; c["initializer_range"] = 0.02; c["layer_norm_eps"] = 1e-12;
  c["position_embedding_type"] = "absolute"; c["classifier_dropout"] = 0.1; c["sequence_length"] = 512;
  c["batch_size"] = 64; c["token_ids"] = false;
  return c;
}
Graph build_bert(const Json &user) {
  Json cfg = cfg_defaults(user, default_bert_config());
  if (cfg.at("position_embedding_type").as_string() != "absolute")
    throw Error("bert: only position_embedding_type=absolute is supported");
  int64_t hidden = cfg.at("hidden_size").as_int(), heads = cfg.at("num_heads").as_int(), ffn_dim = cfg.at("dim_feedforward").as_int();
  int64_t batch = cfg.at("batch_size").as_int(), seq = cfg.at("sequence_length").as_int(), vocab = cfg.at("vocab_size").as_int();
  double pdrop = cfg.at("hidden_dropout_prob").as_float(), adrop = cfg.at("attention_probs_dropout_prob").as_float();
  double eps = cfg.at("layer_norm_eps").as_float();
  std::string act = cfg.at("hidden_act").as_string();
  bool token_ids = cfg.get_bool("token_ids", false);
  // lib/models/src/models/bert/bert.cc:66-67 takes the head width from dim_feedforward; the token-id
  // variant uses the usual hidden / heads.
  int64_t kdim = cfg.get_int("kdim", token_ids ? hidden / heads : ffn_dim / heads);
  Json winit = truncated_normal_init(cfg.at("initializer_range").as_float());
  Json binit = zero_init();
  GraphBuilder b;
  V x;
  if (token_ids) {
    V ids = b.create_input({batch, seq, 1}, DataType::INT32, false, "input_ids");
    V pos = b.create_input({batch, seq, 1}, DataType::INT32, false, "position_ids");
    V we = b.embedding(ids, vocab, hidden, "SUM", DataType::FLOAT, winit, "word_emb");
    V pe = b.embedding(pos, cfg.get_int("max_position_embeddings", 512), hidden, "SUM", DataType::FLOAT, winit, "pos_emb");
    x = b.layer_norm(b.add(we, pe), {-1}, true, eps, "emb_ln");
    if (pdrop > 0) x = b.dropout(x, pdrop);
  } else {
    x = b.create_input({batch, seq, hidden}, DataType::FLOAT, true, "input");
  }
  for (int i = 0; i < cfg.at("num_encoder_layers").as_int(); ++i) {
    std::string p = "layer" + std::to_string(i) + ".";
    V a = b.multihead_attention(x, x, x, hidden, heads, kdim, kdim, adrop, true, false, false, winit, p + "attn");
    V n = b.layer_norm(b.add(a, x), {-1}, true, eps, p + "ln1");
    V h = b.dense(n, ffn_dim, act, true, winit, binit, p + "ffn1");
    if (pdrop > 0) h = b.dropout(h, pdrop);
    h = b.dense(h, hidden, std::nullopt, true, winit, binit, p + "ffn2");
    if (pdrop > 0) h = b.dropout(h, pdrop);
    x = b.layer_norm(b.add(n, h), {-1}, true, eps, p + "ln2");
  }
  std::optional<std::string> head_act = token_ids ? std::nullopt : std::optional<std::string>(act);
  b.softmax(b.dense(x, vocab, head_act, true, winit, binit, "lm_head"), -1, "out_prob");
  return b.graph;
}

// ---------------------------------------------------------------- Inception-v3
Json default_inception_v3_config() {
  Json c = Json::object();
  c["num_classes"] = 1000; c["batch_size"] = 32; c["aux_logits"] = true;
  return c;
}
namespace {
V conv_block(GraphBuilder &b, V x, int64_t filters, int kh, int kw, int sh = 1, int sw = 1, int ph = 0, int pw = 0) {
  V c = b.conv2d(x, filters, kh, kw, sh, sw, ph, pw, std::nullopt, 1, false);
  return b.batch_norm(c, true, std::string("RELU"), 1e-3, 0.1);
}
V module_a(GraphBuilder &b, V x, int64_t pool_features) {
  V b1 = conv_block(b, x, 64, 1, 1);
  V b5 = conv_block(b, conv_block(b, x, 48, 1, 1), 64, 5, 5, 1, 1, 2, 2);
  V b3 = conv_block(b, x, 64, 1, 1);
  b3 = conv_block(b, b3, 96, 3, 3, 1, 1, 1, 1);
  b3 = conv_block(b, b3, 96, 3, 3, 1, 1, 1, 1);
  V bp = conv_block(b, b.pool2d(x, 3, 3, 1, 1, 1, 1, "AVG"), pool_features, 1, 1);
  return b.concat({b1, b5, b3, bp}, 1);
}
V module_b(GraphBuilder &b, V x) {
  V b3 = conv_block(b, x, 384, 3, 3, 2, 2);
  V d = conv_block(b, x, 64, 1, 1);
  d = conv_block(b, d, 96, 3, 3, 1, 1, 1, 1);
  d = conv_block(b, d, 96, 3, 3, 2, 2);
  V bp = b.pool2d(x, 3, 3, 2, 2, 0, 0, "MAX");
  return b.concat({b3, d, bp}, 1);
}
V module_c(GraphBuilder &b, V x, int64_t c7) {
  V b1 = conv_block(b, x, 192, 1, 1);
  V s = conv_block(b, x, c7, 1, 1);
  s = conv_block(b, s, c7, 1, 7, 1, 1, 0, 3);
  s = conv_block(b, s, 192, 7, 1, 1, 1, 3, 0);
  V d = conv_block(b, x, c7, 1, 1);
  d = conv_block(b, d, c7, 7, 1, 1, 1, 3, 0);
  d = conv_block(b, d, c7, 1, 7, 1, 1, 0, 3);
  d = conv_block(b, d, c7, 7, 1, 1, 1, 3, 0);
  d = conv_block(b, d, 192, 1, 7, 1, 1, 0, 3);
  V bp = conv_block(b, b.pool2d(x, 3, 3, 1, 1, 1, 1, "AVG"), 192, 1, 1);
  return b.concat({b1, s, d, bp}, 1);
}
V module_d(GraphBuilder &b, V x) {
  V b3 = conv_block(b, conv_block(b, x, 192, 1, 1), 320, 3, 3, 2, 2);
  V s = conv_block(b, x, 192, 1, 1);
  s = conv_block(b, s, 192, 1, 7, 1, 1, 0, 3);
  s = conv_block(b, s, 192, 7, 1, 1, 1, 3, 0);
  s = conv_block(b, s, 192, 3, 3, 2, 2);
  V bp = b.pool2d(x, 3, 3, 2, 2, 0, 0, "MAX");
  return b.concat({b3, s, bp}, 1);
}
V module_e(GraphBuilder &b, V x) {
  V b1 = conv_block(b, x, 320, 1, 1);
  V t = conv_block(b, x, 384, 1, 1);
  V b3 = b.concat({conv_block(b, t, 384, 1, 3, 1, 1, 0, 1), conv_block(b, t, 384, 3, 1, 1, 1, 1, 0)}, 1);
  V d = conv_block(b, x, 448, 1, 1);
  d = conv_block(b, d, 384, 3, 3, 1, 1, 1, 1);
  V bd = b.concat({conv_block(b, d, 384, 1, 3, 1, 1, 0, 1), conv_block(b, d, 384, 3, 1, 1, 1, 1, 0)}, 1);
  V bp = conv_block(b, b.pool2d(x, 3, 3, 1, 1, 1, 1, "AVG"), 192, 1, 1);
  return b.concat({b1, b3, bd, bp}, 1);
}
}  // namespace

Graph build_inception_v3(const Json &user) {
  Json cfg = cfg_defaults(user, default_inception_v3_config());
  int64_t batch = cfg.at("batch_size").as_int(), classes = cfg.at("num_classes").as_int();
  GraphBuilder b;
  V x = b.create_input({batch, 3, 299, 299}, DataType::FLOAT, true, "input");
  x = conv_block(b, x, 32, 3, 3, 2, 2);
  x = conv_block(b, x, 32, 3, 3);
  x = conv_block(b, x, 64, 3, 3, 1, 1, 1, 1);
  x = b.pool2d(x, 3, 3, 2, 2, 0, 0, "MAX");
  x = conv_block(b, x, 80, 1, 1);
  x = conv_block(b, x, 192, 3, 3);
  x = b.pool2d(x, 3, 3, 2, 2, 0, 0, "MAX");
  x = module_a(b, x, 32);
  x = module_a(b, x, 64);
  x = module_a(b, x, 64);
  x = module_b(b, x);
  x = module_c(b, x, 128);
  x = module_c(b, x, 160);
  x = module_c(b, x, 160);
  x = module_c(b, x, 192);
  if (cfg.get_bool("aux_logits", true)) {
    V a = b.pool2d(x, 5, 5, 3, 3, 0, 0, "AVG");
    a = conv_block(b, a, 128, 1, 1);
    a = conv_block(b, a, 768, 5, 5);
    a = b.adaptive_pool2d(a, 1, 1);
    a = b.flat(a, 1, -1);
    b.dense(a, classes, std::nullopt, true, std::nullopt, std::nullopt, "aux_logits");
  }
  x = module_d(b, x);
  x = module_e(b, x);
  x = module_e(b, x);
  x = b.pool2d(x, 8, 8, 1, 1, 0, 0, "AVG");
  x = b.dropout(x, 0.5);
  x = b.flat(x, 1, -1);
  x = b.dense(x, classes, std::nullopt, true, std::nullopt, std::nullopt, "fc");
  b.softmax(x, -1, "out_prob");
  return b.graph;
}

// ---------------------------------------------------------------- DLRM
Json default_dlrm_config() {
  Json c = Json::object();
  c["embedding_dim"] = 64; c["embedding_bag_size"] = 1;
  c["embedding_size"] = Json::from_ints(std::vector<int64_t>{1000000, 1000000, 1000000, 1000000});
  c["dense_arch_layer_sizes"] = Json::from_ints(std::vector<int64_t>{4, 64, 64});
  c["over_arch_layer_sizes"] = Json::from_ints(std::vector<int64_t>{64, 64, 2});
  c["arch_interaction_op"] = "CAT"; c["batch_size"] = 64; c["seed"] = 0;
  c["embedding_data_type"] = "HALF"; c["final_activation"] = "RELU";
  return c;
}
// concat is limited to 8 numbered input slots (INPUT_0..INPUT_7): longer lists are concatenated in stages
static V concat_many(GraphBuilder &b, std::vector<V> xs, int axis) {
  while (xs.size() > 8) {
    std::vector<V> head(xs.begin(), xs.begin() + 8);
    V c = b.concat(head, axis);
    xs.erase(xs.begin(), xs.begin() + 8);
    xs.insert(xs.begin(), c);
  }
  return xs.size() == 1 ? xs[0] : b.concat(xs, axis);
}
static V dlrm_mlp(GraphBuilder &b, V x, const std::vector<long long> &sizes, long long seed, const std::string &p,
                  const std::string &last_act) {
  for (size_t i = 0; i + 1 < sizes.size(); ++i) {
    Json wi = normal_init(std::sqrt(2.0 / (double)(sizes[i + 1] + sizes[i])), seed);
    Json bi = normal_init(std::sqrt(2.0 / (double)sizes[i + 1]), seed);
    std::string act = (i + 2 == sizes.size()) ? last_act : "RELU";
    std::optional<std::string> a = act.empty() ? std::nullopt : std::optional<std::string>(act);
    x = b.dense(x, sizes[i + 1], a, true, wi, bi, p + std::to_string(i));
  }
  return x;
}
Graph build_dlrm(const Json &user) {
  Json cfg = cfg_defaults(user, default_dlrm_config());
  int64_t batch = cfg.at("batch_size").as_int(), dim = cfg.at("embedding_dim").as_int(), bag = cfg.at("embedding_bag_size").as_int();
  auto tables = cfg.at("embedding_size").as_ints();
  auto bottom = cfg.at("dense_arch_layer_sizes").as_ints();
  auto top = cfg.at("over_arch_layer_sizes").as_ints();
  long long seed = cfg.get_int("seed", 0);
  std::string inter = cfg.at("arch_interaction_op").as_string();
  DataType edt = datatype_from_string(cfg.get_string("embedding_data_type", "HALF"));
  GraphBuilder b;
  std::vector<V> sparse;
  for (size_t i = 0; i < tables.size(); ++i)
    sparse.push_back(b.create_input({batch, bag}, DataType::INT64, false, "sparse" + std::to_string(i)));
  V dense_in = b.create_input({batch, bottom.front()}, DataType::FLOAT, true, "dense");
  V bot = dlrm_mlp(b, dense_in, bottom, seed, "bottom", "RELU");
  std::vector<V> embs;
  for (size_t i = 0; i < tables.size(); ++i) {
    double range = std::sqrt(1.0 / (double)tables[i]);
    Json init = cfg.contains("embedding_init_range")
                    ? uniform_init(-cfg.at("embedding_init_range").as_float(), cfg.at("embedding_init_range").as_float(), seed)
                    : uniform_init(-range, range, seed);
    V e = b.embedding(sparse[i], tables[i], dim, "SUM", edt, init, "emb" + std::to_string(i));
    if (edt != DataType::FLOAT) e = b.cast(e, DataType::FLOAT);
    embs.push_back(e);
  }
  V feat;
  if (inter == "CAT") {
    std::vector<V> all{bot};
    all.insert(all.end(), embs.begin(), embs.end());
    feat = concat_many(b, all, 1);
  } else if (inter == "DOT") {
    // pairwise dot products of the (1 + #tables) feature vectors, concatenated with the dense feature
    if (bottom.back() != dim) throw Error("dlrm: DOT interaction needs bottom MLP width == embedding_dim");
    // the lookups are stacked on their own first, so that a strategy can keep that stack table-parallel and hand
    // it to the sample-parallel rest of the model in one all-to-all
    std::vector<V> rows;
    for (auto &e : embs) rows.push_back(b.reshape(e, {batch, 1, dim}));
    V stack = rows.size() > 1 ? concat_many(b, rows, 1) : rows[0];
    V x = b.concat({b.reshape(bot, {batch, 1, dim}), stack}, 1);  // [batch, F, dim]
    V xt = b.transpose(x, {0, 2, 1});              // [batch, dim, F]
    V z = b.batch_matmul(x, xt);                   // [batch, F, F]
    V zf = b.flat(z, 1, -1);
    feat = b.concat({bot, zf}, 1);
  } else throw Error("dlrm: arch_interaction_op must be CAT or DOT");
  std::vector<long long> top_sizes;
  top_sizes.push_back(b.shape(feat).dims[1].size);
  // as in the reference, the first entry of over_arch_layer_sizes is the nominal input width and only
  // the following entries create layers (dlrm.cc:44-66)
  size_t start = 1;
  for (size_t i = start; i < top.size(); ++i) top_sizes.push_back(top[i]);
  dlrm_mlp(b, feat, top_sizes, seed, "top", cfg.get_string("final_activation", "RELU"));
  return b.graph;
}

// ---------------------------------------------------------------- CANDLE-Uno
Json default_candle_uno_config() {
  Json c = Json::object();
  c["batch_size"] = 64;
  c["dense_layers"] = Json::from_ints(std::vector<int64_t>(4, 4192));
  c["dense_feature_layers"] = Json::from_ints(std::vector<int64_t>(8, 4192));
  Json fs = Json::object();
  fs["dose"] = 1; fs["cell.rnaseq"] = 942; fs["drug.descriptors"] = 5270; fs["drug.fingerprints"] = 2048;
  c["feature_shapes"] = fs;
  Json inf = Json::object();
  inf["dose1"] = "dose"; inf["dose2"] = "dose"; inf["cell.rnaseq"] = "cell.rnaseq";
  inf["drug1.descriptors"] = "drug.descriptors"; inf["drug1.fingerprints"] = "drug.fingerprints";
  inf["drug2.descriptors"] = "drug.descriptors"; inf["drug2.fingerprints"] = "drug.fingerprints";
  c["input_features"] = inf;
  c["dropout"] = 0.1; c["residual"] = false;
  return c;
}
Graph build_candle_uno(const Json &user) {
  Json cfg = cfg_defaults(user, default_candle_uno_config());
  int64_t batch = cfg.at("batch_size").as_int();
  double dropout = cfg.at("dropout").as_float();
  bool residual = cfg.at("residual").as_bool();
  Json ki = glorot_normal_init();
  GraphBuilder b;
  std::vector<V> encoded;
  for (auto &kv : cfg.at("input_features").fields()) {
    std::string fname = kv.second.as_string();
    int64_t width = cfg.at("feature_shapes").at(fname).as_int();
    V in = b.create_input({batch, width}, DataType::FLOAT, true, kv.first);
    std::string base = fname.substr(0, fname.find('.'));
    bool has_model = fname.find('.') != std::string::npos && (base == "cell" || base == "drug");
    if (has_model) {
      V t = in;
      for (auto dd : cfg.at("dense_feature_layers").as_ints()) {
        t = b.dense(t, dd, std::string("RELU"), false, ki);
        if (dropout > 0) t = b.dropout(t, dropout);
      }
      encoded.push_back(t);
    } else encoded.push_back(in);
  }
  V out = b.concat(encoded, 1);
  for (auto dd : cfg.at("dense_layers").as_ints()) {
    V res = out;
    out = b.dense(out, dd, std::string("RELU"), false, ki);
    if (dropout > 0) out = b.dropout(out, dropout);
    if (residual && b.shape(res).sizes() == b.shape(out).sizes()) out = b.add(out, res);
  }
  b.dense(out, 1, std::nullopt, false, ki, std::nullopt, "regression_head");
  return b.graph;
}

// ---------------------------------------------------------------- split_test, MLP, single operator
Graph build_split_test(const Json &user) {
  int64_t batch = user.is_object() ? user.get_int("batch_size", 8) : 8;
  GraphBuilder b;
  V t = b.create_input({batch, 256}, DataType::FLOAT, true, "input");
  t = b.relu(b.dense(t, 128));
  t = b.relu(b.add(b.dense(t, 64), b.dense(t, 64)));
  t = b.relu(b.add(b.dense(t, 32), b.dense(t, 32)));
  b.softmax(t);
  return b.graph;
}
Graph build_mlp(const Json &user) {
  Json cfg = cfg_defaults(user, Json::object());
  int64_t batch = cfg.get_int("batch_size", 64), in_dim = cfg.get_int("input_dim", 784);
  std::vector<long long> hidden = cfg.contains("hidden") ? cfg.at("hidden").as_ints() : std::vector<long long>{512, 512};
  int64_t classes = cfg.get_int("num_classes", 10);
  GraphBuilder b;
  V t = b.create_input({batch, in_dim}, DataType::FLOAT, true, "input");
  int i = 0;
  for (auto h : hidden) t = b.dense(t, h, std::string("RELU"), true, std::nullopt, std::nullopt, "fc" + std::to_string(i++));
  t = b.dense(t, classes, std::nullopt, true, std::nullopt, std::nullopt, "logits");
  b.softmax(t, -1, "out_prob");
  return b.graph;
}
Graph build_single_operator(const Json &) {
  // bin/export-model-arch "single_operator": one dense layer
  GraphBuilder b;
  V t = b.create_input({8, 16}, DataType::FLOAT, true, "input");
  b.dense(t, 32);
  return b.graph;
}

std::vector<std::string> model_names() {
  return {"transformer", "transformer_lm", "bert", "inception_v3", "dlrm", "candle_uno", "split_test", "mlp", "single_operator"};
}
Json default_model_config(const std::string &name) {
  if (name == "transformer") return default_transformer_config();
  if (name == "transformer_lm") return default_transformer_lm_config();
  if (name == "bert") return default_bert_config();
  if (name == "inception_v3") return default_inception_v3_config();
  if (name == "dlrm") return default_dlrm_config();
  if (name == "candle_uno") return default_candle_uno_config();
  return Json::object();
}
Graph build_model(const std::string &name, const Json &cfg) {
  if (name == "transformer") return build_transformer(cfg);
  if (name == "transformer_lm") return build_transformer_lm(cfg);
  if (name == "bert") return build_bert(cfg);
  if (name == "inception_v3") return build_inception_v3(cfg);
  if (name == "dlrm") return build_dlrm(cfg);
  if (name == "candle_uno") return build_candle_uno(cfg);
  if (name == "split_test") return build_split_test(cfg);
  if (name == "mlp") return build_mlp(cfg);
  if (name == "single_operator") return build_single_operator(cfg);
  throw Error("unknown model '" + name + "'");
}

}  // namespace ff
