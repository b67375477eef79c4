// models.h -- model zoo entry points (lib/models of the reference).
#pragma once
#include <string>
#include <vector>

#include "builder.h"

namespace ff {
Json default_transformer_config();
Json default_transformer_lm_config();
Json default_bert_config();
Json default_inception_v3_config();
Json default_dlrm_config();
Json default_candle_uno_config();
Graph build_transformer(const Json &cfg);
Graph build_transformer_lm(const Json &cfg);
Graph build_bert(const Json &cfg);
Graph build_inception_v3(const Json &cfg);
Graph build_dlrm(const Json &cfg);
Graph build_candle_uno(const Json &cfg);
Graph build_split_test(const Json &cfg);
Graph build_mlp(const Json &cfg);
Graph build_single_operator(const Json &cfg);
std::vector<std::string> model_names();
Json default_model_config(const std::string &name);
Graph build_model(const std::string &name, const Json &cfg);
}  // namespace ff
