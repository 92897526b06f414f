// Parses the config.json texts under config_cases/ with the reference's own parser
// (src/model/config.cc, unmodified) and prints what it read, one JSON object a file.
// make_golden.sh compiles this against the reference's sources; the output is committed as
// config_golden.jsonl, and tests/test_scheduler_golden.py compares this repository's typed
// configuration with it, key by key, and names the keys where the two differ on purpose.
#include <cstdio>
#include <fstream>
#include <sstream>
#include <string>

#include "inferx/model/config.h"

int main(int argc, char** argv) {
  for (int i = 1; i < argc; ++i) {
    std::ifstream in(argv[i]);
    std::stringstream text;
    text << in.rdbuf();
    std::string name = argv[i];
    name = name.substr(name.find_last_of('/') + 1);
    name = name.substr(0, name.find_last_of('.'));
    auto cfg = inferx::model::ModelConfig::FromJson(text.str());
    if (!cfg.ok()) {
      std::printf("{\"case\": \"%s\", \"ok\": false, \"error\": \"%s\"}\n", name.c_str(),
                  cfg.status().ToString().c_str());
      continue;
    }
    const auto& c = *cfg;
    std::printf("{\"case\": \"%s\", \"ok\": true, \"architecture\": \"%s\", \"hidden_size\": %lld, "
                "\"intermediate_size\": %lld, \"num_hidden_layers\": %lld, "
                "\"num_attention_heads\": %lld, \"num_key_value_heads\": %lld, \"head_dim\": %lld, "
                "\"vocab_size\": %lld, \"max_position_embeddings\": %lld, \"rms_norm_eps\": %.17g, "
                "\"rope_theta\": %.17g, \"tie_word_embeddings\": %s, \"attention_bias\": %s, "
                "\"num_experts\": %lld, \"num_experts_per_tok\": %lld, "
                "\"moe_intermediate_size\": %lld, \"norm_topk_prob\": %s, "
                "\"shared_expert_intermediate_size\": %lld, \"routed_scaling_factor\": %.17g, "
                "\"sliding_window\": %lld, \"layer_is_sliding\": [",
                name.c_str(), inferx::model::ArchitectureName(c.architecture),
                (long long)c.hidden_size, (long long)c.intermediate_size,
                (long long)c.num_hidden_layers, (long long)c.num_attention_heads,
                (long long)c.num_key_value_heads, (long long)c.head_dim, (long long)c.vocab_size,
                (long long)c.max_position_embeddings, c.rms_norm_eps, c.rope_theta,
                c.tie_word_embeddings ? "true" : "false", c.attention_bias ? "true" : "false",
                (long long)c.num_experts, (long long)c.num_experts_per_tok,
                (long long)c.moe_intermediate_size, c.norm_topk_prob ? "true" : "false",
                (long long)c.shared_expert_intermediate_size, c.routed_scaling_factor,
                (long long)c.sliding_window);
    for (size_t l = 0; l < c.layer_is_sliding.size(); ++l)
      std::printf("%s%s", l ? ", " : "", c.layer_is_sliding[l] ? "true" : "false");
    std::printf("], \"moe_layers\": [");
    for (long long l = 0; l < c.num_hidden_layers; ++l)
      std::printf("%s%s", l ? ", " : "", c.IsMoeLayer(l) ? "true" : "false");
    std::printf("]}\n");
  }
  return 0;
}
