// Runs the reference's own host sampler (src/engine/host_sampling.cc, unmodified) over a
// few logits rows and prints what it chose, one JSON object a row: the greedy token after
// penalties and masks, its log-probability and the most probable alternatives.
// make_golden.sh compiles this against the reference's sources; the output is committed as
// sampling_golden.jsonl, and tests/test_scheduler_golden.py compares the plain statements
// of tests/plain_qwen2_moe.py (penalised, greedy, logprobs) with it.
//
// Rows are made by a formula (no generator state): x[v] = 4 sin(0.37 v + 1.3 r) +
// 2 cos(0.11 v r + 0.5), with a few equal entries put in to exercise ties.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <vector>

#include "inferx/engine/host_sampling.h"
#include "inferx/model/forward_batch.h"

using inferx::engine::HostSampleRow;
using inferx::engine::SampledLogprob;
using inferx::model::ForwardBatch;

int main() {
  const int64_t kVocab = 211;
  struct Case {
    float presence, frequency, repetition;
    std::vector<int32_t> hist_ids, hist_counts, mask;
    int32_t logprobs_k;
  };
  const std::vector<Case> cases = {
      {0.f, 0.f, 1.f, {}, {}, {}, 0},
      {0.f, 0.f, 1.f, {}, {}, {}, 5},
      {0.6f, 0.f, 1.f, {17, 4, 99}, {1, 2, 1}, {}, 3},
      {0.f, 0.45f, 1.f, {17, 4, 99, 210}, {3, 1, 7, 2}, {}, 4},
      {0.f, 0.f, 1.7f, {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11}, {1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1}, {}, 2},
      {-0.5f, 0.25f, 0.6f, {17, 44, 45, 46, 120, 121}, {2, 2, 1, 1, 5, 1}, {}, 20},
      {0.f, 0.f, 1.f, {}, {}, {3, 17, 18, 19}, 6},
      {1.5f, 1.0f, 2.0f, {3, 17, 18, 19, 20}, {1, 1, 4, 1, 1}, {17, 18, 200}, 8},
      {0.3f, 0.f, 1.f, {500, -1, 17}, {1, 0, 1}, {-1, 900}, -1},   // ids past the vocabulary, padding
  };
  for (size_t r = 0; r < cases.size(); ++r) {
    const Case& c = cases[r];
    std::vector<float> row(kVocab);
    for (int64_t v = 0; v < kVocab; ++v)
      row[v] = 4.0f * std::sin(0.37f * v + 1.3f * r) + 2.0f * std::cos(0.11f * v * r + 0.5f);
    row[18] = row[17];                 // ties
    row[120] = row[121] = row[44];
    ForwardBatch batch;
    const size_t hist = static_cast<size_t>(ForwardBatch::kPenaltyHistoryCap);
    const size_t mask = static_cast<size_t>(ForwardBatch::kMaskCap);
    batch.temperature = {0.0f};
    batch.top_p = {1.0f};
    batch.top_k = {0};
    batch.min_p = {0.0f};
    batch.seeds = {0};
    batch.presence_penalty = {c.presence};
    batch.frequency_penalty = {c.frequency};
    batch.repetition_penalty = {c.repetition};
    batch.penalty_history_ids.assign(hist, -1);
    batch.penalty_history_counts.assign(hist, 0);
    for (size_t j = 0; j < c.hist_ids.size(); ++j) {
      batch.penalty_history_ids[j] = c.hist_ids[j];
      batch.penalty_history_counts[j] = c.hist_counts[j];
    }
    batch.mask_token_ids.assign(mask, -1);
    for (size_t j = 0; j < c.mask.size(); ++j) batch.mask_token_ids[j] = c.mask[j];
    batch.logprobs_k = {c.logprobs_k};
    std::vector<float> before = row;
    SampledLogprob lp;
    const int32_t chosen = HostSampleRow(row.data(), kVocab, batch, 0, &lp);
    std::printf("{\"row\": %zu, \"vocab\": %lld, \"presence\": %.9g, \"frequency\": %.9g, "
                "\"repetition\": %.9g, \"history\": [", r, (long long)kVocab, c.presence,
                c.frequency, c.repetition);
    for (size_t j = 0; j < c.hist_ids.size(); ++j)
      std::printf("%s[%d, %d]", j ? ", " : "", c.hist_ids[j], c.hist_counts[j]);
    std::printf("], \"mask\": [");
    for (size_t j = 0; j < c.mask.size(); ++j) std::printf("%s%d", j ? ", " : "", c.mask[j]);
    std::printf("], \"logprobs_k\": %d, \"chosen\": %d, \"has_logprob\": %s, \"logprob\": %.9g, "
                "\"top\": [", c.logprobs_k, chosen, lp.present ? "true" : "false", lp.logprob);
    for (size_t j = 0; j < lp.top.size(); ++j)
      std::printf("%s[%d, %.9g]", j ? ", " : "", lp.top[j].first, lp.top[j].second);
    // the logits after penalties and masks, where they differ from before (-1e30 for -inf)
    std::printf("], \"changed\": [");
    bool first = true;
    for (int64_t v = 0; v < kVocab; ++v) {
      if (row[v] == before[v]) continue;
      std::printf("%s[%lld, %.9g]", first ? "" : ", ", (long long)v,
                  std::isinf(row[v]) ? -1e30 : row[v]);
      first = false;
    }
    std::printf("]}\n");
  }
  return 0;
}
