// Drives the reference's own scheduler (src/scheduler/scheduler.cc, unmodified, over a
// host-allocated block pool as its unit tests do, tests/unit/scheduler_test.cc:28-37)
// through a scripted scenario and prints what it decided, one JSON object a step.
// make_golden.sh compiles this against the reference's sources; the output is committed as
// scheduler_golden.jsonl, and tests/test_scheduler_golden.py replays the same scenario
// through this repository's scheduler and compares the decisions.
//
// The "model" is a formula: the token sampled after a row is
//   (last input token * 31 + its position * 17) % 97 + 3,
// which both sides can compute from the batch alone.
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "inferx/core/kv_cache.h"
#include "inferx/model/forward_batch.h"
#include "inferx/scheduler/scheduler.h"

using inferx::DataType;
using inferx::DeviceId;
using inferx::KvBlockPool;
using inferx::KvLayout;
using inferx::model::ForwardBatch;
using namespace inferx::scheduler;

namespace {

struct Arrival {
  int step;
  int64_t id;
  std::vector<int32_t> prompt;
  SamplingParams params;
};

std::vector<int32_t> Prompt(int n, int salt) {
  std::vector<int32_t> p;
  for (int i = 0; i < n; ++i) p.push_back((salt * 37 + i * 11) % 89 + 5);
  return p;
}

void PrintInts(const char* key, const std::vector<int32_t>& v, size_t from, size_t n) {
  std::printf("\"%s\": [", key);
  bool first = true;
  for (size_t i = from; i < from + n && i < v.size(); ++i) {
    if (v[i] < 0) continue;                    // padding
    std::printf("%s%d", first ? "" : ", ", v[i]);
    first = false;
  }
  std::printf("]");
}

}  // namespace

int main() {
  KvLayout layout;
  layout.entries_per_token = 2;
  layout.kv_heads = 1;
  layout.head_dim = 8;
  layout.dtype = DataType::kBFloat16;
  const int64_t kBlocks = 12, kBlockSize = 4;
  auto pool_or = KvBlockPool::Create(1, kBlocks, kBlockSize, layout, DeviceId::Cpu());
  if (!pool_or.ok()) {
    std::fprintf(stderr, "pool: %s\n", pool_or.status().ToString().c_str());
    return 1;
  }
  KvBlockPool pool = *std::move(pool_or);
  SchedulerConfig config;
  config.max_running = 3;
  config.max_batch_tokens = 16;
  config.max_seq_len = 40;
  config.enable_prefix_cache = false;
  auto sched_or = Scheduler::Create(config, &pool);
  if (!sched_or.ok()) {
    std::fprintf(stderr, "scheduler: %s\n", sched_or.status().ToString().c_str());
    return 1;
  }
  Scheduler sched = *std::move(sched_or);

  std::vector<Arrival> arrivals;
  {
    SamplingParams p;
    p.max_tokens = 6;
    arrivals.push_back({0, 1, Prompt(9, 1), p});
    p = SamplingParams();
    p.max_tokens = 9;
    p.temperature = 0.7f;
    p.seed = 12345;
    p.top_k = 5;
    p.top_p = 0.9f;
    p.min_p = 0.05f;
    p.repetition_penalty = 1.3f;
    p.presence_penalty = 0.25f;
    arrivals.push_back({0, 2, Prompt(5, 2), p});
    p = SamplingParams();
    p.max_tokens = 5;
    p.frequency_penalty = 0.5f;
    p.want_logprobs = true;
    p.top_logprobs = 3;
    arrivals.push_back({0, 3, Prompt(20, 3), p});
    p = SamplingParams();
    p.max_tokens = 30;
    p.stop_tokens = {40, 41, 42, 43, 44, 45, 46, 47, 48, 49};
    p.min_tokens = 4;
    p.want_logprobs = true;
    p.top_logprobs = 40;                      // more than the cap of 20
    arrivals.push_back({3, 4, Prompt(3, 4), p});
    p = SamplingParams();
    p.max_tokens = 3;
    arrivals.push_back({5, 5, Prompt(7, 5), p});
    p = SamplingParams();
    p.max_tokens = 8;
    p.seed = 0xfedcba9876543210ULL;
    p.temperature = 1.0f;
    arrivals.push_back({8, 6, Prompt(12, 6), p});
    p = SamplingParams();
    p.max_tokens = 4;
    arrivals.push_back({8, 7, Prompt(45, 7), p});        // longer than max_seq_len
    p = SamplingParams();
    p.max_tokens = 50;                                    // runs into max_seq_len
    arrivals.push_back({10, 8, Prompt(30, 8), p});
    p = SamplingParams();
    p.max_tokens = 12;
    arrivals.push_back({11, 9, Prompt(14, 9), p});
  }
  const int kCancelStep = 14;
  const int64_t kCancelId = 9;

  for (int step = 0; step < 400; ++step) {
    for (const Arrival& a : arrivals) {
      if (a.step == step) {
        auto s = sched.AddRequest(a.id, a.prompt, a.params);
        if (!s.ok()) std::fprintf(stderr, "add %lld: %s\n", (long long)a.id, s.ToString().c_str());
      }
    }
    if (step == kCancelStep) sched.Cancel(kCancelId);
    bool more = false;
    for (const Arrival& a : arrivals) more = more || a.step > step;
    if (!sched.HasWork() && !more) break;
    ForwardBatch batch;
    auto s = sched.PrepareStep(&batch);
    std::printf("{\"step\": %d, \"prepare_ok\": %s, ", step, s.ok() ? "true" : "false");
    // one row per sequence in the batch: how many tokens, the first one's position, the last token
    std::printf("\"rows\": [");
    {
      int64_t t = 0;
      bool first = true;
      const int64_t n = static_cast<int64_t>(batch.token_ids.size());
      while (t < n) {
        int64_t e = t;
        while (e + 1 < n && batch.seq_of_token[e + 1] == batch.seq_of_token[t]) ++e;
        std::printf("%s[%lld, %d, %d, %d]", first ? "" : ", ", (long long)(e - t + 1),
                    batch.positions[t], batch.token_ids[e],
                    batch.seq_lens.empty() ? -1 : batch.seq_lens[batch.seq_of_token[t]]);
        first = false;
        t = e + 1;
      }
    }
    std::printf("], \"sampled_rows\": [");
    std::vector<int32_t> sampled;
    const size_t hist = static_cast<size_t>(ForwardBatch::kPenaltyHistoryCap);
    const size_t mask = static_cast<size_t>(ForwardBatch::kMaskCap);
    for (size_t i = 0; i < batch.logits_indices.size(); ++i) {
      const int32_t at = batch.logits_indices[i];
      const int32_t tok = (batch.token_ids[at] * 31 + batch.positions[at] * 17) % 97 + 3;
      sampled.push_back(tok);
      std::printf("%s{\"token_index\": %d, \"seed\": \"%llu\", \"temperature\": %.9g, "
                  "\"top_p\": %.9g, \"top_k\": %d, \"min_p\": %.9g, \"presence\": %.9g, "
                  "\"frequency\": %.9g, \"repetition\": %.9g, \"logprobs_k\": %d, ",
                  i ? ", " : "", at, (unsigned long long)batch.seeds[i], batch.temperature[i],
                  batch.top_p[i], batch.top_k[i], batch.min_p[i], batch.presence_penalty[i],
                  batch.frequency_penalty[i], batch.repetition_penalty[i], batch.logprobs_k[i]);
      PrintInts("history_ids", batch.penalty_history_ids, i * hist, hist);
      std::printf(", ");
      {
        std::printf("\"history_counts\": [");
        bool first = true;
        for (size_t j = 0; j < hist; ++j) {
          if (batch.penalty_history_ids[i * hist + j] < 0) continue;
          std::printf("%s%d", first ? "" : ", ", batch.penalty_history_counts[i * hist + j]);
          first = false;
        }
        std::printf("], ");
      }
      PrintInts("mask", batch.mask_token_ids, i * mask, mask);
      std::printf("}");
    }
    std::printf("], ");
    std::vector<TokenDelta> deltas;
    std::vector<StepLogprob> lps(sampled.size());
    for (size_t i = 0; i < lps.size(); ++i) {
      lps[i].present = batch.logprobs_k[i] >= 0;
      lps[i].logprob = -0.5f * static_cast<float>(i + 1);
    }
    auto c = sched.CommitStep(sampled, &deltas, &lps);
    std::printf("\"commit_ok\": %s, \"deltas\": [", c.ok() ? "true" : "false");
    for (size_t i = 0; i < deltas.size(); ++i)
      std::printf("%s[%lld, %d, \"%s\", %s]", i ? ", " : "", (long long)deltas[i].id,
                  deltas[i].token, FinishReasonName(deltas[i].finish),
                  deltas[i].has_logprob ? "true" : "false");
    std::printf("], \"completed\": [");
    auto done = sched.TakeCompleted();
    for (size_t i = 0; i < done.size(); ++i)
      std::printf("%s[%lld, \"%s\", %zu]", i ? ", " : "", (long long)done[i].id,
                  FinishReasonName(done[i].reason), done[i].output_tokens.size());
    std::printf("], \"running\": %lld, \"waiting\": %lld, \"preemptions\": %lld, "
                "\"free_blocks\": %lld}\n",
                (long long)sched.num_running(), (long long)sched.num_waiting(),
                (long long)sched.preemptions(), (long long)pool.free_blocks());
  }
  return 0;
}
