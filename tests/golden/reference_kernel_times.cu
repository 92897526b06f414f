// Times the reference's own CUDA kernels (unmodified src/backends/cuda/ops/layers.cu and
// moe.cu, built by make_golden_gpu.sh with this file as the driver) at the sizes of the
// benchmark's model: 60 experts of 1408 features over a width of 2048, 16 heads of 128,
// a vocabulary of 151936; 8 tokens (a decode step) and 2048 tokens (a prompt).  Each kernel
// runs alone, twice untimed and then several times between CUDA events; the median is
// printed, one JSON object a line.  kernel_times.py times this repository's kernels at the
// same shapes.  These are the reference's in-tree kernels: its expert products always run
// through them (moe.cu:647-690); for attention it prefers FlashInfer where that is built in,
// and this kernel is what it runs otherwise (layers.cu:865-940, src/model/qwen2.cc:649-655).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <string>
#include <vector>
#include "inferx/core/tensor_view.h"
#include "inferx/ops/layers.h"
#include "inferx/ops/moe.h"
using inferx::DataType; using inferx::DeviceId; using inferx::Shape; using inferx::TensorView;
namespace ops = inferx::ops;
static uint64_t st = 88172645463325252ULL;
static float U() { st ^= st << 13; st ^= st >> 7; st ^= st << 17; return (float)((st >> 40) & 0xFFFFFF) / 8388608.0f - 1.0f; }
struct B { void* d; DataType t; std::vector<int64_t> s; };
static B Bf(std::vector<int64_t> s, float scale) {
  size_t n = 1; for (auto v : s) n *= v;
  std::vector<__nv_bfloat16> h(n);
  // fill a block and repeat it: generating 700M values one by one takes too long
  const size_t blk = std::min<size_t>(n, 1 << 20);
  for (size_t i = 0; i < blk; ++i) h[i] = __float2bfloat16(U() * scale);
  for (size_t i = blk; i < n; ++i) h[i] = h[i % blk];
  B b{nullptr, DataType::kBFloat16, s};
  cudaMalloc(&b.d, n * 2); cudaMemcpy(b.d, h.data(), n * 2, cudaMemcpyHostToDevice); return b;
}
static B I32(std::vector<int64_t> s, const std::vector<int32_t>& v) {
  B b{nullptr, DataType::kInt32, s}; cudaMalloc(&b.d, std::max<size_t>(v.size() * 4, 16));
  cudaMemcpy(b.d, v.data(), v.size() * 4, cudaMemcpyHostToDevice); return b;
}
static B Raw(DataType t, std::vector<int64_t> s, size_t bytes) { B b{nullptr, t, s}; cudaMalloc(&b.d, bytes); cudaMemset(b.d, 0, bytes); return b; }
static TensorView V(const B& b) { auto v = TensorView::Create(b.d, b.t, Shape(b.s), DeviceId::Cuda(0)); if (!v.ok()) { fprintf(stderr, "view\n"); exit(1);} return *v; }
static void Time(const char* name, int reps, const std::function<inferx::Status()>& f) {
  cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
  std::vector<float> ms;
  for (int i = 0; i < reps + 2; ++i) {
    cudaDeviceSynchronize(); cudaEventRecord(a);
    auto s = f(); cudaEventRecord(b); cudaEventSynchronize(b);
    if (!s.ok() || cudaGetLastError() != cudaSuccess) { fprintf(stderr, "%s failed: %s\n", name, s.ToString().c_str()); exit(1); }
    float t; cudaEventElapsedTime(&t, a, b); if (i >= 2) ms.push_back(t);
  }
  std::sort(ms.begin(), ms.end());
  printf("{\"kernel\": \"%s\", \"us\": %.1f}\n", name, ms[ms.size() / 2] * 1000.0f); fflush(stdout);
}
int main() {
  const int64_t E = 60, H = 2048, I = 1408;
  B wgu = Bf({E, 2 * I, H}, 0.05f), wd = Bf({E, H, I}, 0.05f);
  for (int64_t T : {8, 2048}) {
    const int64_t A = T * 4;
    // uniform routing: assignment i goes to expert (i * 7) % E, grouped
    std::vector<int32_t> cnt(E, 0); for (int64_t i = 0; i < A; ++i) cnt[(i * 7) % E]++;
    std::vector<int32_t> off(E + 1, 0); for (int e = 0; e < E; ++e) off[e + 1] = off[e] + cnt[e];
    B offs = I32({E + 1}, off), x = Bf({A, H}, 1.0f), gu = Raw(DataType::kBFloat16, {A, 2 * I}, A * 2 * I * 2);
    B act = Bf({A, I}, 1.0f), y = Raw(DataType::kBFloat16, {A, H}, A * H * 2);
    char n1[64], n2[64]; snprintf(n1, 64, "grouped_gate_up_t%lld", (long long)T); snprintf(n2, 64, "grouped_down_t%lld", (long long)T);
    Time(n1, 5, [&] { return ops::MoeGroupedGemmBf16(V(x), V(offs), V(wgu), TensorView(), V(gu)); });
    Time(n2, 5, [&] { return ops::MoeGroupedGemmBf16(V(act), V(offs), V(wd), TensorView(), V(y)); });
  }
  {  // router top-k at 2048 tokens and 8 tokens
    for (int64_t T : {8, 2048}) {
      B lg = Bf({T, E}, 3.0f), w = Raw(DataType::kFloat, {T, 4}, T * 16), e = Raw(DataType::kInt32, {T, 4}, T * 16);
      char n[64]; snprintf(n, 64, "route_topk_t%lld", (long long)T);
      Time(n, 9, [&] { return ops::MoeRouteTopK(V(lg), V(w), V(e), false, 1.0f); });
    }
  }
  {  // RMSNorm
    for (int64_t T : {8, 2048}) {
      B x = Bf({T, H}, 1.0f), w = Bf({H}, 1.0f), y = Raw(DataType::kBFloat16, {T, H}, T * H * 2);
      char n[64]; snprintf(n, 64, "rmsnorm_t%lld", (long long)T);
      Time(n, 9, [&] { return ops::RmsNorm(V(x), V(w), V(y), 1e-6f); });
    }
  }
  {  // paged decode attention: 8 sequences of 4096 keys, 16 heads of 128
    const int64_t S = 8, C = 4096, bs = 16, heads = 16, hd = 128, blocks = S * C / bs;
    B kc = Bf({blocks, bs, heads, hd}, 1.0f), vc = Bf({blocks, bs, heads, hd}, 1.0f);
    std::vector<int32_t> tbl(S * (C / bs)); for (size_t i = 0; i < tbl.size(); ++i) tbl[i] = (int32_t)i;
    std::vector<int32_t> seq(S), pos(S); for (int s = 0; s < S; ++s) { seq[s] = s; pos[s] = C - 1; }
    B table = I32({S, C / bs}, tbl), sq = I32({S}, seq), ps = I32({S}, pos);
    B q = Bf({S, heads, hd}, 1.0f), o = Raw(DataType::kBFloat16, {S, heads, hd}, S * heads * hd * 2);
    Time("paged_attention_decode_b8_ctx4096", 9, [&] { return ops::PagedAttention(V(q), V(kc), V(vc), V(table), V(sq), V(ps), V(o), 0.088f, C); });
  }
  {  // greedy choice over the vocabulary
    B lg = Bf({8, 151936}, 4.0f); std::vector<int32_t> r = {0, 1, 2, 3, 4, 5, 6, 7};
    B rows = I32({8}, r), out = Raw(DataType::kInt32, {8}, 32);
    Time("argmax_b8_vocab151936", 9, [&] { return ops::ArgmaxSample(V(lg), V(rows), V(out)); });
  }
  return 0;
}
