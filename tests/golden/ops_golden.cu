// Runs the reference's own CUDA kernels (src/backends/cuda/ops/layers.cu and moe.cu,
// unmodified, compiled for sm_100a) on small inputs and writes inputs and outputs to
// ops_golden.bin with an index in ops_golden.jsonl.  make_golden_gpu.sh builds and runs it
// on a machine with a GPU; both files are committed, and tests/test_ops_golden.py feeds
// the recorded inputs to the plain statements of tests/plain_qwen2_moe.py and compares
// with the recorded outputs.  It needs neither the reference nor a GPU.
//
// Inputs come from a linear congruential generator, rounded to bfloat16 where the kernel
// takes bfloat16; they are recorded, so nothing depends on reproducing the generator.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "inferx/core/tensor_view.h"
#include "inferx/ops/layers.h"
#include "inferx/ops/moe.h"

using inferx::DataType;
using inferx::DeviceId;
using inferx::Shape;
using inferx::TensorView;
namespace ops = inferx::ops;

namespace {

FILE* g_bin = nullptr;
FILE* g_idx = nullptr;
size_t g_off = 0;
uint64_t g_state = 0x2545F4914F6CDD1DULL;

float Uniform() {                       // in [-1, 1)
  g_state = g_state * 6364136223846793005ULL + 1442695040888963407ULL;
  return static_cast<float>((g_state >> 40) & 0xFFFFFF) / 8388608.0f - 1.0f;
}

struct Buf {
  std::vector<unsigned char> host;
  void* dev = nullptr;
  DataType dtype;
  std::vector<int64_t> dims;
  size_t bytes() const { return host.size(); }
};

size_t ElemSize(DataType t) {
  switch (t) {
    case DataType::kBFloat16: return 2;
    case DataType::kFloat: return 4;
    case DataType::kInt32: return 4;
    case DataType::kInt64: return 8;
    case DataType::kUInt64: return 8;
    default: return 0;
  }
}

Buf Make(DataType t, std::vector<int64_t> dims) {
  Buf b;
  b.dtype = t;
  b.dims = std::move(dims);
  size_t n = 1;
  for (int64_t d : b.dims) n *= static_cast<size_t>(d);
  b.host.assign(n * ElemSize(t), 0);
  cudaMalloc(&b.dev, b.host.size() ? b.host.size() : 16);
  cudaMemset(b.dev, 0, b.host.size() ? b.host.size() : 16);
  return b;
}

Buf RandomBf16(std::vector<int64_t> dims, float scale) {
  Buf b = Make(DataType::kBFloat16, std::move(dims));
  auto* p = reinterpret_cast<__nv_bfloat16*>(b.host.data());
  for (size_t i = 0; i < b.host.size() / 2; ++i) p[i] = __float2bfloat16(Uniform() * scale);
  cudaMemcpy(b.dev, b.host.data(), b.host.size(), cudaMemcpyHostToDevice);
  return b;
}

Buf Ints(std::vector<int64_t> dims, const std::vector<int32_t>& values) {
  Buf b = Make(DataType::kInt32, std::move(dims));
  std::memcpy(b.host.data(), values.data(), values.size() * 4);
  cudaMemcpy(b.dev, b.host.data(), b.host.size(), cudaMemcpyHostToDevice);
  return b;
}

Buf Floats(std::vector<int64_t> dims, const std::vector<float>& values) {
  Buf b = Make(DataType::kFloat, std::move(dims));
  std::memcpy(b.host.data(), values.data(), values.size() * 4);
  cudaMemcpy(b.dev, b.host.data(), b.host.size(), cudaMemcpyHostToDevice);
  return b;
}

TensorView View(const Buf& b) {
  auto v = TensorView::Create(b.dev, b.dtype, Shape(b.dims), DeviceId::Cuda(0));
  if (!v.ok()) {
    std::fprintf(stderr, "view: %s\n", v.status().ToString().c_str());
    std::exit(1);
  }
  return *v;
}

const char* Name(DataType t) {
  switch (t) {
    case DataType::kBFloat16: return "bf16";
    case DataType::kFloat: return "f32";
    case DataType::kInt32: return "i32";
    default: return "?";
  }
}

// records the buffer as it stands on the host (inputs) or on the device (outputs)
void Record(const std::string& name, Buf& b, bool from_device) {
  if (from_device) cudaMemcpy(b.host.data(), b.dev, b.host.size(), cudaMemcpyDeviceToHost);
  std::fprintf(g_idx, "{\"name\": \"%s\", \"dtype\": \"%s\", \"shape\": [", name.c_str(),
               Name(b.dtype));
  for (size_t i = 0; i < b.dims.size(); ++i)
    std::fprintf(g_idx, "%s%lld", i ? ", " : "", (long long)b.dims[i]);
  std::fprintf(g_idx, "], \"offset\": %zu, \"nbytes\": %zu}\n", g_off, b.host.size());
  std::fwrite(b.host.data(), 1, b.host.size(), g_bin);
  g_off += b.host.size();
}

void Check(const inferx::Status& s, const char* what) {
  cudaError_t e = cudaDeviceSynchronize();
  if (!s.ok() || e != cudaSuccess) {
    std::fprintf(stderr, "%s: %s / %s\n", what, s.ToString().c_str(), cudaGetErrorString(e));
    std::exit(1);
  }
}

}  // namespace

int main(int argc, char** argv) {
  const std::string out = argc > 1 ? argv[1] : ".";
  g_bin = std::fopen((out + "/ops_golden.bin").c_str(), "wb");
  g_idx = std::fopen((out + "/ops_golden.jsonl").c_str(), "w");
  if (!g_bin || !g_idx) return 1;

  {  // RMSNorm
    Buf x = RandomBf16({5, 96}, 2.0f), w = RandomBf16({96}, 1.0f), y = Make(DataType::kBFloat16, {5, 96});
    Record("rmsnorm.x", x, false);
    Record("rmsnorm.weight", w, false);
    Check(ops::RmsNorm(View(x), View(w), View(y), 1e-5f), "RmsNorm");
    Record("rmsnorm.out", y, true);
  }
  {  // rotary embedding, half-split, in place
    Buf q = RandomBf16({7, 6, 32}, 1.0f), k = RandomBf16({7, 2, 32}, 1.0f);
    Buf pos = Ints({7}, {0, 1, 2, 5, 9, 100, 4095});
    Record("rope.q", q, false);
    Record("rope.k", k, false);
    Record("rope.positions", pos, false);
    Check(ops::RotaryEmbedding(View(q), View(k), View(pos), 1000000.0f), "RotaryEmbedding");
    Record("rope.q_out", q, true);
    Record("rope.k_out", k, true);
  }
  {  // SwiGLU activation, fused gate|up layout
    Buf f = RandomBf16({5, 80}, 3.0f), y = Make(DataType::kBFloat16, {5, 40});
    Record("silu_mul.fused", f, false);
    Check(ops::SiluMulFused(View(f), View(y)), "SiluMulFused");
    Record("silu_mul.out", y, true);
  }
  {  // naive causal attention with grouped heads
    Buf q = RandomBf16({9, 6, 32}, 1.0f), k = RandomBf16({9, 2, 32}, 1.0f), v = RandomBf16({9, 2, 32}, 1.0f);
    Buf y = Make(DataType::kBFloat16, {9, 6, 32});
    Record("attention.q", q, false);
    Record("attention.k", k, false);
    Record("attention.v", v, false);
    Check(ops::Attention(View(q), View(k), View(v), View(y), 0.25f), "Attention");
    Record("attention.out", y, true);
  }
  {  // paged cache: append, then attention over the pages with a window
    const int64_t blocks = 6, bs = 4, kvh = 2, hd = 32, heads = 4;
    Buf kc = Make(DataType::kBFloat16, {blocks, bs, kvh, hd}), vc = Make(DataType::kBFloat16, {blocks, bs, kvh, hd});
    // two sequences: 11 and 6 tokens, pages not in order
    Buf table = Ints({2, 3}, {4, 1, 5, 2, 0, 3});
    std::vector<int32_t> seq, posv, slots;
    const int lens[2] = {11, 6};
    const int tbl[2][3] = {{4, 1, 5}, {2, 0, 3}};
    for (int s = 0; s < 2; ++s)
      for (int p = 0; p < lens[s]; ++p) {
        seq.push_back(s);
        posv.push_back(p);
        slots.push_back(tbl[s][p / 4] * 4 + p % 4);
      }
    const int64_t T = static_cast<int64_t>(seq.size());
    Buf k = RandomBf16({T, kvh, hd}, 1.0f), v = RandomBf16({T, kvh, hd}, 1.0f), q = RandomBf16({T, heads, hd}, 1.0f);
    Buf slot_b = Ints({T}, slots), seq_b = Ints({T}, seq), pos_b = Ints({T}, posv);
    Record("paged.k", k, false);
    Record("paged.v", v, false);
    Record("paged.q", q, false);
    Record("paged.slots", slot_b, false);
    Record("paged.block_table", table, false);
    Record("paged.seq_of_token", seq_b, false);
    Record("paged.q_pos", pos_b, false);
    Check(ops::AppendToKvCache(View(k), View(v), View(kc), View(vc), View(slot_b)), "AppendToKvCache");
    Record("paged.k_cache", kc, true);
    Record("paged.v_cache", vc, true);
    Buf y = Make(DataType::kBFloat16, {T, heads, hd}), y5 = Make(DataType::kBFloat16, {T, heads, hd});
    Check(ops::PagedAttention(View(q), View(kc), View(vc), View(table), View(seq_b), View(pos_b),
                              View(y), 0.2f, 16),
          "PagedAttention");
    Record("paged.out", y, true);
    Check(ops::PagedAttentionWithLse(View(q), View(kc), View(vc), View(table), View(seq_b),
                                     View(pos_b), View(y5), TensorView(), 0.2f, 5, 16),
          "PagedAttentionWithLse");
    Record("paged.out_window5", y5, true);
  }
  {  // router: softmax over all experts, top-k, ties to the lower index
    Buf lg = RandomBf16({6, 8}, 3.0f);
    auto* p = reinterpret_cast<__nv_bfloat16*>(lg.host.data());
    p[8 + 2] = p[8 + 5] = __float2bfloat16(4.0f);      // a tie at the top of row 1
    cudaMemcpy(lg.dev, lg.host.data(), lg.host.size(), cudaMemcpyHostToDevice);
    Record("route.logits", lg, false);
    for (int renorm = 0; renorm < 2; ++renorm) {
      Buf w = Make(DataType::kFloat, {6, 3}), e = Make(DataType::kInt32, {6, 3});
      Check(ops::MoeRouteTopK(View(lg), View(w), View(e), renorm != 0, 1.0f), "MoeRouteTopK");
      Record(renorm ? "route.weights_renorm" : "route.weights", w, true);
      Record(renorm ? "route.experts_renorm" : "route.experts", e, true);
      if (renorm) {
        Buf off = Make(DataType::kInt32, {9}), rows = Make(DataType::kInt32, {18}), dest = Make(DataType::kInt32, {18});
        Check(ops::MoeBuildDispatch(View(e), 8, View(off), View(rows), View(dest)), "MoeBuildDispatch");
        Record("dispatch.offsets", off, true);
        Record("dispatch.rows", rows, true);
        Record("dispatch.dest", dest, true);
        // experts: gather, grouped gate|up product, activation, grouped down product, combine
        Buf x = RandomBf16({6, 64}, 1.0f), xg = Make(DataType::kBFloat16, {18, 64});
        Buf wgu = RandomBf16({8, 48, 64}, 0.2f), wd = RandomBf16({8, 64, 24}, 0.2f);
        Buf gu = Make(DataType::kBFloat16, {18, 48}), act = Make(DataType::kBFloat16, {18, 24});
        Buf yd = Make(DataType::kBFloat16, {18, 64}), mix = Make(DataType::kBFloat16, {6, 64});
        Record("experts.x", x, false);
        Record("experts.w_gate_up", wgu, false);
        Record("experts.w_down", wd, false);
        Check(ops::MoeGatherRows(View(x), View(rows), View(xg)), "MoeGatherRows");
        Check(ops::MoeGroupedGemmBf16(View(xg), View(off), View(wgu), TensorView(), View(gu)), "grouped gate|up");
        Record("experts.gate_up", gu, true);
        Check(ops::SiluMulFused(View(gu), View(act)), "SiluMulFused");
        Check(ops::MoeGroupedGemmBf16(View(act), View(off), View(wd), TensorView(), View(yd)), "grouped down");
        Record("experts.down", yd, true);
        Check(ops::MoeCombineRows(View(yd), View(dest), View(w), View(mix)), "MoeCombineRows");
        Record("experts.combined", mix, true);
        Buf shared = RandomBf16({6, 64}, 1.0f), gate = RandomBf16({6, 1}, 2.0f);
        Record("experts.shared", shared, false);
        Record("experts.shared_gate_logits", gate, false);
        Check(ops::MoeAddSharedExpert(View(shared), View(gate), View(mix)), "MoeAddSharedExpert");
        Record("experts.with_shared", mix, true);
      }
    }
  }
  {  // greedy choice, penalties and masks, log-probabilities
    Buf lg = RandomBf16({4, 211}, 4.0f);
    auto* p = reinterpret_cast<__nv_bfloat16*>(lg.host.data());
    p[17] = p[18] = __float2bfloat16(9.0f);             // a tie at the top of row 0
    cudaMemcpy(lg.dev, lg.host.data(), lg.host.size(), cudaMemcpyHostToDevice);
    Record("sample.logits", lg, false);
    Buf rows = Ints({3}, {0, 2, 3}), out = Make(DataType::kInt32, {3});
    Record("sample.rows", rows, false);
    Check(ops::ArgmaxSample(View(lg), View(rows), View(out)), "ArgmaxSample");
    Record("sample.argmax", out, true);
    const int64_t H = 256, M = 16;
    std::vector<int32_t> hid(3 * H, -1), hcount(3 * H, 0), mask(3 * M, -1);
    const int ids0[] = {17, 4, 99}, c0[] = {1, 2, 1};
    for (int j = 0; j < 3; ++j) { hid[j] = ids0[j]; hcount[j] = c0[j]; }
    const int ids2[] = {3, 200, 44, 45, 46}, c2[] = {2, 1, 1, 5, 1};
    for (int j = 0; j < 5; ++j) { hid[2 * H + j] = ids2[j]; hcount[2 * H + j] = c2[j]; }
    mask[0] = 18; mask[M] = 7; mask[M + 1] = 8;
    Buf pres = Floats({3}, {0.6f, 0.0f, -0.5f}), freq = Floats({3}, {0.0f, 0.0f, 0.25f}), rep = Floats({3}, {1.0f, 1.0f, 1.7f});
    Buf hid_b = Ints({3, H}, hid), hc_b = Ints({3, H}, hcount), mask_b = Ints({3, M}, mask);
    Record("sample.presence", pres, false);
    Record("sample.frequency", freq, false);
    Record("sample.repetition", rep, false);
    Record("sample.history_ids", hid_b, false);
    Record("sample.history_counts", hc_b, false);
    Record("sample.mask_ids", mask_b, false);
    Check(ops::ApplyPenalties(View(lg), View(rows), View(pres), View(freq), View(rep), View(hid_b),
                              View(hc_b), View(mask_b)),
          "ApplyPenalties");
    Record("sample.logits_penalised", lg, true);
    Check(ops::ArgmaxSample(View(lg), View(rows), View(out)), "ArgmaxSample");
    Record("sample.argmax_penalised", out, true);
    Buf kw = Ints({3}, {5, 0, 20}), clp = Make(DataType::kFloat, {3});
    Buf tid = Make(DataType::kInt32, {3, 20}), tlp = Make(DataType::kFloat, {3, 20});
    Record("sample.k_wanted", kw, false);
    Check(ops::ComputeLogprobs(View(lg), View(rows), View(out), View(kw), View(clp), View(tid), View(tlp)),
          "ComputeLogprobs");
    Record("sample.chosen_logprob", clp, true);
    Record("sample.top_ids", tid, true);
    Record("sample.top_logprobs", tlp, true);
  }
  std::fclose(g_bin);
  std::fclose(g_idx);
  std::printf("wrote %zu bytes\n", g_off);
  return 0;
}
