// The reference's own known-answer tests, written against the C++ host layer (include/hanzoquant_b200.hpp):
//   gather_forward_expands_single_route_input / gather_forward_accepts_per_route_input
//     (hanzo-quant/src/unquantized/mod.rs:616-645) with the [2,2,3] bank stored as exactly representable Q8_0,
//   test_deterministic_moe_routing_tie_break_lowest_expert (hanzo-engine/src/ops.rs:3728-3758),
//   a dense forward against a host-side dot product, and the error behaviour (exceptions, no CPU path).
// Exit code 0 = all passed.
#include <cmath>
#include <cstdio>
#include <cstring>

#include "hanzoquant_b200.hpp"

using namespace hq;

static uint16_t f16_one() { return 0x3C00; }

// [rows, 256] integer-valued weights (|v| <= 127) -> Q8_0 blocks with d = 1
static std::vector<uint8_t> q8_exact(const std::vector<float>& w, int rows) {
  std::vector<uint8_t> out((size_t)rows * 8 * 34);
  for (int r = 0; r < rows; ++r)
    for (int b = 0; b < 8; ++b) {
      uint8_t* p = &out[((size_t)r * 8 + b) * 34];
      const uint16_t d = f16_one();
      std::memcpy(p, &d, 2);
      for (int i = 0; i < 32; ++i) p[2 + i] = (uint8_t)(int8_t)w[(size_t)r * 256 + b * 32 + i];
    }
  return out;
}

#define EXPECT(cond)                                                   \
  do {                                                                 \
    if (!(cond)) {                                                     \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);    \
      return 1;                                                        \
    }                                                                  \
  } while (0)

int main() {
  // ---- gather_forward known answers -----------------------------------------------------------
  std::vector<float> bank(4 * 256, 0.f);   // experts {[[1,0,0],[0,1,0]], [[0,0,1],[1,1,1]]}, K padded to 256
  const float vals[12] = {1, 0, 0, 0, 1, 0, 0, 0, 1, 1, 1, 1};
  for (int r = 0; r < 4; ++r)
    for (int c = 0; c < 3; ++c) bank[(size_t)r * 256 + c] = vals[r * 3 + c];
  const std::vector<uint8_t> raw = q8_exact(bank, 4);
  GgufMatMul layer(Tensor::from_host(raw.data(), {2, 2, 8 * 34}, DType::U8), GgufMatMul::GgmlType::Q8_0, 256);
  {
    std::vector<float> x(2 * 256, 0.f);
    for (int t = 0; t < 2; ++t)
      for (int c = 0; c < 3; ++c) x[(size_t)t * 256 + c] = (float)(t * 3 + c + 1);
    const int32_t ids[4] = {0, 1, 1, 0};
    Tensor out = layer.gather_forward(Tensor::from_host(x.data(), {2, 1, 256}, DType::F32),
                                      Tensor::from_host(ids, {2, 2}, DType::I32));
    EXPECT(out.dims() == (std::vector<int64_t>{2, 2, 2}));
    float got[8];
    out.to_host(got);
    const float want[8] = {1, 2, 3, 6, 6, 15, 4, 5};
    for (int i = 0; i < 8; ++i) EXPECT(got[i] == want[i]);
    // per-route input [1, 2, K]
    const int32_t ids2[2] = {0, 1};
    Tensor out2 = layer.gather_forward(Tensor::from_host(x.data(), {1, 2, 256}, DType::F32),
                                       Tensor::from_host(ids2, {1, 2}, DType::I32));
    float got2[4];
    out2.to_host(got2);
    const float want2[4] = {1, 2, 6, 15};
    for (int i = 0; i < 4; ++i) EXPECT(got2[i] == want2[i]);
  }
  // ---- router tie-break -----------------------------------------------------------------------------
  {
    const float s[10] = {1, 5, 2, 5, 4, 7, 7, 7, 7, 7};
    MoeRouterTopKConfig cfg;
    cfg.top_k = 2;
    cfg.score_function = MoeRouterScoreFunction::Raw;
    cfg.selected_weight = MoeRouterSelectedWeight::Score;
    TopKOutput top = moe_router_topk(Tensor::from_host(s, {2, 5}, DType::F32), cfg);
    int32_t ids[4];
    float w[4];
    top.indices.to_host(ids);
    top.values.to_host(w);
    EXPECT(ids[0] == 1 && ids[1] == 3 && ids[2] == 0 && ids[3] == 1);
    EXPECT(w[0] == 5.f && w[1] == 5.f && w[2] == 7.f && w[3] == 7.f);
  }
  // ---- dense forward vs a host dot product -------------------------------------------------------------
  {
    const int n = 40, k = 256, m = 3;
    std::vector<float> w((size_t)n * k), x((size_t)m * k);
    for (size_t i = 0; i < w.size(); ++i) w[i] = (float)((int)((i * 37 + 11) % 15) - 7);
    for (size_t i = 0; i < x.size(); ++i) x[i] = (float)((int)((i * 13 + 5) % 9) - 4) * 0.25f;
    const std::vector<uint8_t> rw = q8_exact(w, n);
    GgufMatMul dense(Tensor::from_host(rw.data(), {n, 8 * 34}, DType::U8), GgufMatMul::GgmlType::Q8_0, k);
    Tensor y = dense.forward(Tensor::from_host(x.data(), {m, k}, DType::F32));
    std::vector<float> got((size_t)m * n);
    y.to_host(got.data());
    for (int i = 0; i < m; ++i)
      for (int j = 0; j < n; ++j) {
        double acc = 0;
        for (int c = 0; c < k; ++c) acc += (double)x[(size_t)i * k + c] * w[(size_t)j * k + c];
        EXPECT(std::fabs(got[(size_t)i * n + j] - acc) <= 1e-3 * (1.0 + std::fabs(acc)));
      }
  }
  // ---- errors are raised, not printed ---------------------------------------------------------------------
  {
    bool threw = false;
    try {
      GgufMatMul bad(Tensor::empty({4, 4 * 34}, DType::U8), GgufMatMul::GgmlType::Q8_0, 128);   // K % 256 != 0
    } catch (const Error&) { threw = true; }
    EXPECT(threw);
    threw = false;
    try {
      std::vector<float> x(128, 0.f);
      layer.forward(Tensor::from_host(x.data(), {1, 128}, DType::F32));   // expert bank + wrong K
    } catch (const Error&) { threw = true; }
    EXPECT(threw);
  }
  check_cuda(cudaDeviceSynchronize(), "sync");
  std::printf("host mirror ok\n");
  return 0;
}
