// Test program for the C++ primitive layer, in the manner of the reference's
// tests/unit/rmsnorm_primitive_test.cpp: every check computes its expectation on the host in
// this file and compares with the primitive's output through the public API only.
// Needs a CUDA device.  Exit code 0 and the line "ALL PASSED" on success.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

#include <mlx/mlx.h>

#include "q_gemm_dequant_primitive.h"
#include "rmsnorm_primitive.h"
#include "rope_apply_primitive.h"
#include "swiglu_mlp_primitive.h"
#include "../graph/layers.h"

namespace mx = mlx::core;
using namespace mlxr::kernels;
namespace gr = mlxr::graph;

static int g_failed = 0, g_run = 0;
#define CHECK(cond)                                                              \
  do {                                                                           \
    if (!(cond)) { std::printf("    CHECK failed: %s (line %d)\n", #cond, __LINE__); ok = false; } \
  } while (0)
#define TEST(name) static bool name()
#define RUN(name)                                                  \
  do {                                                             \
    g_run++;                                                       \
    bool r = false;                                                \
    try { r = name(); } catch (const std::exception& e) { std::printf("    exception: %s\n", e.what()); } \
    std::printf("[%s] %s\n", r ? "  OK  " : "FAILED", #name);      \
    if (!r) g_failed++;                                            \
  } while (0)

static std::vector<float> randn(size_t n, unsigned seed, float std = 1.0f) {
  std::mt19937 g(seed);
  std::normal_distribution<float> d(0.0f, std);
  std::vector<float> v(n);
  for (auto& x : v) x = d(g);
  return v;
}
static double rel_l2(const std::vector<float>& a, const std::vector<float>& b) {
  double num = 0, den = 0;
  for (size_t i = 0; i < a.size(); i++) { num += (double)(a[i] - b[i]) * (a[i] - b[i]); den += (double)b[i] * b[i]; }
  return std::sqrt(num / (den > 0 ? den : 1));
}
static std::vector<float> to_host(mx::array a) {
  mx::array f = mx::astype(a, mx::float32);
  f.eval();
  mx::synchronize();
  return std::vector<float>(f.data<float>(), f.data<float>() + f.size());
}
// Q4_0 blocks (MLXR layout: byte i = elements 2i (low nibble), 2i+1 (high), (nibble - 8) * scale)
// made from random nibbles and a simple scale; returns the packed bytes and the fp32 weights.
static void make_q4_0(int N, int K, unsigned seed, std::vector<uint8_t>& packed, std::vector<float>& w) {
  std::mt19937 g(seed);
  packed.resize((size_t)N * (K / 32) * 18);
  w.resize((size_t)N * K);
  for (int n = 0; n < N; n++)
    for (int b = 0; b < K / 32; b++) {
      uint8_t* blk = packed.data() + ((size_t)n * (K / 32) + b) * 18;
      const float scale = 0.0078125f * (float)(1 + g() % 7);      // exactly representable in fp16
      mx::float16_t h(scale);
      std::memcpy(blk, &h.bits, 2);
      for (int i = 0; i < 16; i++) {
        const int lo = g() % 16, hi = g() % 16;
        blk[2 + i] = (uint8_t)(lo | (hi << 4));
        w[(size_t)n * K + b * 32 + 2 * i] = (float)(lo - 8) * scale;
        w[(size_t)n * K + b * 32 + 2 * i + 1] = (float)(hi - 8) * scale;
      }
    }
}

TEST(rmsnorm_matches_formula) {
  bool ok = true;
  const int rows = 5, hidden = 1024;
  auto x = randn((size_t)rows * hidden, 1), g = randn(hidden, 2, 0.1f);
  for (auto& v : g) v += 1.0f;
  mx::array xa(x.data(), {rows, hidden}, mx::float32), ga(g.data(), {hidden}, mx::float32);
  mx::array y = rmsnorm_fused(xa, ga, 1e-5f);
  CHECK(!y.is_available());                       // lazy, like the reference (rmsnorm_primitive.mm:351-356)
  auto got = to_host(y);
  std::vector<float> want(x.size());
  for (int r = 0; r < rows; r++) {
    double ss = 0;
    for (int i = 0; i < hidden; i++) ss += (double)x[r * hidden + i] * x[r * hidden + i];
    const double inv = 1.0 / std::sqrt(ss / hidden + 1e-5);
    for (int i = 0; i < hidden; i++) want[r * hidden + i] = (float)(x[r * hidden + i] * inv * g[i]);
  }
  CHECK(rel_l2(got, want) < 1e-5);
  CHECK(y.shape() == xa.shape());
  return ok;
}

TEST(rmsnorm_rejects_bad_weight) {
  bool ok = true;
  auto x = randn(64, 3), g = randn(8, 4);
  mx::array xa(x.data(), {2, 32}, mx::float32), ga(g.data(), {8}, mx::float32);
  bool threw = false;
  try { mx::array y = rmsnorm_fused(xa, ga); y.eval(); } catch (const std::invalid_argument&) { threw = true; }
  CHECK(threw);                                   // std::invalid_argument, rmsnorm_primitive.mm:309-321
  return ok;
}

TEST(q_gemm_matches_dequantized_matmul) {
  bool ok = true;
  const int M = 3, N = 96, K = 512;
  std::vector<uint8_t> packed; std::vector<float> w;
  make_q4_0(N, K, 5, packed, w);
  auto x = randn((size_t)M * K, 6);
  mx::array xa = mx::astype(mx::array(x.data(), {M, K}, mx::float32), mx::float16);
  xa.eval();
  auto xr = to_host(xa);                           // the fp16-rounded activations
  mx::array wa(packed.data(), {(int)packed.size()}, mx::uint8);
  CHECK(compute_quantized_weight_size(N, K, QuantType::Q4_0) == packed.size());
  mx::array y = q_gemm_dequant(xa, wa, M, N, K, QuantType::Q4_0, 32);
  auto got = to_host(y);
  std::vector<float> want((size_t)M * N);
  for (int m = 0; m < M; m++)
    for (int n = 0; n < N; n++) {
      double s = 0;
      for (int k = 0; k < K; k++) s += (double)xr[m * K + k] * w[(size_t)n * K + k];
      want[m * N + n] = (float)s;
    }
  CHECK(y.shape() == (mx::Shape{M, N}));
  CHECK(rel_l2(got, want) < 2e-3);
  // the dequantize extension returns exactly the weights the blocks encode
  auto dq = to_host(dequantize(wa, N, K, QuantType::Q4_0, mx::float32));
  CHECK(dq == w);
  return ok;
}

TEST(q_gemm_errors_and_helpers) {
  bool ok = true;
  auto x = randn(64, 7);
  mx::array xa(x.data(), {2, 32}, mx::float32);
  std::vector<uint8_t> bytes(18 * 4, 0);
  mx::array wa(bytes.data(), {(int)bytes.size()}, mx::uint8);
  bool threw = false;
  try { q_gemm_dequant(xa, wa, 3, 4, 32, QuantType::Q4_0, 32); } catch (const std::runtime_error&) { threw = true; }
  CHECK(threw);                                   // input shape != [M, K]: runtime_error (q_gemm_dequant_primitive.mm:490-496)
  threw = false;
  try { q_gemm_dequant(xa, wa, 2, 4, 32, QuantType::Q3_K, 32); } catch (const std::runtime_error&) { threw = true; }
  CHECK(threw);                                   // a format without code
  CHECK(std::string(quant_type_name(QuantType::Q4_K)) == "Q4_K");
  CHECK(QGemmDequantPrimitive::get_default_group_size(QuantType::Q4_K) == 256);
  CHECK(std::fabs(QGemmDequantPrimitive::get_bytes_per_weight(QuantType::Q8_0) - 1.0625f) < 1e-6f);
  QGemmDequantPrimitive a(mx::default_stream(mx::default_device()), 2, 4, 32, QuantType::Q4_0, 32);
  QGemmDequantPrimitive b(mx::default_stream(mx::default_device()), 2, 4, 32, QuantType::Q4_0, 32);
  QGemmDequantPrimitive c(mx::default_stream(mx::default_device()), 2, 8, 32, QuantType::Q4_0, 32);
  CHECK(std::string(a.name()) == "q_gemm_dequant");
  CHECK(a.is_equivalent(b) && !a.is_equivalent(c));
  return ok;
}

TEST(swiglu_and_dense_mlp) {
  bool ok = true;
  const int M = 2, H = 64, I = 160;
  auto x = randn((size_t)M * H, 8), wg = randn((size_t)I * H, 9, 0.1f), wu = randn((size_t)I * H, 10, 0.1f),
       wd = randn((size_t)H * I, 11, 0.1f);
  mx::array xa(x.data(), {M, H}, mx::float32), ga(wg.data(), {I, H}, mx::float32), ua(wu.data(), {I, H}, mx::float32),
      da(wd.data(), {H, I}, mx::float32);
  auto got = to_host(swiglu_mlp(xa, ga, ua, da));
  std::vector<float> h((size_t)M * I), want((size_t)M * H);
  for (int m = 0; m < M; m++)
    for (int i = 0; i < I; i++) {
      double g = 0, u = 0;
      for (int k = 0; k < H; k++) { g += (double)x[m * H + k] * wg[(size_t)i * H + k]; u += (double)x[m * H + k] * wu[(size_t)i * H + k]; }
      h[m * I + i] = (float)(g / (1.0 + std::exp(-g)) * u);
    }
  for (int m = 0; m < M; m++)
    for (int n = 0; n < H; n++) {
      double s = 0;
      for (int i = 0; i < I; i++) s += (double)h[m * I + i] * wd[(size_t)n * I + i];
      want[m * H + n] = (float)s;
    }
  CHECK(rel_l2(got, want) < 1e-4);
  auto sw = to_host(swiglu(mx::array(x.data(), {M, H}, mx::float32), mx::array(x.data(), {M, H}, mx::float32)));
  bool close = true;
  for (size_t i = 0; i < x.size(); i++) close = close && std::fabs(sw[i] - (float)(x[i] / (1.0 + std::exp(-x[i])) * x[i])) < 1e-5f;
  CHECK(close);
  return ok;
}

TEST(rope_matches_interleaved_rotation) {
  bool ok = true;
  const int B = 1, T = 4, heads = 2, d = 16, max_seq = 64;
  auto tables = compute_rope_tables(max_seq, d, 10000.0f);
  auto cosv = to_host(tables.first), sinv = to_host(tables.second);
  auto x = randn((size_t)B * T * heads * d, 12);
  int32_t pos[T] = {0, 5, 17, 63};
  mx::array xa(x.data(), {B, T, heads, d}, mx::float32), pa(pos, {B, T}, mx::int32);
  auto got = to_host(rope_apply(xa, tables.first, tables.second, pa));
  std::vector<float> want(x.size());
  for (int t = 0; t < T; t++)
    for (int hd = 0; hd < heads; hd++)
      for (int p = 0; p < d / 2; p++) {
        const float c = cosv[(size_t)pos[t] * (d / 2) + p], s = sinv[(size_t)pos[t] * (d / 2) + p];
        const size_t o = ((size_t)t * heads + hd) * d + 2 * p;
        want[o] = x[o] * c - x[o + 1] * s;          // pairs (2p, 2p+1): rope_apply_primitive.mm:238-252
        want[o + 1] = x[o + 1] * c + x[o] * s;
      }
  CHECK(rel_l2(got, want) < 1e-6);
  CHECK(std::string(rope_scaling_mode_name(RoPEScalingMode::NTK)) == "ntk" || std::string(rope_scaling_mode_name(RoPEScalingMode::NTK)) == "NTK");
  return ok;
}

TEST(no_cpu_path) {
  bool ok = true;
  RMSNormPrimitive p(mx::default_stream(mx::default_device()), 1e-6f);
  std::vector<mx::array> in, out;
  bool threw = false;
  try { p.eval_cpu(in, out); } catch (const std::runtime_error&) { threw = true; }
  CHECK(threw);
  return ok;
}

// ---- graph layers (core/graph/layers.h): the reference's tests/unit/layers_test.cpp checks shapes
// and finiteness only; these compare with host arithmetic as well -------------------------------
TEST(graph_rmsnorm_and_dense_linear) {
  bool ok = true;
  const int B = 2, T = 3, H = 256, O = 96;
  auto x = randn((size_t)B * T * H, 21);
  gr::RMSNorm norm(H, 1e-5f);
  CHECK(norm.weight().shape() == std::vector<int>({H}));
  gr::Tensor xt = gr::from_data(x.data(), {B, T, H}, mx::float32);
  auto y = to_host(norm.forward(xt).array());
  std::vector<float> want(x.size());
  for (int r = 0; r < B * T; r++) {
    double ss = 0;
    for (int i = 0; i < H; i++) ss += (double)x[r * H + i] * x[r * H + i];
    const double inv = 1.0 / std::sqrt(ss / H + 1e-5);
    for (int i = 0; i < H; i++) want[r * H + i] = (float)(x[r * H + i] * inv);   // weight initialised to ones (layers.cpp:26-29)
  }
  CHECK(rel_l2(y, want) < 1e-5);
  gr::Linear lin(H, O, true);
  CHECK(lin.weight().shape() == std::vector<int>({O, H}) && lin.bias() != nullptr);
  auto w = randn((size_t)O * H, 22, 0.05f), b = randn(O, 23);
  lin.weight() = gr::from_data(w.data(), {O, H}, mx::float32);
  *lin.bias() = gr::from_data(b.data(), {O}, mx::float32);
  gr::Tensor out = lin.forward(xt);
  CHECK(out.shape() == std::vector<int>({B, T, O}));
  auto got = to_host(out.array());
  std::vector<float> wl((size_t)B * T * O);
  for (int r = 0; r < B * T; r++)
    for (int o = 0; o < O; o++) {
      double s = b[o];
      for (int i = 0; i < H; i++) s += (double)x[r * H + i] * w[(size_t)o * H + i];
      wl[(size_t)r * O + o] = (float)s;
    }
  CHECK(rel_l2(got, wl) < 1e-5);
  gr::Linear nob(H, O);
  CHECK(nob.bias() == nullptr);
  bool threw = false;
  try { nob.forward(gr::zeros({2, H + 1})); } catch (const std::invalid_argument&) { threw = true; }
  CHECK(threw);
  return ok;
}

TEST(graph_rotary_embedding_split_half) {
  bool ok = true;
  const int B = 1, T = 5, heads = 2, d = 32, max_seq = 64, offset = 3;
  gr::RotaryEmbedding rope(d, max_seq, 10000.0f);
  CHECK(rope.cos_table().shape() == std::vector<int>({max_seq, d / 2}));
  auto q = randn((size_t)B * T * heads * d, 31), k = randn((size_t)B * T * heads * d, 32);
  auto out = rope.forward(gr::from_data(q.data(), {B, T, heads, d}, mx::float32), gr::from_data(k.data(), {B, T, heads, d}, mx::float32), offset);
  auto gq = to_host(out.first.array()), gk = to_host(out.second.array());
  std::vector<float> wq(q.size()), wk(k.size());
  for (int t = 0; t < T; t++)
    for (int h = 0; h < heads; h++)
      for (int p = 0; p < d / 2; p++) {
        const float freq = 1.0f / std::pow(10000.0f, (2.0f * p) / d);      // layers.cpp:126-129
        const float ang = (float)(offset + t) * freq;
        const float c = std::cos(ang), s = std::sin(ang);
        const size_t o = ((size_t)t * heads + h) * d;
        wq[o + p] = q[o + p] * c - q[o + d / 2 + p] * s;                     // rotate_half: layers.cpp:196-208
        wq[o + d / 2 + p] = q[o + d / 2 + p] * c + q[o + p] * s;
        wk[o + p] = k[o + p] * c - k[o + d / 2 + p] * s;
        wk[o + d / 2 + p] = k[o + d / 2 + p] * c + k[o + p] * s;
      }
  CHECK(rel_l2(gq, wq) < 1e-6 && rel_l2(gk, wk) < 1e-6);
  bool threw = false;
  try { gr::RotaryEmbedding bad(7, 8); } catch (const std::invalid_argument&) { threw = true; }
  CHECK(threw);                                       // layers.cpp:115-117
  threw = false;
  try { rope.forward(gr::zeros({T, heads, d}), gr::zeros({T, heads, d})); } catch (const std::invalid_argument&) { threw = true; }
  CHECK(threw);                                       // layers.cpp:164-168
  return ok;
}

TEST(graph_mlp_dense_and_quantized) {
  bool ok = true;
  const int M = 2, H = 512, I = 1024;
  auto x = randn((size_t)M * H, 41);
  gr::Tensor xt = gr::from_data(x.data(), {M, H}, mx::float32);
  std::vector<uint8_t> pg, pu, pd;
  std::vector<float> wg, wu, wd;
  make_q4_0(I, H, 42, pg, wg);
  make_q4_0(I, H, 43, pu, wu);
  make_q4_0(H, I, 44, pd, wd);
  // host expectation: down(SiLU(gate(n)) * up(n)), n = rmsnorm(x) with unit weight
  std::vector<float> n(x.size()), hbuf((size_t)M * I), want((size_t)M * H);
  for (int m = 0; m < M; m++) {
    double ss = 0;
    for (int i = 0; i < H; i++) ss += (double)x[m * H + i] * x[m * H + i];
    const double inv = 1.0 / std::sqrt(ss / H + 1e-5);
    for (int i = 0; i < H; i++) n[m * H + i] = (float)(x[m * H + i] * inv);
    for (int i = 0; i < I; i++) {
      double g = 0, u = 0;
      for (int k = 0; k < H; k++) { g += (double)n[m * H + k] * wg[(size_t)i * H + k]; u += (double)n[m * H + k] * wu[(size_t)i * H + k]; }
      hbuf[(size_t)m * I + i] = (float)(g / (1.0 + std::exp(-g)) * u);
    }
    for (int o = 0; o < H; o++) {
      double s = 0;
      for (int i = 0; i < I; i++) s += (double)hbuf[(size_t)m * I + i] * wd[(size_t)o * I + i];
      want[(size_t)m * H + o] = (float)s;
    }
  }
  gr::RMSNorm norm(H, 1e-5f);
  // dense weights: three Linear::forward calls and swiglu (layers.cpp:400-420)
  gr::MLP dense(H, I);
  dense.gate_proj().weight() = gr::from_data(wg.data(), {I, H}, mx::float32);
  dense.up_proj().weight() = gr::from_data(wu.data(), {I, H}, mx::float32);
  dense.down_proj().weight() = gr::from_data(wd.data(), {H, I}, mx::float32);
  auto got_dense = to_host(dense.forward(norm.forward(xt)).array());
  CHECK(rel_l2(got_dense, want) < 1e-4);
  // packed weights: the fused block, with the RMSNorm prologue inside the same call
  gr::MLP q(H, I);
  q.gate_proj().set_quantized(gr::from_data(pg.data(), {(int)pg.size()}, mx::uint8), QuantType::Q4_0);
  q.up_proj().set_quantized(gr::from_data(pu.data(), {(int)pu.size()}, mx::uint8), QuantType::Q4_0);
  q.down_proj().set_quantized(gr::from_data(pd.data(), {(int)pd.size()}, mx::uint8), QuantType::Q4_0);
  gr::Tensor yq = q.forward(xt, norm);
  CHECK(yq.shape() == std::vector<int>({M, H}));
  CHECK(rel_l2(to_host(yq.array()), want) < 2e-3);
  // a single quantized Linear
  auto yl = to_host(q.gate_proj().forward(gr::from_data(n.data(), {M, H}, mx::float32)).array());
  std::vector<float> wlg((size_t)M * I);
  for (int m = 0; m < M; m++)
    for (int i = 0; i < I; i++) {
      double g = 0;
      for (int k = 0; k < H; k++) g += (double)n[m * H + k] * wg[(size_t)i * H + k];
      wlg[(size_t)m * I + i] = (float)g;
    }
  CHECK(rel_l2(yl, wlg) < 1e-3);
  bool threw = false;
  try { q.gate_proj().set_quantized(gr::zeros({10}, mx::uint8), QuantType::Q4_0); } catch (const std::invalid_argument&) { threw = true; }
  CHECK(threw);
  return ok;
}

int main() {
  RUN(graph_rmsnorm_and_dense_linear);
  RUN(graph_rotary_embedding_split_half);
  RUN(graph_mlp_dense_and_quantized);
  RUN(rmsnorm_matches_formula);
  RUN(rmsnorm_rejects_bad_weight);
  RUN(q_gemm_matches_dequantized_matmul);
  RUN(q_gemm_errors_and_helpers);
  RUN(swiglu_and_dense_mlp);
  RUN(rope_matches_interleaved_rotation);
  RUN(no_cpu_path);
  std::printf("%d tests, %d failed\n", g_run, g_failed);
  if (g_failed == 0) std::printf("ALL PASSED\n");
  return g_failed == 0 ? 0 : 1;
}
