// Self-test of the C++ host mirror (mlx-serve_b200/host/qb200_host.hpp): the reference's wrapper names driven
// the way its call sites drive them -- quantizeAffine / dequantizeAffine round trip, qmatmulBits at decode and
// prefill widths, gatherExpertMm on rows sorted by expert, KVCache.updateAffine + quantAttention over the
// strided cache views -- each compared with the CPU oracle (test infrastructure) on the same seeded inputs.
// Exit code 0 = all checks passed.  `--link-only` returns before touching a GPU (used by the CPU test suite to
// check that the header compiles and links against the C ABI).
#include <cuda_runtime_api.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "qb200_host.hpp"

extern "C" {
void qo_f32_to_bf16(const float* x, uint16_t* out, int64_t n);
void qo_bf16_to_f32(const uint16_t* x, float* out, int64_t n);
void qo_quantize(const float* x, int64_t rows, int64_t d, int gs, int bits, uint32_t* q, uint16_t* s, uint16_t* b);
void qo_qmm_t(const float* x, const uint32_t* w, const uint16_t* s, const uint16_t* b, int64_t M, int64_t N, int64_t K,
              int gs, int bits, float* y);
void qo_qmm_t_bf16w(const float* x, const uint32_t* w, const uint16_t* s, const uint16_t* b, int64_t M, int64_t N,
                    int64_t K, int gs, int bits, float* y);
void qo_gather_qmm_t(const float* x, const uint32_t* w, const uint16_t* s, const uint16_t* b, const int64_t* lhs,
                     const int64_t* rhs, int64_t I, int64_t M, int64_t N, int64_t K, int gs, int bits, float* y);
void qo_swiglu_bf16(const float* gate, const float* up, uint16_t* out, int64_t n);
void qo_moe_weighted_sum(const float* y, const float* scores, const int64_t* inv, int64_t T, int64_t k, int64_t H, int as_bf16,
                         float* out);
void qo_kv_decode_attention(const float* q, const uint32_t* kq, const uint16_t* ks, const uint16_t* kb, const uint32_t* vq,
                            const uint16_t* vs, const uint16_t* vb, int64_t B, int64_t Hq, int64_t Hkv, int64_t T, int64_t D,
                            int64_t Dv, int gs, int bits, const int64_t* kq_str, const int64_t* ksb_str, const int64_t* vq_str,
                            const int64_t* vsb_str, float scale, const int32_t* kv_lens, const float* mask, float* out);
}

using namespace qb200h;

static uint32_t g_rng = 12345u;
static float frand() {   // uniform in [-1, 1): enough structure for parity, no <random> dependence on the platform
  g_rng = g_rng * 1664525u + 1013904223u;
  return (float)((g_rng >> 8) & 0xFFFF) / 32768.0f - 1.0f;
}
static std::vector<float> rand_bf16(size_t n, float amp) {
  std::vector<float> v(n);
  for (auto& x : v) x = frand() * amp;
  std::vector<uint16_t> h(n);
  qo_f32_to_bf16(v.data(), h.data(), (int64_t)n);
  qo_bf16_to_f32(h.data(), v.data(), (int64_t)n);
  return v;
}
template <typename T> static T* to_dev(const std::vector<T>& h) {
  T* d = nullptr;
  if (cudaMalloc((void**)&d, h.size() * sizeof(T)) != cudaSuccess) { std::fprintf(stderr, "cudaMalloc failed\n"); std::exit(2); }
  cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
  return d;
}
template <typename T> static T* dev_alloc(size_t n) {
  T* d = nullptr;
  if (cudaMalloc((void**)&d, n * sizeof(T)) != cudaSuccess) { std::fprintf(stderr, "cudaMalloc failed\n"); std::exit(2); }
  cudaMemset(d, 0, n * sizeof(T));
  return d;
}
template <typename T> static std::vector<T> to_host(const T* d, size_t n) {
  std::vector<T> h(n);
  cudaMemcpy(h.data(), d, n * sizeof(T), cudaMemcpyDeviceToHost);
  return h;
}
static std::vector<uint16_t> bf16_of(const std::vector<float>& v) {
  std::vector<uint16_t> h(v.size());
  qo_f32_to_bf16(v.data(), h.data(), (int64_t)v.size());
  return h;
}
static std::vector<float> f32_of(const std::vector<uint16_t>& h) {
  std::vector<float> v(h.size());
  qo_bf16_to_f32(h.data(), v.data(), (int64_t)h.size());
  return v;
}
// max |got - ref| <= tol * rms(ref) + half a bf16 ulp of the largest value
static bool gate(const std::vector<float>& got, const std::vector<float>& ref, double tol, const char* what) {
  double rms = 0, worst = 0, mx = 0;
  for (size_t i = 0; i < ref.size(); ++i) { rms += (double)ref[i] * ref[i]; mx = std::fmax(mx, std::fabs(ref[i])); }
  rms = std::sqrt(rms / (double)ref.size());
  for (size_t i = 0; i < ref.size(); ++i) {
    if (std::isnan(got[i])) { std::printf("FAIL %s: NaN at %zu\n", what, i); return false; }
    worst = std::fmax(worst, std::fabs((double)got[i] - ref[i]));
  }
  const bool ok = worst <= tol * rms + mx / 256.0;
  std::printf("%s %s: max|d| %.3e, rms %.3e\n", ok ? "ok  " : "FAIL", what, worst, rms);
  return ok;
}

int main(int argc, char** argv) {
  if (argc > 1 && std::strcmp(argv[1], "--link-only") == 0) {
    std::printf("linked against %s\n", qb200_version());
    return 0;
  }
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { std::fprintf(stderr, "no CUDA device\n"); return 3; }
  cudaSetDevice(0);
  qb200_stream stream = nullptr;
  bool ok = true;
  const int gs = 64, bits = 4;

  // ---- quantizeAffine / dequantizeAffine (src/kv_quant.zig:126-162, :407-430): bit-exact vs the oracle ----
  const int64_t N = 512, K = 1024;
  std::vector<float> w = rand_bf16((size_t)(N * K), 0.05f);
  std::vector<uint32_t> q((size_t)(N * K * bits / 32));
  std::vector<uint16_t> s((size_t)(N * K / gs)), b((size_t)(N * K / gs));
  qo_quantize(w.data(), N, K, gs, bits, q.data(), s.data(), b.data());
  QuantizedKV qw;
  uint16_t* d_w = to_dev(bf16_of(w));
  qw.q = Array(dev_alloc<uint32_t>(q.size()), QB200_UINT32, {N, K * bits / 32});
  qw.scales = Array(dev_alloc<uint16_t>(s.size()), QB200_BFLOAT16, {N, K / gs});
  qw.biases = Array(dev_alloc<uint16_t>(b.size()), QB200_BFLOAT16, {N, K / gs});
  try {
    quantizeAffine(qw, Array(d_w, QB200_BFLOAT16, {N, K}), stream);
    cudaDeviceSynchronize();
    const bool same = to_host((uint32_t*)qw.q.t.data, q.size()) == q && to_host((uint16_t*)qw.scales.t.data, s.size()) == s &&
                      to_host((uint16_t*)qw.biases.t.data, b.size()) == b;
    std::printf("%s quantizeAffine: codes, scales and biases bit-exact\n", same ? "ok  " : "FAIL");
    ok = ok && same;

    // ---- qmatmulBits at one token and at 64 tokens (src/transformer.zig:20894-20983) ----
    QWeight qwt;
    qwt.q = qw.q; qwt.scales = qw.scales; qwt.biases = qw.biases;
    for (int64_t M : {int64_t(1), int64_t(64)}) {
      std::vector<float> x = rand_bf16((size_t)(M * K), 1.0f), ref((size_t)(M * N));
      if (M == 1) qo_qmm_t(x.data(), q.data(), s.data(), b.data(), M, N, K, gs, bits, ref.data());
      else qo_qmm_t_bf16w(x.data(), q.data(), s.data(), b.data(), M, N, K, gs, bits, ref.data());
      Array dx(to_dev(bf16_of(x)), QB200_BFLOAT16, {M, K}), dy(dev_alloc<uint16_t>((size_t)(M * N)), QB200_BFLOAT16, {M, N});
      qmatmulBits(dy, dx, qwt, stream);
      cudaDeviceSynchronize();
      ok = gate(f32_of(to_host((uint16_t*)dy.t.data, (size_t)(M * N))), ref, 1e-2, M == 1 ? "qmatmulBits M=1" : "qmatmulBits M=64") && ok;
    }

    // ---- gatherExpertMm on rows sorted by expert (src/transformer.zig:20763-20784, :15007-15035) ----
    {
      const int64_t E = 4, EN = 128, I = 12;
      std::vector<float> bank = rand_bf16((size_t)(E * EN * K), 0.05f);
      std::vector<uint32_t> bq((size_t)(E * EN * K * bits / 32));
      std::vector<uint16_t> bs((size_t)(E * EN * K / gs)), bb(bs.size());
      qo_quantize(bank.data(), E * EN, K, gs, bits, bq.data(), bs.data(), bb.data());
      QWeight qb_;
      qb_.q = Array(to_dev(bq), QB200_UINT32, {E, EN, K * bits / 32});
      qb_.scales = Array(to_dev(bs), QB200_BFLOAT16, {E, EN, K / gs});
      qb_.biases = Array(to_dev(bb), QB200_BFLOAT16, {E, EN, K / gs});
      std::vector<int64_t> rhs = {0, 0, 0, 1, 1, 2, 2, 2, 2, 3, 3, 3}, lhs(I);
      for (int64_t i = 0; i < I; ++i) lhs[i] = i;
      std::vector<float> x = rand_bf16((size_t)(I * K), 1.0f), ref((size_t)(I * EN));
      qo_gather_qmm_t(x.data(), bq.data(), bs.data(), bb.data(), lhs.data(), rhs.data(), I, 1, EN, K, gs, bits, ref.data());
      Array dx(to_dev(bf16_of(x)), QB200_BFLOAT16, {I, 1, K}), dr(to_dev(rhs), QB200_INT64, {I});
      Array dy(dev_alloc<uint16_t>((size_t)(I * EN)), QB200_BFLOAT16, {I, 1, EN});
      gatherExpertMm(dy, dx, qb_, nullptr, dr, true, stream);
      cudaDeviceSynchronize();
      ok = gate(f32_of(to_host((uint16_t*)dy.t.data, (size_t)(I * EN))), ref, 1e-2, "gatherExpertMm (sorted)") && ok;

      // ---- the same rows through gate and up banks with fusedSwiGLU (src/transformer.zig:15007-15035, :19925-19931) ----
      std::vector<float> bank2 = rand_bf16((size_t)(E * EN * K), 0.05f), ref2((size_t)(I * EN));
      std::vector<uint32_t> uq(bq.size());
      std::vector<uint16_t> us(bs.size()), ub(bs.size());
      qo_quantize(bank2.data(), E * EN, K, gs, bits, uq.data(), us.data(), ub.data());
      QWeight qu_;
      qu_.q = Array(to_dev(uq), QB200_UINT32, {E, EN, K * bits / 32});
      qu_.scales = Array(to_dev(us), QB200_BFLOAT16, {E, EN, K / gs});
      qu_.biases = Array(to_dev(ub), QB200_BFLOAT16, {E, EN, K / gs});
      qo_gather_qmm_t(x.data(), uq.data(), us.data(), ub.data(), lhs.data(), rhs.data(), I, 1, EN, K, gs, bits, ref2.data());
      std::vector<uint16_t> act16((size_t)(I * EN));
      qo_swiglu_bf16(ref.data(), ref2.data(), act16.data(), I * EN);
      Array da(dev_alloc<uint16_t>((size_t)(I * EN)), QB200_BFLOAT16, {I, 1, EN});
      gatherExpertGateUpSwiGLU(da, dx, qb_, qu_, nullptr, dr, true, stream);
      cudaDeviceSynchronize();
      ok = gate(f32_of(to_host((uint16_t*)da.t.data, (size_t)(I * EN))), f32_of(act16), 2e-2, "gatherExpertGateUpSwiGLU") && ok;

      // ---- rows back to token order, times the scores, summed over top-k (src/transformer.zig:15036-15042, :15127-15140) ----
      const int64_t T = 4, topk = 3;   // I = T * topk rows
      std::vector<int64_t> inv = {5, 0, 9, 1, 6, 10, 2, 7, 11, 3, 4, 8};
      std::vector<float> yrows = f32_of(to_host((uint16_t*)da.t.data, (size_t)(I * EN))), sc = rand_bf16((size_t)(T * topk), 1.0f);
      std::vector<float> sref((size_t)(T * EN));
      qo_moe_weighted_sum(yrows.data(), sc.data(), inv.data(), T, topk, EN, 1, sref.data());
      Array dsc(to_dev(bf16_of(sc)), QB200_BFLOAT16, {T, topk}), dinv(to_dev(inv), QB200_INT64, {I});
      Array dsum(dev_alloc<uint16_t>((size_t)(T * EN)), QB200_BFLOAT16, {T, EN});
      moeWeightedSum(dsum, da, dsc, &dinv, stream);
      cudaDeviceSynchronize();
      std::vector<float> got = f32_of(to_host((uint16_t*)dsum.t.data, (size_t)(T * EN)));
      bool exact = true;
      for (size_t i = 0; i < got.size(); ++i) exact = exact && got[i] == sref[i];
      std::printf("%s moeWeightedSum: bit-exact against the oracle\n", exact ? "ok  " : "FAIL");
      ok = ok && exact;
    }

    // ---- KVCache.updateAffine + quantAttention over strided views (src/transformer.zig:3224-3337, src/kv_quant.zig:478-687) ----
    {
      const int64_t B = 2, Hq = 8, Hkv = 2, D = 128, cap = 512, T = 300;
      KVCacheEntry e;
      for (QuantizedKV* c : {&e.keys, &e.values}) {
        c->q = Array(dev_alloc<uint32_t>((size_t)(B * Hkv * cap * D * bits / 32)), QB200_UINT32, {B, Hkv, cap, D * bits / 32});
        c->scales = Array(dev_alloc<uint16_t>((size_t)(B * Hkv * cap * D / gs)), QB200_BFLOAT16, {B, Hkv, cap, D / gs});
        c->biases = Array(dev_alloc<uint16_t>((size_t)(B * Hkv * cap * D / gs)), QB200_BFLOAT16, {B, Hkv, cap, D / gs});
      }
      std::vector<float> kd = rand_bf16((size_t)(B * Hkv * T * D), 1.0f), vd = rand_bf16((size_t)(B * Hkv * T * D), 1.0f);
      // prefill of 299 tokens, then one decode token: two appends, as the reference's cache sees them
      auto rows = [&](const std::vector<float>& src, int64_t t0, int64_t n) {
        std::vector<float> out((size_t)(B * Hkv * n * D));
        for (int64_t bh = 0; bh < B * Hkv; ++bh)
          std::memcpy(&out[(size_t)(bh * n * D)], &src[(size_t)((bh * T + t0) * D)], sizeof(float) * (size_t)(n * D));
        return out;
      };
      for (auto [t0, n] : {std::pair<int64_t, int64_t>{0, T - 1}, std::pair<int64_t, int64_t>{T - 1, 1}}) {
        Array kn(to_dev(bf16_of(rows(kd, t0, n))), QB200_BFLOAT16, {B, Hkv, n, D});
        Array vn(to_dev(bf16_of(rows(vd, t0, n))), QB200_BFLOAT16, {B, Hkv, n, D});
        updateAffine(e, kn, vn, stream);
      }
      std::vector<uint32_t> kq((size_t)(B * Hkv * T * D * bits / 32)), vq(kq.size());
      std::vector<uint16_t> ks((size_t)(B * Hkv * T * D / gs)), kb(ks.size()), vs(ks.size()), vb(ks.size());
      qo_quantize(kd.data(), B * Hkv * T, D, gs, bits, kq.data(), ks.data(), kb.data());
      qo_quantize(vd.data(), B * Hkv * T, D, gs, bits, vq.data(), vs.data(), vb.data());
      std::vector<float> qv = rand_bf16((size_t)(B * Hq * D), 1.0f), ref((size_t)(B * Hq * D));
      std::vector<int32_t> lens = {(int32_t)T, 123};
      const int64_t qstr[3] = {Hkv * T * (D * bits / 32), T * (D * bits / 32), D * bits / 32};
      const int64_t sstr[3] = {Hkv * T * (D / gs), T * (D / gs), D / gs};
      const float scale = 1.0f / std::sqrt((float)D);
      qo_kv_decode_attention(qv.data(), kq.data(), ks.data(), kb.data(), vq.data(), vs.data(), vb.data(), B, Hq, Hkv, T, D, D, gs,
                             bits, qstr, sstr, qstr, sstr, scale, lens.data(), nullptr, ref.data());
      Array dq(to_dev(bf16_of(qv)), QB200_BFLOAT16, {B, Hq, 1, D}), dl(to_dev(lens), QB200_INT32, {B});
      Array out(dev_alloc<uint16_t>((size_t)(B * Hq * D)), QB200_BFLOAT16, {B, Hq, 1, D});
      const size_t need = quantAttentionWorkspace(B, Hq, Hkv, e.offset, D);
      void* ws = dev_alloc<char>(need);
      quantAttention(out, dq, e.view(e.keys), e.view(e.values), scale, nullptr, &dl, ws, need, stream);
      cudaDeviceSynchronize();
      ok = (e.offset == T) && ok;
      ok = gate(f32_of(to_host((uint16_t*)out.t.data, (size_t)(B * Hq * D))), ref, 1e-2, "updateAffine + quantAttention") && ok;
    }

    // ---- a declined request surfaces as Declined, not as a crash (src/transformer.zig:20463-20475) ----
    {
      QWeight odd = QWeight{qw.q, qw.scales, qw.biases, 64, 3};   // 3-bit codes are not served
      Array dx(dev_alloc<uint16_t>((size_t)K), QB200_BFLOAT16, {1, K}), dy(dev_alloc<uint16_t>((size_t)N), QB200_BFLOAT16, {1, N});
      bool declined = false;
      try { qmatmulBits(dy, dx, odd, stream); } catch (const Declined&) { declined = true; } catch (const Error&) { declined = true; }
      std::printf("%s unsupported width is refused with an error\n", declined ? "ok  " : "FAIL");
      ok = ok && declined;
    }
  } catch (const Error& err) {
    std::printf("FAIL: qb200 error %d: %s\n", err.status, err.what());
    return 1;
  }
  if (cudaDeviceSynchronize() != cudaSuccess) { std::printf("FAIL: CUDA error at exit\n"); return 1; }
  std::printf(ok ? "host self-test passed\n" : "host self-test FAILED\n");
  return ok ? 0 : 1;
}
