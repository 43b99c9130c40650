// Drop-in check: the reference's own operator layer (tfcc::blas::matmul, tfcc::data::set/get,
// Variable, Shape -- all compiled from the reference sources) running on the B200 backend.
// It replays the cases of the reference's tests (tfcc/test/blas.cpp:34-61: four batch layouts
// with m,n,k in [1,100), with and without bias; tfcc/test/quantization.cpp:191-218: raw u8/s8
// operands, exact int32 result) with a seeded generator and compares against double / int64
// host loops, using the reference's is_similar predicate for floats.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <string>
#include <tuple>
#include <random>
#include <vector>

#include "tfcc_b200.h"

namespace {

// Weights served from memory, the way an .npz file would serve them
// (tfcc/core/dataloaders/tfcc_dataloader.h:24-57): name -> (shape, type tag, raw bytes).
class MemoryLoader : public tfcc::DataLoader {
  std::map<std::string, std::tuple<tfcc::Shape, std::string, std::string>> _data;

 public:
  template <class T>
  void add(const std::string& name, std::vector<unsigned> shape, const std::vector<T>& values,
           const char* type) {
    std::string raw(reinterpret_cast<const char*>(values.data()), values.size() * sizeof(T));
    _data[name] = std::make_tuple(tfcc::Shape(std::move(shape)), std::string(type), std::move(raw));
  }
  const std::tuple<tfcc::Shape, std::string, std::string>& loadData(
      const std::string& name) const override {
    auto it = _data.find(name);
    if (it == _data.end()) throw tfcc::RuntimeError("no such constant: " + name);
    return it->second;
  }
  std::vector<std::tuple<std::string, std::string>> getAllNames() const override {
    std::vector<std::tuple<std::string, std::string>> names;
    for (const auto& kv : _data) names.emplace_back(kv.first, std::get<1>(kv.second));
    return names;
  }
  bool hasData(const std::string& name) const override { return _data.count(name) != 0; }
};

int g_failures = 0;
int g_cases = 0;

void expect(bool ok, const char* what) {
  ++g_cases;
  if (!ok) {
    ++g_failures;
    std::printf("FAIL: %s\n", what);
  }
}

std::vector<float> host_matmul(const std::vector<float>& a, const std::vector<float>& b,
                               const std::vector<float>* bias, unsigned batch, unsigned m,
                               unsigned n, unsigned k, bool aBatched, bool bBatched) {
  std::vector<float> c(static_cast<size_t>(batch) * m * n);
  for (unsigned bt = 0; bt < batch; ++bt) {
    const float* pa = a.data() + (aBatched ? static_cast<size_t>(bt) * m * k : 0);
    const float* pb = b.data() + (bBatched ? static_cast<size_t>(bt) * k * n : 0);
    for (unsigned i = 0; i < m; ++i)
      for (unsigned j = 0; j < n; ++j) {
        double s = bias ? (*bias)[j] : 0.0;
        for (unsigned kk = 0; kk < k; ++kk) s += static_cast<double>(pa[i * k + kk]) * pb[kk * n + j];
        c[(static_cast<size_t>(bt) * m + i) * n + j] = static_cast<float>(s);
      }
  }
  return c;
}

// Normwise relative error <= 1e-5 always; for the reference-sized cases (k < 100) also the
// reference's elementwise predicate tfcc::is_similar (tfcc/core/utils/tfcc_debugutils.cpp:102-127).
// With k in the hundreds an element that happens to land near zero misses that predicate in
// any fp32 implementation, which is why the reference only applies it to small k.
bool close_enough(const std::vector<float>& got, const std::vector<float>& want, bool elementwise) {
  if (got.size() != want.size()) return false;
  double num = 0, den = 0;
  for (size_t i = 0; i < got.size(); ++i) {
    const double d = std::fabs(static_cast<double>(got[i]) - want[i]);
    if (elementwise &&
        !(d < 1e-3 * std::fabs(static_cast<double>(got[i]) + want[i]) || d < 1e-5))
      return false;
    num += d * d;
    den += static_cast<double>(want[i]) * want[i];
  }
  return den == 0 || std::sqrt(num / den) < 1e-5;
}

void fp32_case(std::mt19937& rng, std::vector<unsigned> sa, std::vector<unsigned> sb, bool withBias) {
  std::uniform_real_distribution<float> u(-1.f, 1.f);
  size_t na = 1, nb = 1;
  for (unsigned d : sa) na *= d;
  for (unsigned d : sb) nb *= d;
  std::vector<float> ha(na), hb(nb);
  for (auto& x : ha) x = u(rng);
  for (auto& x : hb) x = u(rng);
  const unsigned m = sa[sa.size() - 2], k = sa.back(), n = sb.back();
  std::vector<float> hbias(n);
  for (auto& x : hbias) x = u(rng);

  tfcc::Variable<float> a{tfcc::Shape(sa)}, b{tfcc::Shape(sb)}, bias({n});
  tfcc::data::set(a, ha);
  tfcc::data::set(b, hb);
  tfcc::data::set(bias, hbias);
  tfcc::Variable<float> c = withBias ? tfcc::blas::matmul(a, b, bias) : tfcc::blas::matmul(a, b);
  std::vector<float> got = tfcc::data::get(c);
  const unsigned batch = c.size() / (m * n);
  std::vector<float> want =
      host_matmul(ha, hb, withBias ? &hbias : nullptr, batch, m, n, k, sa.size() > 2, sb.size() > 2);
  char label[160];
  std::snprintf(label, sizeof label, "fp32 matmul rankA=%zu rankB=%zu m=%u n=%u k=%u bias=%d",
                sa.size(), sb.size(), m, n, k, withBias ? 1 : 0);
  expect(close_enough(got, want, k < 100), label);
}

void int8_case(std::mt19937& rng, unsigned m, unsigned n, unsigned k, float minA, float maxA,
               float minB, float maxB) {
  std::uniform_int_distribution<int> ua(0, 255), ub(-128, 127);
  std::vector<uint8_t> ha(static_cast<size_t>(m) * k);
  std::vector<int8_t> hb(static_cast<size_t>(k) * n);
  for (auto& x : ha) x = static_cast<uint8_t>(ua(rng));
  for (auto& x : hb) x = static_cast<int8_t>(ub(rng));
  tfcc::Variable<uint8_t> a({m, k});
  tfcc::Variable<int8_t> b({k, n});
  tfcc::Variable<float> vminA({1}), vmaxA({1}), vminB({1}), vmaxB({1});
  tfcc::data::set(a, ha);
  tfcc::data::set(b, hb);
  tfcc::data::set(vminA, {minA});
  tfcc::data::set(vmaxA, {maxA});
  tfcc::data::set(vminB, {minB});
  tfcc::data::set(vmaxB, {maxB});
  tfcc::Variable<int32_t> ra = tfcc::b200::quantization::reduce_sum(a, true);
  tfcc::Variable<int32_t> rb = tfcc::b200::quantization::reduce_sum(b, false);
  tfcc::Variable<int32_t> c;
  tfcc::Variable<float> minC, maxC;
  std::tie(c, minC, maxC) =
      tfcc::b200::quantization::matmul(a, ra, vminA, vmaxA, b, rb, vminB, vmaxB);
  std::vector<int32_t> got = tfcc::data::get(c);

  // offsets as the reference's generator derives them
  // (tfcc/test/python/testcase/quantization/mklquantizationmatmul.py:25-48)
  auto offset = [](float mn, float mx) {
    const double scale = 256.0 / ((static_cast<double>(mx - mn)) * (256.0 / 255.0));
    return static_cast<int64_t>(std::llround(mn * scale));
  };
  const int64_t offA = offset(minA, maxA), offB = offset(minB, maxB) + 128;
  bool ok = got.size() == static_cast<size_t>(m) * n;
  for (unsigned i = 0; ok && i < m; ++i)
    for (unsigned j = 0; j < n; ++j) {
      int64_t s = 0;
      for (unsigned kk = 0; kk < k; ++kk)
        s += (static_cast<int64_t>(ha[i * k + kk]) + offA) * (static_cast<int64_t>(hb[kk * n + j]) + offB);
      if (static_cast<int32_t>(static_cast<uint32_t>(s)) != got[i * n + j]) {
        ok = false;
        break;
      }
    }
  char label[128];
  std::snprintf(label, sizeof label, "int8 matmul m=%u n=%u k=%u", m, n, k);
  expect(ok, label);
}

}  // namespace

int main() {
  try {
    tfcc::initialize_b200();
    std::mt19937 rng(20240607);
    std::uniform_int_distribution<unsigned> dim(1, 99), bs(1, 5);
    for (int rep = 0; rep < 5; ++rep) {
      for (int bias = 0; bias < 2; ++bias) {
        unsigned m = dim(rng), n = dim(rng), k = dim(rng), b = bs(rng);
        fp32_case(rng, {m, k}, {k, n}, bias);
        fp32_case(rng, {b, m, k}, {k, n}, bias);
        fp32_case(rng, {m, k}, {b, k, n}, bias);
        fp32_case(rng, {b, m, k}, {b, k, n}, bias);
      }
    }
    // shapes that take the tensor-core, CTA-pair and streaming kernels
    fp32_case(rng, {8, 128, 768}, {768, 3072}, true);
    fp32_case(rng, {96, 128, 64}, {96, 64, 128}, false);
    fp32_case(rng, {1024, 512}, {512, 2048}, false);
    fp32_case(rng, {4, 1024}, {1024, 4096}, true);

    int8_case(rng, 256, 384, 512, -1.5f, 2.0f, -0.7f, 0.9f);
    int8_case(rng, 130, 72, 301, -3.f, 1.f, 0.25f, 4.f);
    int8_case(rng, 333, 1, 401, -4.f, -1.f, 0.5f, 3.f);

    // QuantizationTest.mkl_matmul / 2 / 3 (tfcc/test/quantization.cpp:105-189): quantize ->
    // reduce_sum -> matmul -> dequantize through the reference's operator layer, all on the
    // device; the truncated results must be 5, 11, 17 twice
    {
      struct Layout { std::vector<unsigned> sa, sb; std::vector<float> a, b; };
      const std::vector<float> six = {1, 2, 3, 4, 5, 6}, twelve = {1, 2, 3, 4, 5, 6, 1, 2, 3, 4, 5, 6};
      const Layout layouts[3] = {{{2, 3, 2}, {2, 2, 1}, twelve, {1, 2, 1, 2}},
                                 {{3, 2}, {2, 2, 1}, six, {1, 2, 1, 2}},
                                 {{2, 3, 2}, {2, 1}, twelve, {1, 2}}};
      for (const Layout& l : layouts) {
        tfcc::Variable<float> v1{tfcc::Shape(l.sa)}, v2{tfcc::Shape(l.sb)};
        tfcc::data::set(v1, l.a);
        tfcc::data::set(v2, l.b);
        tfcc::Variable<uint8_t> qa;
        tfcc::Variable<int8_t> qb;
        tfcc::Variable<float> minA, maxA, minB, maxB, minC, maxC;
        std::tie(qa, minA, maxA) = tfcc::quantization::quantize<uint8_t>(v1);
        std::tie(qb, minB, maxB) = tfcc::quantization::quantize<int8_t>(v2);
        tfcc::Variable<int32_t> ra = tfcc::b200::quantization::reduce_sum(qa, true);
        tfcc::Variable<int32_t> rb = tfcc::b200::quantization::reduce_sum(qb, false);
        tfcc::Variable<int32_t> qc;
        std::tie(qc, minC, maxC) = tfcc::b200::quantization::matmul(qa, ra, minA, maxA, qb, rb, minB, maxB);
        std::vector<float> vr = tfcc::data::get(tfcc::quantization::dequantize(qc, minC, maxC));
        const int want[6] = {5, 11, 17, 5, 11, 17};
        bool ok = vr.size() == 6;
        for (int i = 0; ok && i < 6; ++i) ok = static_cast<int>(vr[i]) == want[i];
        expect(ok, "quantized dense layer known answers 5/11/17");
      }
      // QuantizationTest.dequantize / requantize (tfcc/test/quantization.cpp:60-102)
      tfcc::Variable<int8_t> q({6});
      tfcc::data::set(q, {23, -115, -128, 127, -20, -11});
      tfcc::Variable<float> mn({1}), mx({1}), mno({1}), mxo({1});
      tfcc::data::set(mn, {-2.5f});
      tfcc::data::set(mx, {3.4f});
      tfcc::data::set(mno, {-12.7f});
      tfcc::data::set(mxo, {24.5f});
      std::vector<float> dq = tfcc::data::get(tfcc::quantization::dequantize(q, mn, mx));
      const float dq_want[6] = {9.9372554e-01f, -2.1992157e+00f, -2.5000000e+00f,
                                3.4000001e+00f, -1.1765957e-03f, 2.0705891e-01f};
      bool ok = dq.size() == 6;
      for (int i = 0; ok && i < 6; ++i) ok = std::fabs(dq[i] - dq_want[i]) < 1e-5f;
      expect(ok, "dequantize known answers");
      std::vector<uint16_t> rq =
          tfcc::data::get(tfcc::quantization::requantize<uint16_t>(q, mn, mx, mno, mxo));
      const uint16_t rq_want[6] = {24125, 18500, 17970, 28364, 22372, 22739};
      ok = rq.size() == 6;
      for (int i = 0; ok && i < 6; ++i) ok = rq[i] == rq_want[i];
      expect(ok, "requantize known answers");
    }

    // the glue operators of an attention block through the reference's operator layer:
    // tfcc::base::transpose, tfcc::math::softmax, tfcc::math::gelu_accurate,
    // tfcc::nn::layer_normalization
    {
      std::uniform_real_distribution<float> u(-2.f, 2.f);
      const unsigned B = 2, H = 3, S = 20, D = 16;
      std::vector<float> hx(B * S * H * D);
      for (auto& v : hx) v = u(rng);
      tfcc::Variable<float> x({B, S, H, D});
      tfcc::data::set(x, hx);
      std::vector<float> t1 = tfcc::data::get(tfcc::base::transpose(x, {0, 2, 1, 3}));
      bool ok = true;
      for (unsigned b = 0; b < B; ++b)
        for (unsigned s = 0; s < S; ++s)
          for (unsigned h = 0; h < H; ++h)
            for (unsigned d = 0; d < D; ++d)
              ok = ok && t1[((b * H + h) * S + s) * D + d] == hx[((b * S + s) * H + h) * D + d];
      expect(ok, "transpose perm (0,2,1,3)");
      std::vector<float> t2 = tfcc::data::get(tfcc::base::transpose(x, {0, 1, 3, 2}));
      ok = true;
      for (unsigned o = 0; o < B * S; ++o)
        for (unsigned h = 0; h < H; ++h)
          for (unsigned d = 0; d < D; ++d)
            ok = ok && t2[(o * D + d) * H + h] == hx[(o * H + h) * D + d];
      expect(ok, "transpose of the last two axes");

      tfcc::Variable<float> m({7, 33});
      std::vector<float> hm(7 * 33);
      for (auto& v : hm) v = u(rng);
      tfcc::data::set(m, hm);
      std::vector<float> sm = tfcc::data::get(tfcc::math::softmax(m, 1));
      std::vector<float> ge = tfcc::data::get(tfcc::math::gelu_accurate(m));
      std::vector<float> sm_want(hm.size()), ge_want(hm.size());
      for (unsigned r = 0; r < 7; ++r) {
        float mx = hm[r * 33];
        for (unsigned c = 1; c < 33; ++c) mx = std::max(mx, hm[r * 33 + c]);
        double sum = 0;
        for (unsigned c = 0; c < 33; ++c) sum += std::exp(static_cast<double>(hm[r * 33 + c]) - mx);
        for (unsigned c = 0; c < 33; ++c)
          sm_want[r * 33 + c] = static_cast<float>(std::exp(static_cast<double>(hm[r * 33 + c]) - mx) / sum);
      }
      for (size_t i = 0; i < hm.size(); ++i)
        ge_want[i] = static_cast<float>(0.5 * hm[i] * (1.0 + std::erf(hm[i] / std::sqrt(2.0))));
      expect(close_enough(sm, sm_want, true), "softmax over the last axis");
      expect(close_enough(ge, ge_want, true), "gelu_accurate");

      tfcc::Variable<float> gamma({33}), beta({33});
      std::vector<float> hg(33), hb(33);
      for (auto& v : hg) v = 1.f + 0.25f * u(rng);
      for (auto& v : hb) v = 0.1f * u(rng);
      tfcc::data::set(gamma, hg);
      tfcc::data::set(beta, hb);
      std::vector<float> ln = tfcc::data::get(tfcc::nn::layer_normalization(m, gamma, beta, 1e-5f, 1));
      std::vector<float> ln_want(hm.size());
      for (unsigned r = 0; r < 7; ++r) {
        double mean = 0, var = 0;
        for (unsigned c = 0; c < 33; ++c) mean += hm[r * 33 + c];
        mean /= 33;
        for (unsigned c = 0; c < 33; ++c) var += (hm[r * 33 + c] - mean) * (hm[r * 33 + c] - mean);
        var /= 33;
        for (unsigned c = 0; c < 33; ++c)
          ln_want[r * 33 + c] =
              static_cast<float>((hm[r * 33 + c] - mean) / std::sqrt(var + 1e-5) * hg[c] + hb[c]);
      }
      expect(close_enough(ln, ln_want, true), "layer_normalization");
    }

    // one-kernel attention on a packed Q/K/V tensor against the double-precision formula
    {
      const unsigned batch = 2, seq = 77, heads = 3, dim = 64, width = heads * dim;
      std::uniform_real_distribution<float> u(-1.f, 1.f);
      std::vector<float> h(static_cast<size_t>(batch) * seq * 3 * width);
      for (auto& x : h) x = u(rng);
      tfcc::Variable<float> qkv({batch, seq, 3 * width});
      tfcc::data::set(qkv, h);
      std::vector<float> got = tfcc::data::get(tfcc::b200::attention_packed(qkv, heads, 0.125f));
      std::vector<float> want(static_cast<size_t>(batch) * seq * width);
      auto at = [&](unsigned b, unsigned s, unsigned which, unsigned hd, unsigned d) {
        return static_cast<double>(h[(static_cast<size_t>(b) * seq + s) * 3 * width + which * width + hd * dim + d]);
      };
      for (unsigned b = 0; b < batch; ++b)
        for (unsigned hd = 0; hd < heads; ++hd)
          for (unsigned i = 0; i < seq; ++i) {
            std::vector<double> p(seq);
            double mx = -1e300, sum = 0;
            for (unsigned j = 0; j < seq; ++j) {
              double sc = 0;
              for (unsigned d = 0; d < dim; ++d) sc += at(b, i, 0, hd, d) * at(b, j, 1, hd, d);
              p[j] = sc * 0.125;
              mx = std::max(mx, p[j]);
            }
            for (unsigned j = 0; j < seq; ++j) sum += (p[j] = std::exp(p[j] - mx));
            for (unsigned d = 0; d < dim; ++d) {
              double o = 0;
              for (unsigned j = 0; j < seq; ++j) o += p[j] / sum * at(b, j, 2, hd, d);
              want[(static_cast<size_t>(b) * seq + i) * width + hd * dim + d] = static_cast<float>(o);
            }
          }
      expect(close_enough(got, want, false), "fused attention on a packed Q/K/V tensor");
    }

    // derived constants computed once: column sums of an int8 weight, joined projection weights
    {
      const unsigned k = 96, n = 80;
      std::uniform_int_distribution<int> w8(-127, 127);
      std::vector<int8_t> hw(static_cast<size_t>(k) * n);
      for (auto& x : hw) x = static_cast<int8_t>(w8(rng));
      MemoryLoader* loader = new MemoryLoader();  // lives as long as the process, like the global it becomes
      loader->add<int8_t>("qweight", {k, n}, hw, "i1");
      tfcc::DataLoader::setGlobalDefault(loader);
      const tfcc::Constant<int32_t>& sums = tfcc::b200::cached_column_sums("qweight");
      const tfcc::Constant<int32_t>& again = tfcc::b200::cached_column_sums("qweight");
      std::vector<int32_t> got = tfcc::data::get(sums);
      bool ok = got.size() == n && &sums == &again;
      for (unsigned j = 0; ok && j < n; ++j) {
        int32_t want = 0;
        for (unsigned i = 0; i < k; ++i) want += hw[static_cast<size_t>(i) * n + j];
        ok = got[j] == want;
      }
      expect(ok, "cached column sums of an int8 constant");

      std::vector<float> wa(6 * 4), wb(6 * 2);
      for (size_t i = 0; i < wa.size(); ++i) wa[i] = static_cast<float>(i);
      for (size_t i = 0; i < wb.size(); ++i) wb[i] = 100.f + static_cast<float>(i);
      loader->add<float>("wa", {6, 4}, wa, "f4");
      loader->add<float>("wb", {6, 2}, wb, "f4");
      const tfcc::Constant<float>& joined = tfcc::b200::cached_concat_columns("wab", {"wa", "wb"});
      std::vector<float> hj = tfcc::data::get(joined);
      bool okj = joined.shape().size() == 2 && joined.shape(0) == 6 && joined.shape(1) == 6;
      for (unsigned r = 0; okj && r < 6; ++r)
        for (unsigned c = 0; okj && c < 6; ++c)
          okj = hj[r * 6 + c] == (c < 4 ? wa[r * 4 + c] : wb[r * 2 + (c - 4)]);
      expect(okj, "projection weights joined along their columns, cached");
    }

    // the N split over a device group: two members (two GPUs when present, else both on GPU 0)
    {
      const unsigned gpus = tfcc::B200Device::getDeviceCount();
      std::vector<unsigned> members = {0u, gpus >= 2 ? 1u : 0u};
      tfcc::b200::parallel::NSplitGroup group(members);
      const unsigned m = 256, n = 272, k = 132;
      std::uniform_real_distribution<float> u(-1.f, 1.f);
      float *pa = nullptr, *pb = nullptr, *pc = nullptr;
      cudaMallocHost(reinterpret_cast<void**>(&pa), sizeof(float) * m * k);
      cudaMallocHost(reinterpret_cast<void**>(&pb), sizeof(float) * k * n);
      cudaMallocHost(reinterpret_cast<void**>(&pc), sizeof(float) * m * n);
      std::vector<float> ha(static_cast<size_t>(m) * k), hb(static_cast<size_t>(k) * n);
      for (auto& x : ha) x = u(rng);
      for (auto& x : hb) x = u(rng);
      std::copy(ha.begin(), ha.end(), pa);
      std::copy(hb.begin(), hb.end(), pb);
      group.matmul_host(pa, pb, pc, m, n, k);
      std::vector<float> got(pc, pc + static_cast<size_t>(m) * n);
      expect(close_enough(got, host_matmul(ha, hb, nullptr, 1, m, n, k, false, false), false),
             "N-split product over a device group, host buffers");
      cudaFreeHost(pa);
      cudaFreeHost(pb);
      cudaFreeHost(pc);
    }

    // error behaviour comes from the reference's operator layer, unchanged
    bool threw = false;
    try {
      tfcc::Variable<float> x({2, 3}), y({4, 5});
      tfcc::blas::matmul(x, y);
    } catch (const tfcc::InvalidArgumentError&) {
      threw = true;
    }
    expect(threw, "shape mismatch raises InvalidArgumentError");
    tfcc::Session::getThreadDefault()->sync();
  } catch (const std::exception& e) {
    std::printf("EXCEPTION: %s\n", e.what());
    return 2;
  }
  std::printf("DROPIN %s: %d cases, %d failures\n", g_failures ? "FAILED" : "OK", g_cases, g_failures);
  return g_failures ? 1 : 0;
}
