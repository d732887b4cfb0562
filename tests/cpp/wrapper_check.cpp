// A C++ host program against include/hexb.h alone, in the shape of the reference's MLIR-file wrappers
// (test/python/mlir/hexkl_linalg_matmul/wrapper.cpp and hexkl_attention/wrapper.cpp of
// qualcomm/hexagon-mlir): seeded inputs ~ N(0, 0.5) rounded to four decimals, one timed call of the
// kernel through the library's host-buffer entry point, an element-by-element check against plain
// scalar loops with the wrappers' tolerances (1e-2 for the matmul, 1e-3 for the attention), and a
// Test_Info block written to the path given on the command line (the format of
// test/utils/dsp/include/test_report.h:43-66).  Exit status 0 = Pass, 1 = Fail, 2 = could not run.
//
//   wrapper_check hexkl_linalg_matmul <report path>      1024 x 64 activations, 64 x 512 weights, fp32 out
//   wrapper_check hexkl_attention <report path>          Q, K, V [1, 1, 1024, 64] fp16, fp32 out, scale 0.5
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "hexb.h"

namespace {

void fill_random(std::vector<_Float16> &v, unsigned seed) {
  std::mt19937 gen(seed);
  std::normal_distribution<float> dist(0.0f, 0.5f);
  for (auto &x : v) x = (_Float16)(std::round(dist(gen) * 10000.0f) / 10000.0f);
}

int write_report(const std::string &path, const char *name, double perf_us, bool pass) {
  FILE *fp = std::fopen(path.c_str(), "w");
  if (!fp) return 1;
  std::fprintf(fp, "Test_Info: {\n\tName:%s\n\tResult:%s\n\tPerf:%f\n\tUnits:%s\n}\n", name, pass ? "Pass" : "Fail",
               perf_us, "microseconds");
  std::fclose(fp);
  return 0;
}

template <typename F>
double time_once_us(F &&f) {
  const auto t0 = std::chrono::steady_clock::now();
  f();
  return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
}

int run_matmul(const std::string &report) {
  const int64_t N = 1024, K = 64, M = 512;  // rows, inner, columns
  std::vector<_Float16> act(N * K), w(K * M);
  std::vector<float> out(N * M, 0.f);
  fill_random(act, 1);
  fill_random(w, 2);
  int st = hexb_matmul_f16_host(act.data(), w.data(), out.data(), N, M, K, HEXB_DT_F32);  // first call: set-up
  if (st != HEXB_OK) {
    std::fprintf(stderr, "hexb_matmul_f16_host: %s %s\n", hexb_status_string(st), hexb_last_cuda_error());
    return 2;
  }
  const double us = time_once_us([&] { st = hexb_matmul_f16_host(act.data(), w.data(), out.data(), N, M, K, HEXB_DT_F32); });
  if (st != HEXB_OK) return 2;
  bool pass = true;
  for (int64_t r = 0; r < N && pass; ++r)
    for (int64_t c = 0; c < M; ++c) {
      float acc = 0.f;
      for (int64_t e = 0; e < K; ++e) acc += (float)act[r * K + e] * (float)w[e * M + c];
      if (std::fabs(out[r * M + c] - acc) > 1e-2f) {
        std::fprintf(stderr, "mismatch at %lld: host %f, library %f\n", (long long)(r * M + c), acc, out[r * M + c]);
        pass = false;
        break;
      }
    }
  if (write_report(report, "hexkl_linalg_matmul", us, pass)) return 2;
  return pass ? 0 : 1;
}

int run_attention(const std::string &report) {
  const int64_t S = 1024, D = 64;
  const float scale = 0.5f;
  std::vector<_Float16> q(S * D), k(S * D), v(S * D);
  fill_random(q, 3);
  fill_random(k, 4);
  fill_random(v, 5);
  // fp16 result through the host entry point, compared in fp32 (the wrapper's kernel writes fp32)
  std::vector<_Float16> out(S * D);
  int st = hexb_attention_fwd_host(HEXB_DT_F16, q.data(), k.data(), v.data(), out.data(), 1, 1, S, D, scale, 0);
  if (st != HEXB_OK) {
    std::fprintf(stderr, "hexb_attention_fwd_host: %s %s\n", hexb_status_string(st), hexb_last_cuda_error());
    return 2;
  }
  const double us = time_once_us(
      [&] { st = hexb_attention_fwd_host(HEXB_DT_F16, q.data(), k.data(), v.data(), out.data(), 1, 1, S, D, scale, 0); });
  if (st != HEXB_OK) return 2;
  // S = Q K^T * scale, row softmax, O = P V, all in fp32 from the fp16 inputs
  std::vector<float> s(S), ref(D);
  bool pass = true;
  for (int64_t i = 0; i < S && pass; ++i) {
    float mx = -INFINITY;
    for (int64_t n = 0; n < S; ++n) {
      float acc = 0.f;
      for (int64_t d = 0; d < D; ++d) acc += (float)q[i * D + d] * (float)k[n * D + d];
      s[n] = acc * scale;
      mx = std::fmax(mx, s[n]);
    }
    float sum = 0.f;
    for (int64_t n = 0; n < S; ++n) {
      s[n] = std::exp(s[n] - mx);
      sum += s[n];
    }
    for (int64_t d = 0; d < D; ++d) {
      float acc = 0.f;
      for (int64_t n = 0; n < S; ++n) acc += s[n] / sum * (float)v[n * D + d];
      // 1e-3 is the wrapper's bound for an fp32 result; half an fp16 ulp of the largest |O| (~0.5) is 2.4e-4
      if (std::fabs((float)out[i * D + d] - acc) > 1e-3f) {
        std::fprintf(stderr, "mismatch at %lld: host %f, library %f\n", (long long)(i * D + d), acc, (float)out[i * D + d]);
        pass = false;
        break;
      }
    }
  }
  if (write_report(report, "hexkl_attention", us, pass)) return 2;
  return pass ? 0 : 1;
}

}  // namespace

int main(int argc, char **argv) {
  if (argc != 3) {
    std::fprintf(stderr, "usage: %s hexkl_linalg_matmul|hexkl_attention <report path>\n", argv[0]);
    return 2;
  }
  if (!std::strcmp(argv[1], "hexkl_linalg_matmul")) return run_matmul(argv[2]);
  if (!std::strcmp(argv[1], "hexkl_attention")) return run_attention(argv[2]);
  std::fprintf(stderr, "unknown case %s\n", argv[1]);
  return 2;
}
