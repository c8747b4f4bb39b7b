// cabi_driver.cc — a C++ caller of the C ABI with nothing in between: includes include/ops_b200.h, links libops_b200.so,
// owns its device memory through the CUDA runtime, and runs benchmark config 1 (rms_norm -> rope on [64 tokens, 32 heads,
// 64], causal fused_softmax on [32, 64, 64]) plus one tensor-core mat_mul and one argmax, each checked against the CPU
// oracle (liboracle.so, test infrastructure).  It is what a Rust `impl Operator` shim does, written in the one compiled
// language this environment has: create -> scheme -> launch on a stream -> destroy, errors as return values
// (the crate's test pattern: operators/src/rms_norm/cuda/mod.rs:286-377).  Exit code 0 = all checks passed.
//
// Build (done by __graft_entry__.build()):
//   g++ -O2 -std=c++17 tests/cabi_driver.cc -I/usr/local/cuda/include -Loperators-rs_b200 -lops_b200 -Loracle -loracle
//       -L/usr/local/cuda/lib64 -lcudart -Wl,-rpath,... -o tests/cabi_driver
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../include/ops_b200.h"

typedef _Float16 f16;
typedef ptrdiff_t isz;
typedef size_t usz;

// the oracle's entry points used here (oracle/oracle.cc)
extern "C" {
int orc_rms_norm(uint32_t dt_a, uint32_t dt_w, usz n, usz d, void *y, isz nsy, isz dsy, const void *x, isz nsx, isz dsx, const void *w, isz dsw,
                 float eps);
int orc_rope(uint32_t dt_t, uint32_t dt_p, usz nt, usz nh, usz dh, void *t, isz st, isz sh, const void *p, isz sp, float theta);
int orc_fused_softmax(uint32_t dt, usz nh, usz seq, usz att, void *base, isz sh, isz ss, isz sa, int mask);
int orc_mat_mul(uint32_t dt, usz nd_c, const usz *sh_c, const isz *st_c, void *c, float beta, usz nd_a, const usz *sh_a, const isz *st_a, const void *a,
                usz nd_b, const usz *sh_b, const isz *st_b, const void *b, float alpha);
int orc_random_sample(uint32_t dt, usz n, const void *logits, float t, float top_p, usz top_k, float seed, uint32_t out[2]);
}

static uint64_t splitmix(uint64_t &s) {
  uint64_t z = (s += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
static double uniform01(uint64_t &s) { return (double)(splitmix(s) >> 11) * (1.0 / 9007199254740992.0); }
static std::vector<f16> normal(uint64_t seed, usz n, double std) {
  std::vector<f16> v(n);
  for (usz i = 0; i < n; ++i) {
    double u1 = uniform01(seed), u2 = uniform01(seed);
    if (u1 < 1e-300) u1 = 1e-300;
    v[i] = (f16)(float)(std * std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2));
  }
  return v;
}

static int g_fail = 0;
#define CHECK_CUDA(x)                                                                    \
  do {                                                                                   \
    cudaError_t e_ = (x);                                                                \
    if (e_ != cudaSuccess) {                                                             \
      std::printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); \
      return 2;                                                                          \
    }                                                                                    \
  } while (0)
#define CHECK_OPS(x)                                                                   \
  do {                                                                                 \
    int rc_ = (x);                                                                     \
    if (rc_ != OPS_OK) {                                                               \
      std::printf("%s -> %d: %s (%s:%d)\n", #x, rc_, ops_last_error(), __FILE__, __LINE__); \
      return 3;                                                                        \
    }                                                                                  \
  } while (0)

static void compare(const char *what, const std::vector<f16> &got, const std::vector<f16> &ref, double tol) {
  double worst = 0;
  for (usz i = 0; i < got.size(); ++i) {
    const double d = std::fabs((double)(float)got[i] - (double)(float)ref[i]);
    if (!(d <= worst)) worst = d;  // NaN-propagating maximum
  }
  const bool ok = worst <= tol;
  std::printf("%-28s max-abs %.3e (tolerance %.0e) %s\n", what, worst, tol, ok ? "ok" : "FAIL");
  if (!ok) g_fail = 1;
}

template <class T> static T *upload(const std::vector<T> &h) {
  T *d = nullptr;
  if (cudaMalloc(&d, h.size() * sizeof(T)) != cudaSuccess) return nullptr;
  cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
  return d;
}
template <class T> static std::vector<T> download(const T *d, usz n) {
  std::vector<T> h(n);
  cudaMemcpy(h.data(), d, n * sizeof(T), cudaMemcpyDeviceToHost);
  return h;
}

int main() {
  if (ops_device_count() < 1) {
    std::printf("no CUDA device: the library has no CPU path\n");
    return 77;
  }
  std::printf("library: %s\n", ops_build_info());
  CHECK_CUDA(cudaSetDevice(0));
  cudaStream_t stream;
  CHECK_CUDA(cudaStreamCreate(&stream));

  // ---------------- config 1: rms_norm on x [64, 2048], w U(0.5, 1.5), eps 1e-5 ----------------
  const usz nt = 64, d = 2048, nh = 32, dh = 64;
  std::vector<f16> x = normal(0xB2000010ull, nt * d, 1.0), w(d), y_ref(nt * d);
  uint64_t ws = 0xB2000011ull;
  for (usz i = 0; i < d; ++i) w[i] = (f16)(float)(0.5 + uniform01(ws));
  f16 *xd = upload(x), *wd = upload(w), *yd = nullptr;
  CHECK_CUDA(cudaMalloc(&yd, nt * d * sizeof(f16)));
  {
    const usz sh2[2] = {nt, d}, sh1[1] = {d};
    const isz st2[2] = {(isz)(d * 2), 2}, st1[1] = {2};
    ops_rms_norm_args a{{OPS_DT_F16, 2, sh2, st2}, yd, {OPS_DT_F16, 2, sh2, st2}, xd, {OPS_DT_F16, 1, sh1, st1}, wd, 1e-5f};
    ops_rms_norm *op = nullptr;
    usz need = 1;
    CHECK_OPS(ops_rms_norm_create(0, &op));
    CHECK_OPS(ops_rms_norm_scheme(op, &a, (usz)-1, &need));
    CHECK_OPS(ops_rms_norm_launch(op, &a, nullptr, 0, stream));
    ops_rms_norm_destroy(op);
    orc_rms_norm(OPS_DT_F16, OPS_DT_F16, nt, d, y_ref.data(), d * 2, 2, x.data(), d * 2, 2, w.data(), 2, 1e-5f);
    CHECK_CUDA(cudaStreamSynchronize(stream));
    compare("rms_norm [64,2048]", download(yd, nt * d), y_ref, 1e-2);
  }
  // ---------------- rope on the result viewed as [64, 32, 64], pos 0..63, theta 1e4 ----------------
  {
    std::vector<uint32_t> pos(nt);
    for (usz i = 0; i < nt; ++i) pos[i] = (uint32_t)i;
    uint32_t *pd = upload(pos);
    const usz sh3[3] = {nt, nh, dh}, shp[1] = {nt}, she[2] = {0, dh};
    const isz st3[3] = {(isz)(d * 2), (isz)(dh * 2), 2}, stp[1] = {4}, ste[2] = {(isz)(dh * 2), 2};
    ops_rope_args a{{OPS_DT_F16, 3, sh3, st3}, yd, {OPS_DT_U32, 1, shp, stp}, pd, {OPS_DT_F16, 2, she, ste}, nullptr, {OPS_DT_F16, 2, she, ste}, nullptr, 1e4f};
    ops_rope *op = nullptr;
    CHECK_OPS(ops_rope_create(0, &op));
    CHECK_OPS(ops_rope_launch(op, &a, nullptr, 0, stream));
    ops_rope_destroy(op);
    orc_rope(OPS_DT_F16, OPS_DT_U32, nt, nh, dh, y_ref.data(), d * 2, dh * 2, pos.data(), 4, 1e4f);
    CHECK_CUDA(cudaStreamSynchronize(stream));
    compare("rope [64,32,64]", download(yd, nt * d), y_ref, 1e-2);
    cudaFree(pd);
  }
  // ---------------- causal fused_softmax on scores [32, 64, 64] ~ N(0, 2) ----------------
  {
    std::vector<f16> s = normal(0xB2000012ull, 32 * 64 * 64, 2.0), s_ref = s;
    f16 *sd = upload(s);
    const usz sh3[3] = {32, 64, 64};
    const isz st3[3] = {64 * 64 * 2, 64 * 2, 2};
    ops_fused_softmax_args a{OPS_MASK_CAUSAL, {OPS_DT_F16, 3, sh3, st3}, sd};
    ops_fused_softmax *op = nullptr;
    CHECK_OPS(ops_fused_softmax_create(0, &op));
    CHECK_OPS(ops_fused_softmax_launch(op, &a, nullptr, 0, stream));
    ops_fused_softmax_destroy(op);
    orc_fused_softmax(OPS_DT_F16, 32, 64, 64, s_ref.data(), 64 * 64 * 2, 64 * 2, 2, OPS_MASK_CAUSAL);
    CHECK_CUDA(cudaStreamSynchronize(stream));
    compare("fused_softmax [32,64,64]", download(sd, s.size()), s_ref, 1e-2);
    cudaFree(sd);
  }
  // ---------------- one tensor-core mat_mul: C[256,384] = 0.5 C + A[256,512] B[512,384] ----------------
  {
    const usz m = 256, n = 384, k = 512;
    std::vector<f16> a = normal(21, m * k, 1.0), b = normal(22, k * n, 0.05), c = normal(23, m * n, 1.0), c_ref = c;
    f16 *ad = upload(a), *bd = upload(b), *cd = upload(c);
    const usz shc[2] = {m, n}, sha[2] = {m, k}, shb[2] = {k, n};
    const isz stc[2] = {(isz)(n * 2), 2}, sta[2] = {(isz)(k * 2), 2}, stb[2] = {(isz)(n * 2), 2};
    ops_mat_mul_args args{{OPS_DT_F16, 2, shc, stc}, cd, 0.5f, {OPS_DT_F16, 2, sha, sta}, ad, {OPS_DT_F16, 2, shb, stb}, bd, 1.0f};
    ops_mat_mul *op = nullptr;
    CHECK_OPS(ops_mat_mul_create(0, &op));
    CHECK_OPS(ops_mat_mul_launch(op, &args, nullptr, 0, stream));
    orc_mat_mul(OPS_DT_F16, 2, shc, stc, c_ref.data(), 0.5f, 2, sha, sta, a.data(), 2, shb, stb, b.data(), 1.0f);
    CHECK_CUDA(cudaStreamSynchronize(stream));
    if (ops_mat_mul_status(op) != 0) {
      std::printf("mat_mul: a bounded wait ran out (%d)\n", ops_mat_mul_status(op));
      g_fail = 1;
    }
    ops_mat_mul_destroy(op);
    compare("mat_mul 256x384x512", download(cd, m * n), c_ref, 1e-2);
    // errors are values: a shape mismatch comes back as ShapeMismatch with a message
    const usz bad[2] = {m, n + 8};
    ops_mat_mul_args wrong = args;
    wrong.c_layout.shape = bad;
    ops_mat_mul *op2 = nullptr;
    CHECK_OPS(ops_mat_mul_create(0, &op2));
    const int rc = ops_mat_mul_launch(op2, &wrong, nullptr, 0, stream);
    std::printf("%-28s rc %d (%s) %s\n", "mat_mul shape mismatch", rc, ops_last_error(), rc == OPS_SHAPE_MISMATCH ? "ok" : "FAIL");
    if (rc != OPS_SHAPE_MISMATCH) g_fail = 1;
    ops_mat_mul_destroy(op2);
    cudaFree(ad);
    cudaFree(bd);
    cudaFree(cd);
  }
  // ---------------- argmax over 32000 logits: bit-exact KVPair ----------------
  {
    const usz n = 32000;
    std::vector<f16> lg = normal(31, n, 3.0);
    f16 *ld = upload(lg);
    uint32_t *kvd = nullptr;
    CHECK_CUDA(cudaMalloc(&kvd, 8));
    const usz shl[1] = {n};
    const isz stl[1] = {2}, sti[1] = {4};
    ops_sample_args cfg;
    if (ops_sample_args_new(0.f, 1.f, (usz)-1, &cfg) != 0) return 4;
    ops_random_sample_args a{{OPS_DT_KVPAIR, 0, nullptr, nullptr}, kvd, {OPS_DT_F16, 1, shl, stl}, ld, {OPS_DT_U32, 1, shl, sti}, nullptr, cfg, 0.f};
    ops_random_sample *op = nullptr;
    CHECK_OPS(ops_random_sample_create(0, &op));
    CHECK_OPS(ops_random_sample_launch(op, &a, nullptr, 0, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
    ops_random_sample_destroy(op);
    std::vector<uint32_t> got = download(kvd, 2);
    uint32_t want[2];
    orc_random_sample(OPS_DT_F16, n, lg.data(), 0.f, 1.f, (usz)-1, 0.f, want);
    const bool ok = got[0] == want[0] && got[1] == want[1];
    std::printf("%-28s {%u, 0x%x} vs {%u, 0x%x} %s\n", "random_sample argmax", got[0], got[1], want[0], want[1], ok ? "ok" : "FAIL");
    if (!ok) g_fail = 1;
    cudaFree(ld);
    cudaFree(kvd);
  }
  cudaFree(xd);
  cudaFree(wd);
  cudaFree(yd);
  cudaStreamDestroy(stream);
  std::printf(g_fail ? "FAILED\n" : "all checks passed\n");
  return g_fail;
}
