// The reference engine's three attention call sites, rebuilt against this library's C++ mirror of the
// reference launchers (qwengine_b200/csrc/mixer.hpp) and run on synthetic activations.
// TEST INFRASTRUCTURE ONLY -- never linked into, loaded by or called from the product.
//
// What a maintainer would do to src/model.cu:228-240 (decode / verify, inside the captured graph of
// src/model.cu:318-327), src/mtp.cu:172-179 (draft head, B = 1) and src/prefill.cu:142-156 (prefill chunk) is
// done here on a stand-in for the engine's Runtime: fp32 activations sized by the reference's own constants
// (qwen38.h is included from the reference tree where it lies; nothing of it is copied), a device-resident
// position, a bf16 KV cache, the reference-sized `scores` scratch.  Each site is run twice -- through this
// library, and through the reference's own kernels rebuilt for sm_100a (libref_attn.so, fp32 cache) -- and the
// two attention outputs are compared.  The end-to-end, token-exact check of test/test_spec.cu needs the model
// weights and is not run.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include <cuda_runtime.h>

#include "qwen38.h"                              // the reference's constants (include path: the reference tree)
#include "../qwengine_b200/csrc/mixer.hpp"       // rope / kv_append / attn_decode / attn_prefill / gate_sigmoid

using namespace q38;
namespace qw = qwengine_b200;

extern "C" {  // libref_attn.so: the reference's kernels behind their own launch shapes (oracle/ref_shim.cu)
int ref_rope(float *v, int heads, int dim, int rot, const int *dpos, float theta, void *stream, int B, const int *mpos);
int ref_kv_append(const float *k, const float *v, float *kc, float *vc, const int *dpos, int kvdim, int B, void *stream);
int ref_attn_decode(const float *q, const float *kc, const float *vc, float *out, const int *dpos, int dim, int kv_heads,
                    int q_heads, float scale, float *scratch, int ctx, int B, void *stream);
int ref_attn_prefill(const float *q, const float *kc, const float *vc, float *out, const int *dpos, int dim, int kv_heads,
                     int q_heads, float scale, float *scratch, int ctx, int T, void *stream);
int ref_gate_sigmoid(float *x, const float *gate, int n, void *stream);
}

#define CK(x)                                                                                   \
  do {                                                                                          \
    cudaError_t e_ = (x);                                                                       \
    if (e_ != cudaSuccess) {                                                                    \
      fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__);  \
      exit(2);                                                                                  \
    }                                                                                           \
  } while (0)
#define QW(x)                                                                                   \
  do {                                                                                          \
    int r_ = (x);                                                                               \
    if (r_ != 0) {                                                                              \
      fprintf(stderr, "%s -> %d (%s) [%s]\n", #x, r_, qw_strerror(r_), qw_last_cuda_error());   \
      exit(3);                                                                                  \
    }                                                                                           \
  } while (0)

static uint64_t g_state = 0x9E3779B97F4A7C15ull;
static float next_normal() {  // sum of uniforms: close enough to N(0,1) for a comparison of two implementations
  float s = 0.f;
  for (int i = 0; i < 12; ++i) {
    g_state = g_state * 6364136223846793005ull + 1442695040888963407ull;
    s += (float)((g_state >> 40) & 0xFFFFFF) / 16777216.0f;
  }
  return s - 6.0f;
}
static uint16_t to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  u += 0x7FFF + ((u >> 16) & 1);
  return (uint16_t)(u >> 16);
}
static float from_bf16(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
template <typename T> static T *dev(const std::vector<T> &h) {
  T *d = nullptr;
  CK(cudaMalloc(&d, h.size() * sizeof(T)));
  CK(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
  return d;
}
template <typename T> static T *dev_empty(size_t n) {
  T *d = nullptr;
  CK(cudaMalloc(&d, n * sizeof(T)));
  CK(cudaMemset(d, 0, n * sizeof(T)));
  return d;
}
static bool compare(const char *what, const float *ours_d, const float *ref_d, size_t n, double tol_rel) {
  std::vector<float> a(n), b(n);
  CK(cudaMemcpy(a.data(), ours_d, n * 4, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(b.data(), ref_d, n * 4, cudaMemcpyDeviceToHost));
  double num = 0, den = 0, mx = 0;
  for (size_t i = 0; i < n; ++i) {
    const double d = (double)a[i] - (double)b[i];
    num += d * d;
    den += (double)b[i] * (double)b[i];
    if (std::fabs(d) > mx) mx = std::fabs(d);
    if (!std::isfinite(a[i])) mx = 1e30;
  }
  const double rel = std::sqrt(num / (den > 0 ? den : 1));
  const bool ok = mx <= 2e-2 && rel <= tol_rel;
  printf("%-44s max-abs %.3e rel-L2 %.3e  %s\n", what, mx, rel, ok ? "ok" : "FAIL");
  return ok;
}

// The stand-in for the engine's Runtime (src/model.cu:59-75): one full-attention layer's buffers.
struct Site {
  int ctx, rows;
  float *qh, *kh, *vh, *gateh, *attn_out, *scores;   // fp32 activations, as the reference holds them
  int *dpos;
  uint16_t *kc, *vc;                                 // this library's cache: bf16, same [pos][kv_head][dim] indexing
  float *ref_q, *ref_k, *ref_out, *ref_kc, *ref_vc;  // the reference's own copies (fp32 cache)
};

static Site make_site(int ctx, int rows, int pos0) {
  Site s{};
  s.ctx = ctx;
  s.rows = rows;
  std::vector<float> kc((size_t)ctx * KV_DIM, 0.f), vc((size_t)ctx * KV_DIM, 0.f);
  std::vector<uint16_t> kcb((size_t)ctx * KV_DIM, 0), vcb((size_t)ctx * KV_DIM, 0);
  for (size_t i = 0; i < (size_t)pos0 * KV_DIM; ++i) {  // the history: bf16-exact values, identical for both sides
    kcb[i] = to_bf16(next_normal()); kc[i] = from_bf16(kcb[i]);
    vcb[i] = to_bf16(next_normal()); vc[i] = from_bf16(vcb[i]);
  }
  s.kc = dev(kcb); s.vc = dev(vcb); s.ref_kc = dev(kc); s.ref_vc = dev(vc);
  s.qh = dev_empty<float>((size_t)rows * Q_DIM); s.kh = dev_empty<float>((size_t)rows * KV_DIM);
  s.vh = dev_empty<float>((size_t)rows * KV_DIM); s.gateh = dev_empty<float>((size_t)rows * Q_DIM);
  s.attn_out = dev_empty<float>((size_t)rows * Q_DIM);
  s.ref_q = dev_empty<float>((size_t)rows * Q_DIM); s.ref_k = dev_empty<float>((size_t)rows * KV_DIM);
  s.ref_out = dev_empty<float>((size_t)rows * Q_DIM);
  s.scores = dev_empty<float>((size_t)rows * N_Q_HEADS * ctx);  // src/model.cu:168, src/prefill.cu:75
  s.dpos = dev_empty<int>(1);
  return s;
}
static void new_rows(Site &s, int B) {  // what the projections + QK-norm would have produced for B new tokens
  std::vector<float> q((size_t)B * Q_DIM), k((size_t)B * KV_DIM), v((size_t)B * KV_DIM), g((size_t)B * Q_DIM);
  for (auto &x : q) x = next_normal();
  for (auto &x : k) x = next_normal();
  for (auto &x : v) x = from_bf16(to_bf16(next_normal()));
  for (auto &x : g) x = next_normal();
  CK(cudaMemcpy(s.qh, q.data(), q.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(s.kh, k.data(), k.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(s.vh, v.data(), v.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(s.gateh, g.data(), g.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(s.ref_q, q.data(), q.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(s.ref_k, k.data(), k.size() * 4, cudaMemcpyHostToDevice));
}
static void set_pos(Site &s, int pos) { CK(cudaMemcpy(s.dpos, &pos, 4, cudaMemcpyHostToDevice)); }

// src/model.cu:228-240 with each launch replaced by its mixer.hpp counterpart
static void record_step_ours(Site &s, int B, cudaStream_t st) {
  const float scale = 1.0f / sqrtf((float)HEAD_DIM);
  QW(qw::rope(s.qh, N_Q_HEADS, HEAD_DIM, ROTARY_DIM, s.dpos, ROPE_THETA, st, B));
  QW(qw::rope(s.kh, N_KV_HEADS, HEAD_DIM, ROTARY_DIM, s.dpos, ROPE_THETA, st, B));
  QW(qw::kv_append(s.kh, s.vh, s.kc, s.vc, s.dpos, KV_DIM, st, B));
  QW(qw::attn_decode(s.qh, s.kc, s.vc, s.attn_out, s.dpos, HEAD_DIM, N_KV_HEADS, N_Q_HEADS, scale, s.scores, s.ctx, st, B));
  QW(qw::gate_sigmoid(s.attn_out, s.gateh, B * Q_DIM, st));
}
static void record_step_ref(Site &s, int B, cudaStream_t st) {
  const float scale = 1.0f / sqrtf((float)HEAD_DIM);
  ref_rope(s.ref_q, N_Q_HEADS, HEAD_DIM, ROTARY_DIM, s.dpos, ROPE_THETA, st, B, nullptr);
  ref_rope(s.ref_k, N_KV_HEADS, HEAD_DIM, ROTARY_DIM, s.dpos, ROPE_THETA, st, B, nullptr);
  ref_kv_append(s.ref_k, s.vh, s.ref_kc, s.ref_vc, s.dpos, KV_DIM, B, st);
  ref_attn_decode(s.ref_q, s.ref_kc, s.ref_vc, s.ref_out, s.dpos, HEAD_DIM, N_KV_HEADS, N_Q_HEADS, scale, s.scores, s.ctx, B, st);
  ref_gate_sigmoid(s.ref_out, s.gateh, B * Q_DIM, st);
}
// src/prefill.cu:142-156
static void prefill_chunk_ours(Site &s, int T, cudaStream_t st) {
  const float scale = 1.0f / sqrtf((float)HEAD_DIM);
  QW(qw::rope(s.qh, N_Q_HEADS, HEAD_DIM, ROTARY_DIM, s.dpos, ROPE_THETA, st, T));
  QW(qw::rope(s.kh, N_KV_HEADS, HEAD_DIM, ROTARY_DIM, s.dpos, ROPE_THETA, st, T));
  QW(qw::kv_append(s.kh, s.vh, s.kc, s.vc, s.dpos, KV_DIM, st, T));
  QW(qw::attn_prefill(s.qh, s.kc, s.vc, s.attn_out, s.dpos, HEAD_DIM, N_KV_HEADS, N_Q_HEADS, scale, s.scores, s.ctx, T, st));
  QW(qw::gate_sigmoid(s.attn_out, s.gateh, T * Q_DIM, st));
}
static void prefill_chunk_ref(Site &s, int T, cudaStream_t st) {
  const float scale = 1.0f / sqrtf((float)HEAD_DIM);
  ref_rope(s.ref_q, N_Q_HEADS, HEAD_DIM, ROTARY_DIM, s.dpos, ROPE_THETA, st, T, nullptr);
  ref_rope(s.ref_k, N_KV_HEADS, HEAD_DIM, ROTARY_DIM, s.dpos, ROPE_THETA, st, T, nullptr);
  ref_kv_append(s.ref_k, s.vh, s.ref_kc, s.ref_vc, s.dpos, KV_DIM, T, st);
  ref_attn_prefill(s.ref_q, s.ref_kc, s.ref_vc, s.ref_out, s.dpos, HEAD_DIM, N_KV_HEADS, N_Q_HEADS, scale, s.scores, s.ctx, T, st);
  ref_gate_sigmoid(s.ref_out, s.gateh, T * Q_DIM, st);
}

int main() {
  int n_dev = 0;
  if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0) {
    fprintf(stderr, "no CUDA device\n");
    return 4;
  }
  CK(cudaSetDevice(0));
  cudaStream_t st;
  CK(cudaStreamCreate(&st));
  bool ok = true;
  printf("geometry from the reference's qwen38.h: %d q heads, %d kv heads, head_dim %d, rotary %d, theta %.0f, ABI %d\n",
         N_Q_HEADS, N_KV_HEADS, HEAD_DIM, ROTARY_DIM, (double)ROPE_THETA, qw_abi_version());

  // ---- decode and verify inside a captured graph, replayed as the position advances (src/model.cu:318-327) ----
  const int steps_B[3] = {1, 4, 8};
  for (int bi = 0; bi < 3; ++bi) {
    const int B = steps_B[bi], ctx = 4096, pos0 = 1500;
    Site s = make_site(ctx, 8, pos0);   // buffers sized for MAX_B = 8 rows, as rt_init does
    set_pos(s, pos0);
    new_rows(s, B);
    record_step_ours(s, B, st);         // warm-up outside the capture: one-time kernel attributes are set here
    CK(cudaStreamSynchronize(st));
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    int pos = pos0;
    for (int cycle = 0; cycle < 3; ++cycle) {   // three steps: the graph is captured once and replayed
      set_pos(s, pos);
      new_rows(s, B);
      if (cycle == 0) {
        CK(cudaStreamBeginCapture(st, cudaStreamCaptureModeRelaxed));
        record_step_ours(s, B, st);
        CK(cudaStreamEndCapture(st, &graph));
        CK(cudaGraphInstantiate(&exec, graph, 0));
      }
      CK(cudaGraphLaunch(exec, st));
      record_step_ref(s, B, st);
      CK(cudaStreamSynchronize(st));
      char what[96];
      snprintf(what, sizeof(what), "decode graph B=%d pos=%d (src/model.cu:228-240)", B, pos);
      ok = compare(what, s.attn_out, s.ref_out, (size_t)B * Q_DIM, 2e-3) && ok;
      pos += B;                         // k_advance_by (src/elem.cu:202): the next step sees the rows just appended
    }
    CK(cudaGraphExecDestroy(exec));
    CK(cudaGraphDestroy(graph));
  }
  // ---- a short run: the engine sizes its cache as prompt + new tokens + 8 rows (src/main.cu:38), so the score
  //      buffer of B * q_heads * ctx floats is far smaller than one set of split-KV partials ----
  for (int bi = 0; bi < 2; ++bi) {
    const int B = bi == 0 ? 1 : 4, prompt = 5, ctx = prompt + 32 + 8;
    Site s = make_site(ctx, 8, prompt);
    int pos = prompt;
    for (int step = 0; step < 3; ++step) {
      set_pos(s, pos);
      new_rows(s, B);
      record_step_ours(s, B, st);
      record_step_ref(s, B, st);
      CK(cudaStreamSynchronize(st));
      char what[96];
      snprintf(what, sizeof(what), "short run ctx=%d B=%d pos=%d (src/main.cu:38)", ctx, B, pos);
      ok = compare(what, s.attn_out, s.ref_out, (size_t)B * Q_DIM, 2e-3) && ok;
      pos += B;
    }
  }
  // ---- prefill: two chunks of one prompt, the second behind the first (src/prefill.cu:231-240) ----
  {
    const int T = 512, ctx = 2048;
    Site s = make_site(ctx, T, 0);
    for (int chunk = 0; chunk < 2; ++chunk) {
      set_pos(s, chunk * T);
      new_rows(s, T);
      prefill_chunk_ours(s, T, st);
      prefill_chunk_ref(s, T, st);
      CK(cudaStreamSynchronize(st));
      char what[96];
      snprintf(what, sizeof(what), "prefill chunk T=%d pos=%d (src/prefill.cu:142-156)", T, chunk * T);
      // q enters the tensor cores as bf16 on this route and the cache is bf16: rel-L2 of a few 1e-3 against the
      // reference's all-fp32 arithmetic
      ok = compare(what, s.attn_out, s.ref_out, (size_t)T * Q_DIM, 4e-3) && ok;
    }
  }
  printf(ok ? "CALLSITE_CHECK ok\n" : "CALLSITE_CHECK FAILED\n");
  return ok ? 0 : 1;
}
