// Thin extern "C" launchers around the reference engine's OWN attention kernels.
// TEST INFRASTRUCTURE ONLY -- never linked into, loaded by or called from the product.
//
// The reference sources are compiled where they lie (the include path is given on
// the nvcc command line by oracle/Makefile); nothing of them is copied here.  Each
// launcher reproduces the launch shape of the reference call site it names, so the
// resulting library is "the reference's attention, rebuilt for sm_100a":
//   ref_rope          rope()            src/elem.cu:255-259
//   ref_kv_append     k_kv_append<<<>>> src/model.cu:234
//   ref_attn_decode   k_attn_decode<<<>>>   src/model.cu:236-238
//   ref_attn_prefill  k_attn_prefill<<<>>>  src/prefill.cu:152-154
//   ref_gate_sigmoid  k_gate_sigmoid<<<>>>  src/model.cu:239-240
//   ref_unpack3       unpack3()              src/model.cu:221
//   ref_split_qgate   k_split_qgate<<<>>>    src/model.cu:223-224
//   ref_rmsnorm_head  k_rmsnorm_head<<<>>>   src/model.cu:225-226
// All tensors are fp32, as in the reference.
#include "src/elem.cu"
#include "src/mixers.cu"

using namespace spark27;

extern "C" {

int ref_rope(float *v, int heads, int dim, int rot, const int *dpos, float theta,
             void *stream, int B, const int *mpos) {
  rope(v, heads, dim, rot, dpos, theta, (cudaStream_t)stream, B, mpos);
  return (int)cudaGetLastError();
}

int ref_kv_append(const float *k, const float *v, float *kc, float *vc, const int *dpos,
                  int kvdim, int B, void *stream) {
  k_kv_append<<<dim3((kvdim + 255) / 256, B), 256, 0, (cudaStream_t)stream>>>(k, v, kc, vc,
                                                                              dpos, kvdim);
  return (int)cudaGetLastError();
}

int ref_attn_decode(const float *q, const float *kc, const float *vc, float *out,
                    const int *dpos, int dim, int kv_heads, int q_heads, float scale,
                    float *scratch, int ctx, int B, void *stream) {
  k_attn_decode<<<dim3(q_heads, B), 256, 0, (cudaStream_t)stream>>>(
      q, kc, vc, out, dpos, dim, kv_heads, q_heads, scale, scratch, ctx);
  return (int)cudaGetLastError();
}

int ref_attn_prefill(const float *q, const float *kc, const float *vc, float *out,
                     const int *dpos, int dim, int kv_heads, int q_heads, float scale,
                     float *scratch, int ctx, int T, void *stream) {
  k_attn_prefill<<<dim3(q_heads, (T + ATTN_QT - 1) / ATTN_QT), 256, 0, (cudaStream_t)stream>>>(
      q, kc, vc, out, dpos, dim, kv_heads, q_heads, scale, scratch, ctx, T);
  return (int)cudaGetLastError();
}

int ref_gate_sigmoid(float *x, const float *gate, int n, void *stream) {
  k_gate_sigmoid<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(x, gate, n);
  return (int)cudaGetLastError();
}

int ref_unpack3(const float *fused, float *a, float *b, float *c, int na, int nb, int nc, int B, void *stream) {
  unpack3(fused, a, b, c, na, nb, nc, B, (cudaStream_t)stream);
  return (int)cudaGetLastError();
}

int ref_split_qgate(const float *qproj, float *q, float *gate, int rows_times_heads, int dim, void *stream) {
  k_split_qgate<<<(rows_times_heads * dim + 255) / 256, 256, 0, (cudaStream_t)stream>>>(qproj, q, gate,
                                                                                         rows_times_heads, dim);
  return (int)cudaGetLastError();
}

int ref_rmsnorm_head(float *x, const uint16_t *w, int rows_times_heads, int dim, float eps, void *stream) {
  k_rmsnorm_head<<<rows_times_heads, 256, 0, (cudaStream_t)stream>>>(x, w, dim, eps);
  return (int)cudaGetLastError();
}

}  // extern "C"
