// C++ host-side mirror of the reference engine's launchers for the full-attention path, on top of
// the C ABI (include/qwengine_attn.h).  Same names, argument order and defaults as the reference:
//   rope()            src/elem.cu:255-259
//   kv_append()       launch site src/model.cu:234      (kernel src/mixers.cu:416-425)
//   attn_decode()     launch site src/model.cu:236-238  (kernel src/mixers.cu:436-525)
//   attn_prefill()    launch site src/prefill.cu:152-154 (kernel src/mixers.cu:546-649)
//   gate_sigmoid()    launch site src/model.cu:239-240  (kernel src/mixers.cu:653-657)
// Overloads take fp32 activations (as the reference holds them) or bf16 bit patterns; the KV
// cache is always bf16.  Unlike the reference's void launchers these return the library's status
// code (0 = ok); they never exit the process.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qwengine_attn.h"

namespace qwengine_b200 {

inline int rope(float *v, int heads, int dim, int rot, const int *dpos, float theta, cudaStream_t st = 0, int B = 1,
                const int *mpos = nullptr) {
  return qw_rope_f32(v, heads, dim, rot, dpos, theta, st, B, mpos);
}
inline int rope(uint16_t *v, int heads, int dim, int rot, const int *dpos, float theta, cudaStream_t st = 0, int B = 1,
                const int *mpos = nullptr) {
  return qw_rope_bf16(v, heads, dim, rot, dpos, theta, st, B, mpos);
}

inline int kv_append(const float *k, const float *v, uint16_t *kc, uint16_t *vc, const int *dpos, int kvdim,
                     cudaStream_t st = 0, int B = 1) {
  return qw_kv_append_f32(k, v, kc, vc, dpos, kvdim, B, st);
}
inline int kv_append(const uint16_t *k, const uint16_t *v, uint16_t *kc, uint16_t *vc, const int *dpos, int kvdim,
                     cudaStream_t st = 0, int B = 1) {
  return qw_kv_append_bf16(k, v, kc, vc, dpos, kvdim, B, st);
}

inline int attn_decode(const float *q, const uint16_t *kc, const uint16_t *vc, float *out, const int *dpos, int dim,
                       int kv_heads, int q_heads, float scale, float *scratch, int ctx, cudaStream_t st = 0, int B = 1) {
  return qw_attn_decode_f32(q, kc, vc, out, dpos, dim, kv_heads, q_heads, scale, scratch, ctx, B, st);
}
inline int attn_decode(const uint16_t *q, const uint16_t *kc, const uint16_t *vc, uint16_t *out, const int *dpos,
                       int dim, int kv_heads, int q_heads, float scale, float *scratch, int ctx, cudaStream_t st = 0,
                       int B = 1) {
  return qw_attn_decode_bf16(q, kc, vc, out, dpos, dim, kv_heads, q_heads, scale, scratch, ctx, B, st);
}

inline int attn_prefill(const float *q, const uint16_t *kc, const uint16_t *vc, float *out, const int *dpos, int dim,
                        int kv_heads, int q_heads, float scale, float *scratch, int ctx, int T, cudaStream_t st = 0) {
  return qw_attn_prefill_f32(q, kc, vc, out, dpos, dim, kv_heads, q_heads, scale, scratch, ctx, T, st);
}
inline int attn_prefill(const uint16_t *q, const uint16_t *kc, const uint16_t *vc, uint16_t *out, const int *dpos,
                        int dim, int kv_heads, int q_heads, float scale, float *scratch, int ctx, int T,
                        cudaStream_t st = 0) {
  return qw_attn_prefill_bf16(q, kc, vc, out, dpos, dim, kv_heads, q_heads, scale, scratch, ctx, T, st);
}

inline int gate_sigmoid(float *x, const float *gate, int n, cudaStream_t st = 0) {
  return qw_gate_sigmoid_f32(x, gate, n, st);
}
inline int gate_sigmoid(uint16_t *x, const uint16_t *gate, int n, cudaStream_t st = 0) {
  return qw_gate_sigmoid_bf16(x, gate, n, st);
}

// The whole mixer of one layer for a batch of sequences (bf16 activations): fills a descriptor
// for qw_mixer_forward.  `workspace` must hold qw_mixer_workspace_bytes() bytes.
struct Mixer {
  qw_mixer_desc d{};
  Mixer(int n_seq, int n_new, int kv_heads = 4, float theta = 1e7f, float scale = 1.0f / 16.0f) {
    d.n_seq = n_seq; d.n_new = n_new; d.kv_heads = kv_heads; d.q_heads = 6 * kv_heads;
    d.head_dim = 256; d.rotary_dim = 64; d.theta = theta; d.scale = scale;
    d.flags = QW_F_ROPE | QW_F_APPEND | QW_F_GATE;
  }
  size_t workspace_bytes() const { return qw_mixer_workspace_bytes(&d); }
  int forward(cudaStream_t st = 0) const { return qw_mixer_forward(&d, st); }
  // Fed by the fused projection rows (fp32 as the reference's GEMM emits them): what src/model.cu:221-226
  // does with unpack3, k_split_qgate and k_rmsnorm_head happens inside the call.
  int forward_fused(const float *fused, const qw_bf16 *q_norm_w, const qw_bf16 *k_norm_w, float eps = 1e-6f,
                    cudaStream_t st = 0) const {
    return qw_mixer_forward_fused(&d, fused, 1, q_norm_w, k_norm_w, eps, st);
  }
};

}  // namespace qwengine_b200
