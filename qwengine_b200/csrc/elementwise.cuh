// The small kernels around attention: stand-alone RoPE, KV append, sigmoid gate (the
// reference's k_rope / k_kv_append / k_gate_sigmoid launch sites), and the fused
// rope(k) + append used by the batched mixer.
#pragma once

#include "common.cuh"

namespace qwb {

// In-place partial RoPE on v[B][heads][256]; grid (heads, B), block 32 -- one thread per
// rotary pair, the launch shape of the reference's rope() (src/elem.cu:255-259).
template <typename T>
__global__ void __launch_bounds__(32) rope_inplace_kernel(T *v, int heads, const int *dpos, const int *mpos,
                                                          const __grid_constant__ RopeTable tab) {
  const int h = blockIdx.x, b = blockIdx.y, i = threadIdx.x;
  const int pos = mpos ? mpos[b * 3 + mrope_component(i)] : (*dpos + b);
  T *p = v + ((size_t)b * heads + h) * HEAD_DIM;
  double c, s;
  rope_sincos_exact(pos, tab.inv_freq[i], c, s);
  const double x = load_as_f32<T>(p + i), y = load_as_f32<T>(p + i + ROT_PAIRS);
  store_from_f32<T>(p + i, (float)(x * c - y * s));
  store_from_f32<T>(p + i + ROT_PAIRS, (float)(x * s + y * c));
}

// kc[(pos + b) * kvdim + i] = k[b * kvdim + i], same for V (reference src/mixers.cu:416-425),
// cache in bf16.  grid (ceil(kvdim / 2048), B), block 256, 8 elements per thread.
template <typename T>
__global__ void __launch_bounds__(256) kv_append_kernel(const T *k, const T *v, uint16_t *kc, uint16_t *vc,
                                                        const int *dpos, int kvdim) {
  const int i = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (i >= kvdim) return;
  const int b = blockIdx.y;
  const size_t dst = (size_t)(*dpos + b) * kvdim + i, src = (size_t)b * kvdim + i;
  float x[8];
  load8<T>(k + src, x);
  store8<uint16_t>(kc + dst, x);
  load8<T>(v + src, x);
  store8<uint16_t>(vc + dst, x);
}

// x[i] *= sigmoid(gate[i]) (reference src/mixers.cu:653-657); 8 elements per thread, n % 8 == 0.
template <typename T>
__global__ void __launch_bounds__(256) gate_sigmoid_kernel(T *x, const T *gate, int n) {
  const int i = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (i >= n) return;
  float a[8], g[8];
  load8<T>(x + i, a);
  load8<T>(gate + i, g);
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] *= sigmoidf_(g[j]);
  store8<T>(x + i, a);
}

// dst[i] = bf16(src[i]), round to nearest even; 8 elements per thread, n % 8 == 0.  Stages an fp32 q for the
// tcgen05 prefill kernel behind the fp32 drop-in launcher.
__global__ void __launch_bounds__(256) to_bf16_kernel(const float *src, uint16_t *dst, long long n) {
  const long long i = ((long long)blockIdx.x * 256 + threadIdx.x) * 8;
  if (i >= n) return;
  float x[8];
  load8<float>(src + i, x);
  store8<uint16_t>(dst + i, x);
}

// Fused rope(k) + append for a batch: one block per new token row, kv_heads * 32 threads,
// thread = one 8-channel group of one head.  The 32 (cos, sin) pairs of the row's position
// are computed once in double and shared by all heads.
__global__ void __launch_bounds__(128) rope_append_kernel(const uint16_t *k_new, const uint16_t *v_new, uint16_t *kc,
                                                          uint16_t *vc, const int *pos, const int64_t *cache_row,
                                                          const int *mpos, int n_new, int kv_heads, int do_rope,
                                                          const __grid_constant__ RopeTable tab, int *zero_ints,
                                                          int n_zero, PageMap pages, const int *q_pos) {
  // Launched as a programmatic dependent itself: an attention kernel of this library that ran before it on the
  // stream lets it become resident early (its launch latency then overlaps that kernel), and it waits here until
  // whatever ran before has completed and is visible -- before it reads or writes anything.
  grid_dep_wait();
  grid_dep_launch_dependents();  // the attention launch behind this one may start now; it waits where it must
  // block 0 also clears the split-KV arrival counters of the attention launch that follows
  if (blockIdx.x == 0)
    for (int i = threadIdx.x; i < n_zero; i += blockDim.x) zero_ints[i] = 0;
  __shared__ double cs[ROT_PAIRS][2];
  const size_t r = blockIdx.x;  // flat row s * n_new + b
  const int s = (int)(r / n_new), b = (int)(r % n_new);
  const int pz = pos[s] + b;
  if (do_rope && threadIdx.x < ROT_PAIRS) {
    const int i = threadIdx.x;
    const int pp = mpos ? mpos[r * 3 + mrope_component(i)] : (q_pos ? q_pos[s] + b : pz);
    rope_sincos_exact(pp, tab.inv_freq[i], cs[i][0], cs[i][1]);
  }
  __syncthreads();
  const int h = threadIdx.x >> 5, c16 = threadIdx.x & 31;
  if (h >= kv_heads) return;
  const size_t src = (r * kv_heads + h) * HEAD_DIM + c16 * 8;
  const size_t dst = ((size_t)cache_row_of(pages, cache_row, s, pz) * kv_heads + h) * HEAD_DIM + c16 * 8;
  *reinterpret_cast<uint4 *>(vc + dst) = *reinterpret_cast<const uint4 *>(v_new + src);
  if (!do_rope || c16 >= 8) {
    *reinterpret_cast<uint4 *>(kc + dst) = *reinterpret_cast<const uint4 *>(k_new + src);
  } else if (c16 < 4) {
    float x[8], y[8];
    load8<uint16_t>(k_new + src, x);
    load8<uint16_t>(k_new + src + ROT_PAIRS, y);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const double c = cs[c16 * 8 + j][0], sn = cs[c16 * 8 + j][1];
      const double xr = (double)x[j] * c - (double)y[j] * sn, yr = (double)x[j] * sn + (double)y[j] * c;
      x[j] = (float)xr;
      y[j] = (float)yr;
    }
    store8<uint16_t>(kc + dst, x);
    store8<uint16_t>(kc + dst + ROT_PAIRS, y);
  }
}

// Everything between the fused q/k/v projection and attention, in one launch: the reference's
// unpack3 (src/elem.cu:226-237), k_split_qgate (src/mixers.cu:382-390), both k_rmsnorm_head launches
// (src/mixers.cu:393-413, weights used as 1 + w), rope(k) and k_kv_append (src/model.cu:219-235).
// Row layout: [ (q[256] | gate[256]) x q_heads | k[kv_heads][256] | v[kv_heads][256] ].
// Grid (token rows, kv_heads), 8 warps: block (r, g) takes KV head g of row r and the six query heads
// that share it -- warps 0..5 one query head (and its gate) each, warp 6 the key head, warp 7 the value
// head; a lane holds 8 channels.
//   q heads: fp32 mean square, q * rsqrt(ms + eps) * (1 + w) -> bf16 q_out; gate -> bf16 gate_out
//            (q is rotated later, in the attention prologue)
//   k head:  mean square, scale and rotation in double, rounded once into the bf16 cache row
//   v head:  copied into the bf16 cache row
// Block (0, 0) also clears the split-KV arrival counters, like rope_append_kernel.
template <typename TIn>
__global__ void __launch_bounds__(256) fused_rows_kernel(const TIn *fused, const uint16_t *q_norm_w,
                                                         const uint16_t *k_norm_w, float eps, uint16_t *q_out,
                                                         uint16_t *gate_out, uint16_t *kc, uint16_t *vc, const int *pos,
                                                         const int64_t *cache_row, const int *mpos, int n_new,
                                                         int q_heads, int kv_heads, int do_rope,
                                                         const __grid_constant__ RopeTable tab, int *zero_ints,
                                                         int n_zero, PageMap pages, const int *q_pos) {
  // Launched as a programmatic dependent itself: an attention kernel of this library that ran before it on the
  // stream lets it become resident early (its launch latency then overlaps that kernel), and it waits here until
  // whatever ran before has completed and is visible -- before it reads or writes anything.
  grid_dep_wait();
  grid_dep_launch_dependents();  // the attention launch behind this one may start now; it waits where it must
  if (blockIdx.x == 0 && blockIdx.y == 0)
    for (int i = threadIdx.x; i < n_zero; i += blockDim.x) zero_ints[i] = 0;
  const size_t r = blockIdx.x;  // flat row s * n_new + b
  const int g = blockIdx.y;     // KV head
  const int s = (int)(r / n_new), b = (int)(r % n_new);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t width = (size_t)q_heads * 2 * HEAD_DIM + 2 * (size_t)kv_heads * HEAD_DIM;
  const TIn *row = fused + r * width;
  float w8[8];
  if (warp < GROUP) {
    // ---- one query head and its gate ----
    const int h = g * GROUP + warp;
    float x[8], gt[8];
    load8<TIn>(row + (size_t)h * 2 * HEAD_DIM + lane * 8, x);
    load8<TIn>(row + (size_t)h * 2 * HEAD_DIM + HEAD_DIM + lane * 8, gt);
    load8<uint16_t>(q_norm_w + lane * 8, w8);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float sc = rsqrtf(ss * (1.0f / HEAD_DIM) + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = x[j] * sc * (1.0f + w8[j]);
    store8<uint16_t>(q_out + (r * q_heads + h) * HEAD_DIM + lane * 8, x);
    store8<uint16_t>(gate_out + (r * q_heads + h) * HEAD_DIM + lane * 8, gt);
    return;
  }
  const int pz = pos[s] + b;
  const size_t crow = ((size_t)cache_row_of(pages, cache_row, s, pz) * kv_heads + g) * HEAD_DIM;
  if (warp == GROUP + 1) {
    // ---- value head ----
    float x[8];
    load8<TIn>(row + (size_t)q_heads * 2 * HEAD_DIM + (size_t)(kv_heads + g) * HEAD_DIM + lane * 8, x);
    store8<uint16_t>(vc + crow + lane * 8, x);
    return;
  }
  // ---- key head: normalise, rotate, append ----
  float x[8];
  load8<TIn>(row + (size_t)q_heads * 2 * HEAD_DIM + (size_t)g * HEAD_DIM + lane * 8, x);
  load8<uint16_t>(k_norm_w + lane * 8, w8);
  double cs = 1.0, sn = 0.0;  // lane i: cos / sin of rotary pair i
  if (do_rope) {
    const int pp = mpos ? mpos[r * 3 + mrope_component(lane)] : (q_pos ? q_pos[s] + b : pz);
    rope_sincos_exact(pp, tab.inv_freq[lane], cs, sn);
  }
  double ss = 0.0;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss += (double)x[j] * (double)x[j];
#pragma unroll
  for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const double sc = 1.0 / sqrt(ss / HEAD_DIM + (double)eps);
#pragma unroll
  for (int j = 0; j < 8; ++j) x[j] = (float)((double)x[j] * sc * (1.0 + (double)w8[j]));
  if (do_rope) {
    // rotary pair (i, i + 32): lanes 0..3 hold i = 0..31 (8 each), lanes 4..7 hold i + 32
    const bool lo = lane < 4;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float y = __shfl_xor_sync(0xffffffffu, x[j], 4);
      const int i = (lane & 3) * 8 + j;
      const double c = __shfl_sync(0xffffffffu, cs, i), sv = __shfl_sync(0xffffffffu, sn, i);
      const double a = lo ? (double)x[j] : (double)y, bq = lo ? (double)y : (double)x[j];  // (x_i, x_{i+32})
      if (lane < 8) x[j] = lo ? (float)(a * c - bq * sv) : (float)(a * sv + bq * c);
    }
  }
  store8<uint16_t>(kc + crow + lane * 8, x);
}

}  // namespace qwb
