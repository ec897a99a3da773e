// Shared device helpers for the sm_100a attention kernels: bf16 packing, RoPE angles,
// mbarrier / TMA wrappers whose waits are bounded, and the parameter blocks passed from
// the C ABI layer to the kernels.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace qwb {

constexpr int HEAD_DIM = 256;   // qwen38.h:47 of the reference
constexpr int ROTARY_DIM = 64;  // qwen38.h:62
constexpr int ROT_PAIRS = ROTARY_DIM / 2;
constexpr int GROUP = 6;        // query heads per KV head (24 / 4, qwen38.h:45-46)
constexpr int PART_STRIDE = 260; // floats per split-KV partial row: o[256], m, l, 2 pad (16-byte rows)

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

// Codes written to the device status word.
constexpr int DEV_ERR_FULL_WAIT = 101;   // consumer waited too long for a TMA tile
constexpr int DEV_ERR_EMPTY_WAIT = 102;  // producer waited too long for a free stage
constexpr int DEV_ERR_MMA_WAIT = 103;    // a wait on tcgen05 completion ran out
constexpr int DEV_ERR_SOFTMAX_WAIT = 104;
constexpr int DEV_ERR_TMEM = 105;
constexpr int DEV_ERR_PEER_WAIT = 106;   // another GPU's partials did not show up in time
constexpr int DEV_ERR_RING = 107;        // two roles of a kernel disagree about a ring slot (an internal consistency check)

struct RopeTable {
  double inv_freq[ROT_PAIRS];  // theta^(-2i/rot), computed on the host in double
};

// ---- bf16 helpers ------------------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
  __nv_bfloat16 b = __float2bfloat16_rn(f);
  return *reinterpret_cast<uint16_t *>(&b);
}

template <typename T> __device__ __forceinline__ float load_as_f32(const T *p);
template <> __device__ __forceinline__ float load_as_f32<float>(const float *p) { return *p; }
template <> __device__ __forceinline__ float load_as_f32<uint16_t>(const uint16_t *p) { return bf16_bits_to_f32(*p); }
template <typename T> __device__ __forceinline__ void store_from_f32(T *p, float v);
template <> __device__ __forceinline__ void store_from_f32<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_from_f32<uint16_t>(uint16_t *p, float v) { *p = f32_to_bf16_bits(v); }

// Which mrope position component (t, h, w) rotary slot i uses: sections [11, 11, 10]
// interleaved T,H,W,...  (reference src/elem.cu:112-117).
__device__ __forceinline__ int mrope_component(int slot) {
  const int m = slot % 3;
  if (m == 1 && slot <= 31) return 1;
  if (m == 2 && slot <= 29) return 2;
  return 0;
}

// cos/sin of pos * inv_freq with the angle formed and reduced in double, so that large
// positions keep full accuracy (an fp32 angle at pos 8192 is already off by 5e-4 rad).
__device__ __forceinline__ void rope_sincos_exact(int pos, double inv_freq, double &c, double &s) {
  sincos((double)pos * inv_freq, &s, &c);
}
// Cheaper form for the prefill prologue: double product and range reduction, fp32 sincos.
__device__ __forceinline__ void rope_sincos_fast(int pos, double inv_freq, float &c, float &s) {
  const double a = (double)pos * inv_freq;
  const double k = rint(a * 0.15915494309189535);  // a / 2pi
  const double r = fma(-k, 6.283185307179586, a);  // exact enough: |k| < 2^18
  sincosf((float)r, &s, &c);
}

// Cheapest form, for the tcgen05 prologue: the angle is formed and reduced to [-pi, pi] in double,
// where the hardware sin/cos approximations are good to ~4e-7 absolute -- far below the 2^-17 that
// the bf16 hi + lo pair of the rotated value keeps.
__device__ __forceinline__ void rope_sincos_reduced(int pos, double inv_freq, float &c, float &s) {
  const double a = (double)pos * inv_freq;
  const double k = rint(a * 0.15915494309189535);
  const float r = (float)fma(-k, 6.283185307179586, a);
  __sincosf(r, &s, &c);
}

// Where a sequence's cached tokens live.  Contiguous (table == nullptr): token t of sequence s is row
// cache_row[s] + t of the pool.  Paged: the pool is cut into pages of page_rows rows (a multiple of 128,
// so no K/V tile straddles a page) and token t is row table[s * stride + t / page_rows] * page_rows +
// t % page_rows -- a block table as serving engines keep it, one line per sequence.
struct PageMap {
  const int *table;
  int stride;
  int page_rows;
};
__device__ __forceinline__ long long cache_row_of(const PageMap &pm, const int64_t *cache_row, int s, int t) {
  if (!pm.table) return (cache_row ? cache_row[s] : 0) + t;
  const int pg = t / pm.page_rows;
  return (long long)pm.table[(size_t)s * pm.stride + pg] * pm.page_rows + (t - pg * pm.page_rows);
}
// The same for a producer loop: `base` is the sequence's first row, read once (cache_row[s], or 0); only the
// paged layout costs a memory access per call.  Loads issued while an SM streams K/V through TMA are slow,
// so a producer must not repeat them per copy.
__device__ __forceinline__ long long cache_row_at(const PageMap &pm, long long base, int s, int t) {
  if (!pm.table) return base + t;
  const int pg = t / pm.page_rows;
  return (long long)pm.table[(size_t)s * pm.stride + pg] * pm.page_rows + (t - pg * pm.page_rows);
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }
// Same value to ~2 ulp with the approximate reciprocal: for epilogues that are instruction-bound.
__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
// One special-function operation instead of two: sigmoid(x) = 0.5 + 0.5 tanh(x / 2) with the hardware tanh
// (relative error up to 2^-11, i.e. at most 2.5e-4 absolute on the sigmoid).  For the prefill epilogue, which is
// bound by the special-function unit: a gated output row's relative L2 error goes from ~2e-6 to ~1e-4, an order
// of magnitude inside the 1e-3 bound.
__device__ __forceinline__ float sigmoid_tanh(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(0.5f, t, 0.5f);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Store 8 consecutive values as T (bf16: one 16-byte store).
template <typename T> __device__ __forceinline__ void store8(T *p, const float (&v)[8]);
template <> __device__ __forceinline__ void store8<float>(float *p, const float (&v)[8]) {
  *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4 *>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

template <> __device__ __forceinline__ void store8<uint16_t>(uint16_t *p, const float (&v)[8]) {
  *reinterpret_cast<uint4 *>(p) =
      make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}
template <typename T> __device__ __forceinline__ void load8(const T *p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<float>(const float *p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8<uint16_t>(const uint16_t *p, float (&v)[8]) {
  const uint4 a = *reinterpret_cast<const uint4 *>(p);
  v[0] = bf16lo(a.x); v[1] = bf16hi(a.x); v[2] = bf16lo(a.y); v[3] = bf16hi(a.y);
  v[4] = bf16lo(a.z); v[5] = bf16hi(a.z); v[6] = bf16lo(a.w); v[7] = bf16hi(a.w);
}

// ---- shared-memory address / mbarrier / TMA ------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait: a short spin, then polling against the wall clock.  After WAIT_LIMIT_NS the
// wait gives up and returns false; the caller records an error code and unwinds without
// waiting again, so a lost signal costs a fraction of a second, not the GPU.
constexpr uint64_t WAIT_LIMIT_NS = 200000000ull;
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
  for (int i = 0; i < 64; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 0; i < (1u << 30); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 15) == 15 && global_timer_ns() - t0 > WAIT_LIMIT_NS) return false;
  }
  return false;
}
// Programmatic dependent launch.  The append kernel of a step is launched as a programmatic dependent: it waits
// (grid_dep_wait) for whatever ran before it on the stream, then calls grid_dep_launch_dependents(), which lets the
// attention kernel launched behind it (with the stream-serialisation attribute) start while the append still runs;
// the attention kernel calls grid_dep_wait() only where it first needs the append's results: before it loads a
// tile that holds new rows, and before it takes an arrival ticket (the append kernel clears the counters).  The
// attention kernels call grid_dep_launch_dependents() first thing as well, so that the NEXT launch on the stream, if
// it is a programmatic dependent (this library's append kernel of the next call is), is resident and waiting when
// they end instead of being launched then.  Without the launch attribute both instructions are no-ops.
__device__ __forceinline__ void grid_dep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 3-D tiled TMA load, no multicast.  Coordinate 0 is the innermost (element) index and must be
// a multiple of 8 for bf16 (16-byte rule); this code only ever passes 0 there.
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
      "r"(c2)
      : "memory");
}
// 2-D tiled TMA load, no multicast.  c0 is the element index along the row and must be a
// multiple of 8 for bf16 (16-byte rule); callers pass kv_head*256 + chunk*64.
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// Byte offset of element (row, d) in a K/V stage written by the 3-D TMA box
// (64 elements, ROWS rows, 4 chunks) with the 128-byte swizzle: four [ROWS][128 B] sub-tiles,
// the 16-byte column index XORed with (row % 8).
template <int ROWS>
__device__ __forceinline__ uint32_t kv_tile_off(int row, int d) {
  const int chunk = d >> 6, c16 = (d >> 3) & 7;
  return (uint32_t)(chunk * (ROWS * 128) + row * 128 + ((c16 ^ (row & 7)) << 4) + ((d & 7) << 1));
}

// ---- warp-level mma.sync helpers (used by the split-KV kernel) -----------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2,
                                              uint32_t &r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Host side: kernel launch, optionally as a programmatic dependent of the launch before it on the stream.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool dependent,
                                 Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = dependent ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace qwb
