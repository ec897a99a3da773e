// extern "C" layer of the B200 full-attention mixer: argument checks, tensor-map
// construction and kernel launches.  Nothing here allocates, frees or synchronises.
#include "../../include/qwengine_attn.h"

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "elementwise.cuh"
#include "prefill_umma.cuh"
#include "splitkv.cuh"
#include "splitkv_umma.cuh"

using namespace qwb;


namespace {

thread_local char g_cuda_err[256] = "";
thread_local int g_launches = 0;
thread_local const char *g_attn_kernel = "";  // attention kernel of the last call on this thread

int cuda_fail(cudaError_t e, const char *what) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", what, cudaGetErrorString(e));
  return QW_ERR_CUDA;
}
#define QW_CUDA(x)                                  \
  do {                                              \
    cudaError_t e_ = (x);                           \
    if (e_ != cudaSuccess) return cuda_fail(e_, #x); \
  } while (0)

int check_launch(const char *what) {
  ++g_launches;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? QW_OK : cuda_fail(e, what);
}

constexpr int MAX_DEVICES = 64;
// Current device, or -1 when it cannot be told or lies outside the per-device tables below.
int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -1;
  return dev;
}

// Optional event pair around the dominant kernel of a call (see qw_profile_enable).  Events belong
// to a device, so each host thread keeps one pair per device it has profiled on; g_prof_dev is the
// device of the last complete pair.
thread_local bool g_prof_on = false;
thread_local cudaEvent_t g_prof_ev[MAX_DEVICES][2] = {};
thread_local int g_prof_dev = -1;
thread_local bool g_prof_open = false;
void prof_mark(int which, cudaStream_t st) {
  if (!g_prof_on) return;
  const int dev = current_device();
  if (dev < 0) return;
  if (!g_prof_ev[dev][0] &&
      (cudaEventCreate(&g_prof_ev[dev][0]) != cudaSuccess || cudaEventCreate(&g_prof_ev[dev][1]) != cudaSuccess)) {
    cudaGetLastError();
    return;
  }
  if (which == 0) {
    g_prof_dev = -1;
    g_prof_open = cudaEventRecord(g_prof_ev[dev][0], st) == cudaSuccess;
  } else if (g_prof_open && cudaEventRecord(g_prof_ev[dev][1], st) == cudaSuccess) {
    g_prof_dev = dev;
  }
  if (which == 1) g_prof_open = false;
}

// One-time, per-device set-up steps (kernel attributes) may be reached from several host threads at
// once.  The steps are idempotent, so an atomic flag per device is enough: two threads may both run a
// step, none reads a half-written flag.
template <typename F>
int once_per_device(std::atomic<int> (&done)[MAX_DEVICES], F &&step) {
  const int dev = current_device();
  if (dev >= 0 && done[dev].load(std::memory_order_acquire)) return QW_OK;
  const int rc = step();
  if (rc == QW_OK && dev >= 0) done[dev].store(1, std::memory_order_release);
  return rc;
}

bool geometry_ok(int dim, int kv_heads, int q_heads) {
  return dim == HEAD_DIM && (kv_heads == 1 || kv_heads == 2 || kv_heads == 4) && q_heads == GROUP * kv_heads;
}

RopeTable make_rope_table(float theta, int rot) {
  RopeTable t;
  for (int i = 0; i < ROT_PAIRS; ++i) t.inv_freq[i] = pow((double)theta, -2.0 * (double)i / (double)rot);
  return t;
}

int sm_count() {
  static std::atomic<int> cached[MAX_DEVICES];
  const int dev = current_device();
  if (dev < 0) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (!n) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// cuTensorMapEncodeTiled through the runtime's entry-point lookup: no link-time libcuda.
typedef CUresult (*encode_fn_t)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
encode_fn_t encode_fn() {
  static encode_fn_t fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<encode_fn_t>(p);
  });
  return fn;
}

// Map over a bf16 matrix [rows][width] (row-major, width*2 bytes per row); box = 64 elements
// (128 bytes, the swizzle span) x box_rows rows.  Out-of-range rows read as zero.
int make_rowmajor_map(CUtensorMap *map, const void *base, int64_t rows, int width, int box_rows) {
  encode_fn_t fn = encode_fn();
  if (!fn) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled entry point not found");
    return QW_ERR_CUDA;
  }
  if (reinterpret_cast<uintptr_t>(base) & 15) return QW_ERR_ARG;
  const cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)width * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return QW_ERR_CUDA;
  }
  return QW_OK;
}

// ---- split-KV launch ------------------------------------------------------------------------
struct AttnCall {
  const void *q;
  bool q_is_f32;
  const uint16_t *gate;
  void *out;
  bool out_is_f32;
  float *lse;
  float *partial_out;
  const uint16_t *kc, *vc;
  int64_t cache_rows;
  const int64_t *cache_row;
  PageMap pages;
  const int *pos;
  const int *q_pos;
  const int *mpos;
  int n_seq, n_new, q_heads, kv_heads;
  float theta, scale;
  bool do_rope, do_gate, no_causal;
  bool q_dep;  // q / gate are produced by the launch before the attention kernel (fused projection rows)
  bool pdl;    // the launch right before the attention kernel is this call's append kernel: overlap with it
  bool no_grid_wait;  // QW_F_NO_GRID_WAIT: no kernel variant whose CTAs wait for one another
  float *ws;
  size_t ws_floats;
  int *cnt;  // zeroed arrival counters (one per unit) or null
  int *status;
};

int splitkv_rb(int n_new) { return n_new < 5 ? n_new : 5; }  // tokens per unit: <= 30 rows = two 16-row tiles
size_t splitkv_slot_floats(int rb) { return (size_t)rb * GROUP * PART_STRIDE; }

template <int MT, int DS, int STAGES, int LOK, typename TIn, typename TOut>
int launch_splitkv_t(const CUtensorMap &mk, const CUtensorMap &mv, const SplitKVParams &p, cudaStream_t st, bool pdl,
                     bool no_grid_wait) {
  // The 8-warp block (producer folded into warp 0) leaves every thread up to 255 registers, which the
  // two-row-tile variant needs.  The one-tile variant is faster with its dedicated producer warp:
  // folded, with Q fragments in registers, config 2 took 140 us instead of 104 us.
  constexpr bool FOLD = MT > 1;
  auto kern = splitkv_kernel<MT, DS, STAGES, LOK, FOLD, TIn, TOut>;
  // Few long units on the whole device (one to four sequences decoding alone: every unit is cut into eight parts or
  // more): the variant whose CTAs merge a unit together, a slice each.  It needs the whole grid resident at once,
  // which one CTA per SM on a grid of the SM count is.
  constexpr bool HAS_SLICED = MT == 1;
  auto kern_sliced = splitkv_kernel<MT, DS, STAGES, LOK, FOLD, TIn, TOut, HAS_SLICED>;
  constexpr size_t smem = splitkv_smem_bytes<MT, DS, STAGES>();
  static std::atomic<int> configured[MAX_DEVICES];
  int rc = once_per_device(configured, [&]() -> int {
    QW_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (HAS_SLICED) QW_CUDA(cudaFuncSetAttribute(kern_sliced, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    return QW_OK;
  });
  if (rc) return rc;
  g_attn_kernel = "splitkv_kernel";
  const bool sliced = HAS_SLICED && !no_grid_wait && p.cnt && p.G == sm_count() && 8ll * p.n_seq * p.nblk * p.kv_heads <= p.G;
  prof_mark(0, st);
  // behind this step's append kernel the launch is a programmatic dependent: it starts while that one still runs
  const cudaError_t le = launch_kernel(sliced ? kern_sliced : kern, dim3(p.G), dim3((SK_KS * DS + (FOLD ? 0 : 1)) * 32),
                                       smem, st, pdl, mk, mv, p);
  prof_mark(1, st);
  if (le != cudaSuccess) {
    ++g_launches;
    return cuda_fail(le, "splitkv_kernel");
  }
  rc = check_launch("splitkv_kernel");
  if (rc) return rc;
  if (p.cnt) return QW_OK;  // units cut across CTAs were merged by their last CTA
  const int n_units = p.n_seq * p.nblk * p.kv_heads;
  splitkv_merge_kernel<TOut><<<n_units, 256, 0, st>>>(p);
  return check_launch("splitkv_merge_kernel");
}

// Picks the instantiation: fp32 queries carry a bf16 "lo" part on all 256 channels (16 k-steps),
// bf16 queries only on the 64 rotated ones (4 k-steps) and none when they arrive rotated.
template <int MT, int STAGES>
int launch_splitkv_mt(const AttnCall &c, const CUtensorMap &mk, const CUtensorMap &mv, const SplitKVParams &p,
                      cudaStream_t st) {
  if (c.q_is_f32) return launch_splitkv_t<MT, 2, STAGES, 16, float, float>(mk, mv, p, st, c.pdl, c.no_grid_wait);
  if (c.out_is_f32)
    return c.do_rope ? launch_splitkv_t<MT, 2, STAGES, 4, uint16_t, float>(mk, mv, p, st, c.pdl, c.no_grid_wait)
                     : launch_splitkv_t<MT, 2, STAGES, 0, uint16_t, float>(mk, mv, p, st, c.pdl, c.no_grid_wait);
  return c.do_rope ? launch_splitkv_t<MT, 2, STAGES, 4, uint16_t, uint16_t>(mk, mv, p, st, c.pdl, c.no_grid_wait)
                   : launch_splitkv_t<MT, 2, STAGES, 0, uint16_t, uint16_t>(mk, mv, p, st, c.pdl, c.no_grid_wait);
}

int launch_splitkv(const AttnCall &c, cudaStream_t st) {
  SplitKVParams p;
  memset(&p, 0, sizeof(p));
  p.q = c.q; p.gate = c.gate; p.out = c.out; p.lse = c.lse; p.partial_out = c.partial_out;
  p.pos = c.pos; p.q_pos = c.q_pos; p.cache_row = c.cache_row; p.pages = c.pages; p.mpos = c.mpos; p.ws = c.ws;
  p.status = c.status; p.cnt = c.cnt;
  p.n_seq = c.n_seq; p.n_new = c.n_new; p.q_heads = c.q_heads; p.kv_heads = c.kv_heads;
  p.rb = splitkv_rb(c.n_new);
  p.nblk = (c.n_new + p.rb - 1) / p.rb;
  const long long n_units = (long long)c.n_seq * p.nblk * c.kv_heads;
  if (n_units > (1 << 24)) return QW_ERR_SHAPE;
  const size_t slot = splitkv_slot_floats(p.rb);
  const long long max_slots = (long long)(c.ws_floats / slot);
  long long G = sm_count();
  if (max_slots - n_units < G) G = max_slots - n_units;
  if (G < 1) return QW_ERR_WORKSPACE;
  p.G = (int)G;
  p.q_lo_dims = c.q_is_f32 ? HEAD_DIM : (c.do_rope ? ROTARY_DIM : 0);
  p.scale_log2 = c.scale * LOG2E;
  p.do_rope = c.do_rope; p.do_gate = c.do_gate && c.gate; p.no_causal = c.no_causal; p.q_dep = c.q_dep;
  p.rope = make_rope_table(c.theta, ROTARY_DIM);

  CUtensorMap mk, mv;
  int rc = make_rowmajor_map(&mk, c.kc, c.cache_rows, c.kv_heads * HEAD_DIM, SK_TK);
  if (rc) return rc;
  rc = make_rowmajor_map(&mv, c.vc, c.cache_rows, c.kv_heads * HEAD_DIM, SK_TK);
  if (rc) return rc;

  const int mt = (p.rb * GROUP + 15) / 16;
  return mt == 1 ? launch_splitkv_mt<1, 3>(c, mk, mv, p, st) : launch_splitkv_mt<2, 3>(c, mk, mv, p, st);
}

long long splitkv_units(int n_seq, int n_new, int kv_heads) {
  const int rb = splitkv_rb(n_new);
  return (long long)n_seq * ((n_new + rb - 1) / rb) * kv_heads;
}
size_t splitkv_ws_floats(int n_seq, int n_new, int kv_heads) {
  return (size_t)(sm_count() + splitkv_units(n_seq, n_new, kv_heads)) * splitkv_slot_floats(splitkv_rb(n_new));
}

// Workspace of the fused mixer: [arrival counters][partial slots].  Sized for whichever split-KV
// kernel needs more (the mma.sync kernel cuts new tokens into blocks of 5, the tcgen05 one of 21).
long long umma_units(int n_seq, int n_new, int kv_heads) {
  const int rb = splitkv_umma_rb(n_new);
  return (long long)n_seq * ((n_new + rb - 1) / rb) * kv_heads;
}
size_t mixer_cnt_bytes(int n_seq, int n_new, int kv_heads) {
  long long n = splitkv_units(n_seq, n_new, kv_heads);
  if (splitkv_umma_usable(n_new) && umma_units(n_seq, n_new, kv_heads) > n) n = umma_units(n_seq, n_new, kv_heads);
  return ((size_t)n * sizeof(int) + 255) & ~(size_t)255;
}
size_t mixer_slot_floats(int n_seq, int n_new, int kv_heads) {
  size_t f = splitkv_ws_floats(n_seq, n_new, kv_heads);
  if (splitkv_umma_usable(n_new)) {
    const size_t g = (size_t)(sm_count() + umma_units(n_seq, n_new, kv_heads)) * splitkv_slot_floats(splitkv_umma_rb(n_new));
    if (g > f) f = g;
  }
  return f;
}
// Which split-KV kernel serves chunks of n_new < 64 tokens in the fused path: the tcgen05 one for
// two or more new tokens (environment QWB_DECODE_KERNEL=umma / mma overrides, for experiments).
bool prefer_umma_decode(int n_new) {
  static std::atomic<int> cached{-1};
  int mode = cached.load(std::memory_order_relaxed);
  if (mode < 0) {
    const char *e = getenv("QWB_DECODE_KERNEL");
    mode = !e ? 0 : (e[0] == 'u' ? 1 : (e[0] == 'm' ? 2 : 0));
    cached.store(mode, std::memory_order_relaxed);
  }
  if (mode == 1) return true;
  if (mode == 2) return false;
  return n_new >= 2;
}

int launch_splitkv_umma_call(const AttnCall &c, cudaStream_t st) {
  SplitKVParams p;
  memset(&p, 0, sizeof(p));
  p.q = c.q; p.gate = c.gate; p.out = c.out; p.lse = c.lse; p.partial_out = c.partial_out;
  p.pos = c.pos; p.q_pos = c.q_pos; p.cache_row = c.cache_row; p.pages = c.pages; p.mpos = c.mpos; p.ws = c.ws;
  p.status = c.status; p.cnt = c.cnt;
  p.n_seq = c.n_seq; p.n_new = c.n_new; p.q_heads = c.q_heads; p.kv_heads = c.kv_heads;
  p.rb = splitkv_umma_rb(c.n_new);
  p.nblk = (c.n_new + p.rb - 1) / p.rb;
  splitkv_umma_layout(p.rb, &p.q_rows_pad, &p.nslot);
  const long long n_units = (long long)c.n_seq * p.nblk * c.kv_heads;
  if (n_units > (1 << 24)) return QW_ERR_SHAPE;
  const long long max_slots = (long long)(c.ws_floats / splitkv_slot_floats(p.rb));
  long long G = sm_count();
  if (max_slots - n_units < G) G = max_slots - n_units;
  if (G < 1) return QW_ERR_WORKSPACE;
  p.G = (int)G;
  // few long units on the whole device: all CTAs of a unit merge it together (see splitkv_kernel's sliced variant)
  p.sliced = (!c.no_grid_wait && c.cnt && p.G == sm_count() && 8 * n_units <= p.G) ? 1 : 0;
  p.q_lo_dims = c.do_rope ? ROTARY_DIM : 0;
  p.scale_log2 = c.scale * LOG2E;
  p.do_rope = c.do_rope; p.do_gate = c.do_gate && c.gate; p.no_causal = c.no_causal; p.q_dep = c.q_dep;
  p.rope = make_rope_table(c.theta, ROTARY_DIM);
  CUtensorMap mk, mv;
  int rc = make_rowmajor_map(&mk, c.kc, c.cache_rows, c.kv_heads * HEAD_DIM, 128);
  if (rc) return rc;
  rc = make_rowmajor_map(&mv, c.vc, c.cache_rows, c.kv_heads * HEAD_DIM, 64);
  if (rc) return rc;
  g_attn_kernel = "splitkv_umma_kernel";
  prof_mark(0, st);
  rc = launch_splitkv_umma(mk, mv, p, c.out_is_f32, st, c.pdl);
  prof_mark(1, st);
  ++g_launches;
  if (rc == QW_ERR_CUDA) return cuda_fail(cudaGetLastError(), "splitkv_umma_kernel");
  return rc;
}

// The fused projection rows of qw_mixer_forward_fused, when that is the caller.
struct FusedRows {
  const void *rows;
  bool is_f32;
  const uint16_t *q_norm_w, *k_norm_w;
  float eps;
};

bool desc_ok(const qw_mixer_desc *d, const FusedRows *fr) {
  if (!d || d->n_seq < 0 || d->n_new < 0) return false;
  if (!d->kc || !d->vc || !d->pos || d->cache_rows <= 0) return false;
  if (d->flags & QW_F_NO_ATTENTION) return !fr && (d->flags & QW_F_APPEND) && d->k_new && d->v_new;
  if (!d->q || !d->out) return false;
  if (fr) {
    if (!fr->rows || !fr->q_norm_w || !fr->k_norm_w || !d->gate || !(d->flags & QW_F_APPEND)) return false;
  } else if ((d->flags & QW_F_APPEND) && (!d->k_new || !d->v_new)) {
    return false;
  }
  if ((d->flags & QW_F_GATE) && !d->gate) return false;
  return true;
}

// The append kernels run right in front of an attention kernel that takes nearly all of an SM's shared
// memory.  Asking for the same carve-out here spares the SMs a reconfiguration of the L1 / shared
// split between the two launches of a step.
void prefer_max_shared_once() {
  static std::atomic<int> done[MAX_DEVICES];
  once_per_device(done, []() -> int {
    cudaFuncSetAttribute(rope_append_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(fused_rows_kernel<float>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(fused_rows_kernel<uint16_t>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    cudaGetLastError();  // a refusal of the hint is harmless
    return QW_OK;
  });
}

// What the split-KV launch of a fused call will be: which kernel, how many units, floats per slot.
struct SplitPlan {
  bool umma;
  long long units;
  size_t slot;
};
SplitPlan split_plan(int n_seq, int n_new, int kv_heads, bool allow_umma) {
  SplitPlan sp;
  sp.umma = allow_umma && splitkv_umma_usable(n_new) && prefer_umma_decode(n_new);
  sp.units = sp.umma ? umma_units(n_seq, n_new, kv_heads) : splitkv_units(n_seq, n_new, kv_heads);
  sp.slot = splitkv_slot_floats(sp.umma ? splitkv_umma_rb(n_new) : splitkv_rb(n_new));
  return sp;
}

int mixer_forward_impl(const qw_mixer_desc *d, float *partial, cudaStream_t st, const FusedRows *fr = nullptr) {
  g_launches = 0;
  g_attn_kernel = "";
  if (!desc_ok(d, fr)) return QW_ERR_ARG;
  if (!geometry_ok(d->head_dim, d->kv_heads, d->q_heads) || d->rotary_dim != ROTARY_DIM) return QW_ERR_SHAPE;
  if (d->n_seq == 0 || d->n_new == 0) return QW_OK;
  if ((long long)d->n_seq * d->n_new > (1ll << 30)) return QW_ERR_SHAPE;
  const RopeTable tab = make_rope_table(d->theta, ROTARY_DIM);
  PageMap pm = {nullptr, 0, 0};
  if (d->block_table) {
    if (d->page_rows <= 0 || d->page_rows % 128 || d->block_table_stride <= 0) return QW_ERR_ARG;
    pm.table = d->block_table; pm.stride = d->block_table_stride; pm.page_rows = d->page_rows;
  }
  if ((d->flags & QW_F_NO_CAUSAL) && (d->flags & QW_F_APPEND)) return QW_ERR_ARG;  // a sub-range call never owns the new rows
  // the rows of a sub-range call do not sit at pos[s] + b: their angles need q_pos (or mpos)
  if ((d->flags & QW_F_NO_CAUSAL) && (d->flags & QW_F_ROPE) && !d->q_pos && !d->mpos) return QW_ERR_ARG;
  if (d->flags & QW_F_NO_ATTENTION) {  // rope(k) + append only
    if (partial) return QW_ERR_ARG;
    launch_kernel(rope_append_kernel, dim3((unsigned)((size_t)d->n_seq * d->n_new)), dim3(128), 0, st, true, d->k_new,
                  d->v_new, d->kc, d->vc, d->pos, d->cache_row, d->mpos, d->n_new, d->kv_heads,
                  (d->flags & QW_F_ROPE) ? 1 : 0, tab, static_cast<int *>(nullptr), 0, pm, d->q_pos);
    return check_launch("rope_append_kernel");
  }
  const bool use_umma =
      !(d->flags & (QW_F_NO_UMMA | QW_F_NO_CAUSAL)) && !partial && prefill_umma_supported(d->n_new);
  // Workspace of the split-KV kernels: arrival counters (one per unit), then the partial slots.  The
  // counters let the CTA that completes a unit last merge it inside the attention kernel; they must be
  // zero at launch: the append kernel of the same call clears them, a memset node when there is none.
  // Everything about the workspace is checked before the first launch, so that an error return means
  // that nothing was enqueued and nothing (cache, q, gate) was touched.
  const size_t cnt_bytes = mixer_cnt_bytes(d->n_seq, d->n_new, d->kv_heads);
  const SplitPlan sp = split_plan(d->n_seq, d->n_new, d->kv_heads, !(d->flags & QW_F_NO_UMMA));
  int *cnt = nullptr;
  float *ws = nullptr;
  size_t ws_floats = 0;
  if (!use_umma) {
    if (!d->workspace || (reinterpret_cast<uintptr_t>(d->workspace) & 15) || d->workspace_bytes <= cnt_bytes)
      return QW_ERR_WORKSPACE;
    cnt = reinterpret_cast<int *>(d->workspace);
    ws = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(d->workspace) + cnt_bytes);
    ws_floats = (d->workspace_bytes - cnt_bytes) / sizeof(float);
    if (sp.units > (1 << 24)) return QW_ERR_SHAPE;
    if ((long long)(ws_floats / sp.slot) - sp.units < 1) return QW_ERR_WORKSPACE;  // not even one CTA's slot
  }
  const int n_zero = cnt ? (int)(cnt_bytes / sizeof(int)) : 0;
  bool appended = false;
  if (fr) {
    prefer_max_shared_once();
    const unsigned rows = (unsigned)((size_t)d->n_seq * d->n_new);
    uint16_t *qo = const_cast<uint16_t *>(d->q), *go = const_cast<uint16_t *>(d->gate);
    const int do_rope = (d->flags & QW_F_ROPE) ? 1 : 0;
    if (fr->is_f32)
      launch_kernel(fused_rows_kernel<float>, dim3(rows, (unsigned)d->kv_heads), dim3(256), 0, st, true,
                    static_cast<const float *>(fr->rows), fr->q_norm_w, fr->k_norm_w, fr->eps, qo, go, d->kc, d->vc, d->pos,
                    d->cache_row, d->mpos, d->n_new, d->q_heads, d->kv_heads, do_rope, tab, cnt, n_zero, pm, d->q_pos);
    else
      launch_kernel(fused_rows_kernel<uint16_t>, dim3(rows, (unsigned)d->kv_heads), dim3(256), 0, st, true,
                    static_cast<const uint16_t *>(fr->rows), fr->q_norm_w, fr->k_norm_w, fr->eps, qo, go, d->kc, d->vc, d->pos,
                    d->cache_row, d->mpos, d->n_new, d->q_heads, d->kv_heads, do_rope, tab, cnt, n_zero, pm, d->q_pos);
    int rc = check_launch("fused_rows_kernel");
    if (rc) return rc;
    appended = true;
  } else if (d->flags & QW_F_APPEND) {
    prefer_max_shared_once();
    launch_kernel(rope_append_kernel, dim3((unsigned)((size_t)d->n_seq * d->n_new)), dim3(128), 0, st, true, d->k_new,
                  d->v_new, d->kc, d->vc, d->pos, d->cache_row, d->mpos, d->n_new, d->kv_heads,
                  (d->flags & QW_F_ROPE) ? 1 : 0, tab, cnt, n_zero, pm, d->q_pos);
    int rc = check_launch("rope_append_kernel");
    if (rc) return rc;
    appended = true;
  } else if (cnt) {
    QW_CUDA(cudaMemsetAsync(cnt, 0, cnt_bytes, st));
  }
  if (use_umma) {
    PrefillCall pc;
    memset(&pc, 0, sizeof(pc));
    pc.q = d->q; pc.gate = (d->flags & QW_F_GATE) ? d->gate : nullptr; pc.out = d->out;
    pc.out_is_f32 = (d->flags & QW_F_OUT_F32) != 0; pc.lse = d->lse;
    pc.kc = d->kc; pc.vc = d->vc; pc.cache_rows = d->cache_rows; pc.cache_row = d->cache_row; pc.pages = pm;
    pc.pos = d->pos; pc.q_pos = d->q_pos; pc.mpos = d->mpos; pc.n_seq = d->n_seq; pc.n_new = d->n_new;
    pc.q_heads = d->q_heads; pc.kv_heads = d->kv_heads; pc.scale = d->scale;
    pc.do_rope = (d->flags & QW_F_ROPE) != 0; pc.status = d->status;
    pc.rope = tab;
    pc.fast_p = (d->flags & QW_F_FAST_P) ? 1 : 0;
    int n = 0;
    g_attn_kernel = "prefill_umma_pair_kernel";
    prof_mark(0, st);
    int rc = launch_prefill_umma_pair(pc, st, &n);
    prof_mark(1, st);
    g_launches += n;
    if (rc == QW_ERR_CUDA) {
      cudaError_t e = cudaGetLastError();
      return cuda_fail(e, "prefill_umma_pair_kernel");
    }
    return rc;
  }
  AttnCall c;
  memset(&c, 0, sizeof(c));
  c.q = d->q; c.q_is_f32 = false; c.gate = d->gate; c.out = d->out;
  c.out_is_f32 = (d->flags & QW_F_OUT_F32) != 0; c.lse = d->lse; c.partial_out = partial;
  c.kc = d->kc; c.vc = d->vc; c.cache_rows = d->cache_rows; c.cache_row = d->cache_row; c.pages = pm;
  c.pos = d->pos; c.q_pos = d->q_pos; c.mpos = d->mpos; c.n_seq = d->n_seq; c.n_new = d->n_new;
  c.q_heads = d->q_heads; c.kv_heads = d->kv_heads; c.theta = d->theta; c.scale = d->scale;
  c.do_rope = (d->flags & QW_F_ROPE) != 0; c.do_gate = (d->flags & QW_F_GATE) != 0;
  c.no_causal = (d->flags & QW_F_NO_CAUSAL) != 0;
  c.q_dep = fr != nullptr;
  c.pdl = appended;
  c.no_grid_wait = (d->flags & QW_F_NO_GRID_WAIT) != 0;
  c.ws = ws;
  c.ws_floats = ws_floats;
  c.cnt = cnt;
  c.status = d->status;
  return sp.umma ? launch_splitkv_umma_call(c, st) : launch_splitkv(c, st);
}

// ---- allocation-free decode: split-KV partials in a fixed array inside the library image --------
// Sized for the largest request the entry point accepts: B <= 8 tokens (two unit blocks of <= 5)
// and kv_heads <= 4 give at most 8 units; up to 160 CTAs; one slot = 5 tokens x 6 heads x 260 floats.
constexpr int NOALLOC_MAX_B = 8;
constexpr int NOALLOC_MAX_KV_HEADS = 4;
constexpr size_t NOALLOC_SCRATCH_FLOATS = (size_t)(160 + 2 * NOALLOC_MAX_KV_HEADS) * 5 * GROUP * PART_STRIDE;
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_SCRATCH_FLOATS];

// In host code the name g_noalloc_scratch is only a handle for the symbol, not an address a kernel
// could use.  The device address is looked up once per device, with that device current.
int noalloc_scratch_address(float **out) {
  static std::mutex mu;
  static float *addr[MAX_DEVICES] = {nullptr};
  int dev = 0;
  QW_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) return QW_ERR_ARG;
  std::lock_guard<std::mutex> lock(mu);
  if (!addr[dev]) {
    void *p = nullptr;
    QW_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    if (!p) return QW_ERR_CUDA;
    addr[dev] = static_cast<float *>(p);
  }
  *out = addr[dev];
  return QW_OK;
}

// Drop-in attention launchers share this: one sequence, rows already rotated and appended
// (src/model.cu:228-236, src/prefill.cu:142-152 of the reference run rope and k_kv_append first).
//   chunks of >= 64 rows      tcgen05 CTA-pair prefill kernel (an fp32 q is first copied to bf16 in scratch)
//   2..63 rows, bf16          tcgen05 split-KV kernel
//   1 row, and fp32 < 64 rows mma.sync split-KV kernel (fp32 q kept exact as bf16 hi + lo)
// Split-KV arrival counters sit at the head of the scratch and are cleared by a memset node in front of
// the kernel, which is legal inside a stream capture.
template <typename T>
int attn_dropin(const T *q, const qw_bf16 *kc, const qw_bf16 *vc, T *out, const int *dpos, int dim, int kv_heads,
                int q_heads, float scale, float *scratch, int ctx, int rows, bool decode, cudaStream_t st) {
  constexpr bool F32 = sizeof(T) == 4;
  g_launches = 0;
  g_attn_kernel = "";
  if (!q || !kc || !vc || !out || !dpos || !scratch || ctx <= 0 || rows < 0) return QW_ERR_ARG;
  if (reinterpret_cast<uintptr_t>(scratch) & 15) return QW_ERR_ARG;
  if (!geometry_ok(dim, kv_heads, q_heads)) return QW_ERR_SHAPE;
  if (decode && rows > 8) return QW_ERR_SHAPE;
  if (rows == 0) return QW_OK;
  // The launcher is not told how large `scratch` is.  A caller may have sized it as the reference does
  // (rows * q_heads * ctx floats: src/model.cu:168, src/prefill.cu:75) or, for prefill, by the query function; the
  // launcher counts on the smaller of the two and, where that does not hold what the call needs (a cache of a few
  // hundred rows: the reference sizes ctx as prompt + new tokens + 8, src/main.cu:38), leaves `scratch` untouched
  // and uses the library's own fixed array, as the allocation-free entry point does.
  const size_t ref_size = (size_t)rows * q_heads * ctx;
  const size_t have = decode ? ref_size : std::min(ref_size, qw_attn_prefill_scratch_floats(q_heads, kv_heads, ctx, rows));
  if (!decode && prefill_umma_supported(rows)) {
    const uint16_t *qb = reinterpret_cast<const uint16_t *>(q);
    if (F32) {
      const long long n = (long long)rows * q_heads * HEAD_DIM;
      uint16_t *copy = reinterpret_cast<uint16_t *>(scratch);
      if (have < (size_t)n / 2) {  // ctx < 128: the bf16 copy of q does not fit the reference-sized buffer
        if ((size_t)n / 2 > NOALLOC_SCRATCH_FLOATS) return QW_ERR_WORKSPACE;  // not reachable: rows <= ctx < 128
        float *own = nullptr;
        int rc = noalloc_scratch_address(&own);
        if (rc) return rc;
        copy = reinterpret_cast<uint16_t *>(own);
      }
      to_bf16_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, st>>>(reinterpret_cast<const float *>(q), copy, n);
      int rc = check_launch("to_bf16_kernel");
      if (rc) return rc;
      qb = copy;
    }
    PrefillCall pc;
    memset(&pc, 0, sizeof(pc));
    pc.q = qb; pc.out = out; pc.out_is_f32 = F32;
    pc.kc = kc; pc.vc = vc; pc.cache_rows = ctx; pc.pos = dpos;
    pc.n_seq = 1; pc.n_new = rows; pc.q_heads = q_heads; pc.kv_heads = kv_heads; pc.scale = scale;
    pc.rope = make_rope_table(1e7f, ROTARY_DIM);  // unused: q arrives rotated
    int n = 0;
    g_attn_kernel = "prefill_umma_pair_kernel";
    prof_mark(0, st);
    int rc = launch_prefill_umma_pair(pc, st, &n);
    prof_mark(1, st);
    g_launches += n;
    if (rc == QW_ERR_CUDA) return cuda_fail(cudaGetLastError(), "prefill_umma_pair_kernel");
    return rc;
  }
  const SplitPlan sp = split_plan(1, rows, kv_heads, !F32);
  const size_t cnt_bytes = mixer_cnt_bytes(1, rows, kv_heads);
  const bool scratch_short = have * sizeof(float) <= cnt_bytes ||
                             (long long)((have - cnt_bytes / sizeof(float)) / sp.slot) - sp.units < 1;
  if (scratch_short) {  // not even one set of split-KV partials: they go to the fixed array
    float *own = nullptr;
    int rc = noalloc_scratch_address(&own);
    if (rc) return rc;
    AttnCall c;
    memset(&c, 0, sizeof(c));
    c.q = q; c.q_is_f32 = F32; c.out = out; c.out_is_f32 = F32;
    c.kc = kc; c.vc = vc; c.cache_rows = ctx; c.pos = dpos;
    c.n_seq = 1; c.n_new = rows; c.q_heads = q_heads; c.kv_heads = kv_heads;
    c.theta = 1e7f; c.scale = scale;
    c.ws = own; c.ws_floats = NOALLOC_SCRATCH_FLOATS;
    return launch_splitkv(c, st);
  }
  AttnCall c;
  memset(&c, 0, sizeof(c));
  c.q = q; c.q_is_f32 = F32; c.out = out; c.out_is_f32 = F32;
  c.kc = kc; c.vc = vc; c.cache_rows = ctx; c.pos = dpos;
  c.n_seq = 1; c.n_new = rows; c.q_heads = q_heads; c.kv_heads = kv_heads;
  c.theta = 1e7f; c.scale = scale;
  c.cnt = reinterpret_cast<int *>(scratch);
  c.ws = scratch + cnt_bytes / sizeof(float);
  c.ws_floats = have - cnt_bytes / sizeof(float);
  QW_CUDA(cudaMemsetAsync(c.cnt, 0, cnt_bytes, st));
  return sp.umma ? launch_splitkv_umma_call(c, st) : launch_splitkv(c, st);
}

}  // namespace


extern "C" {

const char *qw_strerror(int code) {
  switch (code) {
    case QW_OK: return "ok";
    case QW_ERR_ARG: return "bad argument (null pointer, negative count or misaligned buffer)";
    case QW_ERR_SHAPE: return "unsupported geometry (need head_dim 256, rotary 64, q_heads = 6 * kv_heads, kv_heads 1/2/4)";
    case QW_ERR_CUDA: return "a CUDA call failed (see qw_last_cuda_error)";
    case QW_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case QW_ERR_DEVICE: return "a kernel reported an error through the status word";
    case QW_ERR_TOO_LARGE: return "request exceeds a fixed built-in capacity (allocation-free decode: B <= 8, kv_heads <= 4)";
    default: return "unknown error code";
  }
}
int qw_abi_version(void) { return 3; }
const char *qw_last_cuda_error(void) { return g_cuda_err; }
int qw_last_launch_count(void) { return g_launches; }
const char *qw_last_attention_kernel(void) { return g_attn_kernel; }

int qw_profile_enable(int on) {
  g_prof_on = on != 0;
  g_prof_dev = -1;
  g_prof_open = false;
  return QW_OK;
}
int qw_profile_last_kernel_ms(float *ms) {
  if (!ms || g_prof_dev < 0) return QW_ERR_ARG;
  QW_CUDA(cudaEventSynchronize(g_prof_ev[g_prof_dev][1]));
  QW_CUDA(cudaEventElapsedTime(ms, g_prof_ev[g_prof_dev][0], g_prof_ev[g_prof_dev][1]));
  return QW_OK;
}

int qw_rope_bf16(qw_bf16 *v, int heads, int dim, int rot, const int *dpos, float theta, qw_stream stream, int B,
                 const int *mpos) {
  g_launches = 0;
  if (!v || !dpos || heads <= 0 || B < 0) return QW_ERR_ARG;
  if (dim != HEAD_DIM || rot != ROTARY_DIM) return QW_ERR_SHAPE;
  if (B == 0) return QW_OK;
  rope_inplace_kernel<uint16_t><<<dim3(heads, B), 32, 0, (cudaStream_t)stream>>>(v, heads, dpos, mpos,
                                                                                 make_rope_table(theta, rot));
  return check_launch("rope_inplace_kernel");
}
int qw_rope_f32(float *v, int heads, int dim, int rot, const int *dpos, float theta, qw_stream stream, int B,
                const int *mpos) {
  g_launches = 0;
  if (!v || !dpos || heads <= 0 || B < 0) return QW_ERR_ARG;
  if (dim != HEAD_DIM || rot != ROTARY_DIM) return QW_ERR_SHAPE;
  if (B == 0) return QW_OK;
  rope_inplace_kernel<float><<<dim3(heads, B), 32, 0, (cudaStream_t)stream>>>(v, heads, dpos, mpos,
                                                                              make_rope_table(theta, rot));
  return check_launch("rope_inplace_kernel");
}

int qw_kv_append_bf16(const qw_bf16 *k, const qw_bf16 *v, qw_bf16 *kc, qw_bf16 *vc, const int *dpos, int kvdim,
                      int B, qw_stream stream) {
  g_launches = 0;
  if (!k || !v || !kc || !vc || !dpos || kvdim <= 0 || B < 0) return QW_ERR_ARG;
  if (kvdim % 8) return QW_ERR_SHAPE;
  if (B == 0) return QW_OK;
  kv_append_kernel<uint16_t><<<dim3((kvdim + 2047) / 2048, B), 256, 0, (cudaStream_t)stream>>>(k, v, kc, vc, dpos,
                                                                                              kvdim);
  return check_launch("kv_append_kernel");
}
int qw_kv_append_f32(const float *k, const float *v, qw_bf16 *kc, qw_bf16 *vc, const int *dpos, int kvdim, int B,
                     qw_stream stream) {
  g_launches = 0;
  if (!k || !v || !kc || !vc || !dpos || kvdim <= 0 || B < 0) return QW_ERR_ARG;
  if (kvdim % 8) return QW_ERR_SHAPE;
  if (B == 0) return QW_OK;
  kv_append_kernel<float><<<dim3((kvdim + 2047) / 2048, B), 256, 0, (cudaStream_t)stream>>>(k, v, kc, vc, dpos,
                                                                                           kvdim);
  return check_launch("kv_append_kernel");
}

int qw_gate_sigmoid_bf16(qw_bf16 *x, const qw_bf16 *gate, int n, qw_stream stream) {
  g_launches = 0;
  if (!x || !gate || n < 0) return QW_ERR_ARG;
  if (n % 8) return QW_ERR_SHAPE;
  if (n == 0) return QW_OK;
  gate_sigmoid_kernel<uint16_t><<<(n / 8 + 255) / 256, 256, 0, (cudaStream_t)stream>>>(x, gate, n);
  return check_launch("gate_sigmoid_kernel");
}
int qw_gate_sigmoid_f32(float *x, const float *gate, int n, qw_stream stream) {
  g_launches = 0;
  if (!x || !gate || n < 0) return QW_ERR_ARG;
  if (n % 8) return QW_ERR_SHAPE;
  if (n == 0) return QW_OK;
  gate_sigmoid_kernel<float><<<(n / 8 + 255) / 256, 256, 0, (cudaStream_t)stream>>>(x, gate, n);
  return check_launch("gate_sigmoid_kernel");
}

size_t qw_attn_decode_scratch_floats(int q_heads, int kv_heads, int ctx, int B) {
  (void)kv_heads;
  if (B <= 0 || q_heads <= 0 || ctx <= 0) return 0;
  return (size_t)B * q_heads * ctx;  // the reference kernel's own need at the same launch; all of it is used
}
size_t qw_attn_prefill_scratch_floats(int q_heads, int kv_heads, int ctx, int T) {
  (void)ctx;
  if (T <= 0 || kv_heads <= 0 || q_heads <= 0) return 0;
  if (prefill_umma_supported(T)) return (size_t)T * q_heads * (HEAD_DIM / 2);  // bf16 copy of an fp32 q
  return mixer_cnt_bytes(1, T, kv_heads) / sizeof(float) + mixer_slot_floats(1, T, kv_heads);
}

int qw_attn_decode_bf16(const qw_bf16 *q, const qw_bf16 *kc, const qw_bf16 *vc, qw_bf16 *out, const int *dpos,
                        int dim, int kv_heads, int q_heads, float scale, float *scratch, int ctx, int B,
                        qw_stream stream) {
  return attn_dropin<qw_bf16>(q, kc, vc, out, dpos, dim, kv_heads, q_heads, scale, scratch, ctx, B, true,
                              (cudaStream_t)stream);
}
int qw_attn_decode_f32(const float *q, const qw_bf16 *kc, const qw_bf16 *vc, float *out, const int *dpos, int dim,
                       int kv_heads, int q_heads, float scale, float *scratch, int ctx, int B, qw_stream stream) {
  return attn_dropin<float>(q, kc, vc, out, dpos, dim, kv_heads, q_heads, scale, scratch, ctx, B, true,
                            (cudaStream_t)stream);
}
int qw_attn_decode_bf16_noalloc(const qw_bf16 *q, const qw_bf16 *kc, const qw_bf16 *vc, qw_bf16 *out,
                                const int *dpos, int dim, int kv_heads, int q_heads, float scale, int ctx, int B,
                                qw_stream stream) {
  g_launches = 0;
  if (!q || !kc || !vc || !out || !dpos || ctx <= 0 || B < 0) return QW_ERR_ARG;
  if (!geometry_ok(dim, kv_heads, q_heads)) return QW_ERR_SHAPE;
  if (B > NOALLOC_MAX_B || kv_heads > NOALLOC_MAX_KV_HEADS) return QW_ERR_TOO_LARGE;
  if (B == 0) return QW_OK;
  float *scratch = nullptr;
  int rc = noalloc_scratch_address(&scratch);
  if (rc) return rc;
  AttnCall c;
  memset(&c, 0, sizeof(c));
  c.q = q; c.out = out; c.kc = kc; c.vc = vc; c.cache_rows = ctx; c.pos = dpos;
  c.n_seq = 1; c.n_new = B; c.q_heads = q_heads; c.kv_heads = kv_heads;
  c.theta = 1e7f; c.scale = scale;
  c.ws = scratch; c.ws_floats = NOALLOC_SCRATCH_FLOATS;
  return launch_splitkv(c, (cudaStream_t)stream);
}

int qw_attn_prefill_bf16(const qw_bf16 *q, const qw_bf16 *kc, const qw_bf16 *vc, qw_bf16 *out, const int *dpos,
                         int dim, int kv_heads, int q_heads, float scale, float *scratch, int ctx, int T,
                         qw_stream stream) {
  return attn_dropin<qw_bf16>(q, kc, vc, out, dpos, dim, kv_heads, q_heads, scale, scratch, ctx, T, false,
                              (cudaStream_t)stream);
}
int qw_attn_prefill_f32(const float *q, const qw_bf16 *kc, const qw_bf16 *vc, float *out, const int *dpos, int dim,
                        int kv_heads, int q_heads, float scale, float *scratch, int ctx, int T, qw_stream stream) {
  return attn_dropin<float>(q, kc, vc, out, dpos, dim, kv_heads, q_heads, scale, scratch, ctx, T, false,
                            (cudaStream_t)stream);
}

size_t qw_mixer_workspace_bytes(const qw_mixer_desc *d) {
  if (!d || d->n_seq <= 0 || d->n_new <= 0 || d->kv_heads <= 0) return 256;
  return mixer_cnt_bytes(d->n_seq, d->n_new, d->kv_heads) +
         mixer_slot_floats(d->n_seq, d->n_new, d->kv_heads) * sizeof(float) + 256;
}
int qw_mixer_forward(const qw_mixer_desc *d, qw_stream stream) {
  return mixer_forward_impl(d, nullptr, (cudaStream_t)stream);
}
int qw_mixer_forward_fused(const qw_mixer_desc *d, const void *fused, int fused_is_f32, const qw_bf16 *q_norm_w,
                           const qw_bf16 *k_norm_w, float eps, qw_stream stream) {
  if ((reinterpret_cast<uintptr_t>(fused) & 15) || (reinterpret_cast<uintptr_t>(q_norm_w) & 15) ||
      (reinterpret_cast<uintptr_t>(k_norm_w) & 15) || !(eps >= 0.f))
    return QW_ERR_ARG;
  const FusedRows fr = {fused, fused_is_f32 != 0, q_norm_w, k_norm_w, eps};
  return mixer_forward_impl(d, nullptr, (cudaStream_t)stream, &fr);
}
int qw_mixer_forward_partial(const qw_mixer_desc *d, float *partial, qw_stream stream) {
  if (!partial) return QW_ERR_ARG;
  return mixer_forward_impl(d, partial, (cudaStream_t)stream);
}

int qw_combine_partials(const float *parts, int n_parts, int64_t rows, int q_heads, const qw_bf16 *gate, void *out,
                        float *lse, int flags, qw_stream stream) {
  g_launches = 0;
  if (!parts || !out || n_parts <= 0 || rows < 0 || q_heads <= 0) return QW_ERR_ARG;
  if ((flags & QW_F_GATE) && !gate) return QW_ERR_ARG;
  if (rows == 0) return QW_OK;
  const long long n = (long long)rows * q_heads;
  const unsigned blocks = (unsigned)((n + 7) / 8);
  if (flags & QW_F_OUT_F32)
    combine_partials_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>(
        parts, n_parts, n, (flags & QW_F_GATE) ? gate : nullptr, reinterpret_cast<float *>(out), lse);
  else
    combine_partials_kernel<uint16_t><<<blocks, 256, 0, (cudaStream_t)stream>>>(
        parts, n_parts, n, (flags & QW_F_GATE) ? gate : nullptr, reinterpret_cast<uint16_t *>(out), lse);
  return check_launch("combine_partials_kernel");
}

int qw_combine_partials_peer(const float *const *part_ptrs, int *const *flag_ptrs, int rank, int n_parts, int step,
                             int64_t rows, int q_heads, const qw_bf16 *gate, void *out, float *lse, int flags, int *status,
                             qw_stream stream) {
  g_launches = 0;
  if (!part_ptrs || !flag_ptrs || !out || n_parts <= 0 || rank < 0 || rank >= n_parts || rows < 0 || q_heads <= 0 || step <= 0)
    return QW_ERR_ARG;
  if ((flags & QW_F_GATE) && !gate) return QW_ERR_ARG;
  if (rows == 0) return QW_OK;
  const long long n = (long long)rows * q_heads;
  const unsigned blocks = (unsigned)((n + 7) / 8);
  if (flags & QW_F_OUT_F32)
    combine_partials_peer_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>(
        part_ptrs, flag_ptrs, rank, n_parts, step, n, (flags & QW_F_GATE) ? gate : nullptr, reinterpret_cast<float *>(out),
        lse, status);
  else
    combine_partials_peer_kernel<uint16_t><<<blocks, 256, 0, (cudaStream_t)stream>>>(
        part_ptrs, flag_ptrs, rank, n_parts, step, n, (flags & QW_F_GATE) ? gate : nullptr,
        reinterpret_cast<uint16_t *>(out), lse, status);
  return check_launch("combine_partials_peer_kernel");
}

}  // extern "C"
