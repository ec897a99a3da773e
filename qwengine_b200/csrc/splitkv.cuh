// Split-KV ("flash-decoding") attention for decode, speculative verify and short chunks.
//
// Work model.  A *unit* is one (sequence, block of <= 5 new tokens, KV head): its 6*tokens
// query rows all read the same K/V rows.  The key range of every unit is cut into tiles of
// 64 keys; all tiles of all units form one flat list that is divided evenly over the G CTAs
// of a persistent grid, so ragged batches stay balanced and the grid never depends on a
// length the host does not know (lengths live in device memory so the launch can be replayed
// from a CUDA graph, as the reference's decode graph requires, src/model.cu:318-327).
// A CTA walks its slice as 1..n *segments* (unit, tile range).  A segment that covers its
// whole unit writes the final output; otherwise it writes an un-normalised partial
// (o[256], m, l) to workspace slot (cta + unit), and a second small kernel merges the
// partials of each unit in CTA order -- fixed order, no atomics, bit-stable run to run.
//
// Inside a CTA: one producer warp streams K and V tiles with TMA into a 128-byte-swizzled
// shared-memory ring (HBM is the bound, so bytes in flight are what matter); 4*DS consumer
// warps each own a 16-key slice of the tile (and 256/DS output channels) and run
// QK^T -> online softmax -> PV on mma.sync m16n8k16 bf16 tensor-core tiles with fp32
// accumulation.  Tensor cores are used because at 6 rows per KV head the CUDA-core FMA issue
// time is already ~2/3 of the HBM time, and at 24 rows (4-token verify) 2.5x over it.
// Q (after RoPE) and P are fed as bf16 hi + lo pairs so that neither is rounded to 8 bits.
#pragma once

#include "common.cuh"

namespace qwb {

constexpr int SK_TK = 64;                       // keys per tile
constexpr int SK_TILE_BYTES = SK_TK * 512;      // one head's K (or V) tile: 64 keys x 256 bf16
constexpr int SK_STAGE_BYTES = 2 * SK_TILE_BYTES;
constexpr int SK_KS = SK_TK / 16;               // key slices (consumer warps along keys)

struct SplitKVParams {
  const void *q;          // [n_seq][n_new][q_heads][256]
  const uint16_t *gate;   // same shape, bf16, or null
  void *out;              // same shape
  float *lse;             // [n_seq][n_new][q_heads] or null
  float *partial_out;     // non-null: emit (o, m, l) per (row, head) instead of out / lse
  const int *pos;         // [n_seq]
  const int *q_pos;       // [n_seq] or null: absolute position of a sequence's first new row (RoPE angles) when it is not pos[s]
  const int64_t *cache_row;  // [n_seq] or null
  PageMap pages;             // block table, if the cache is paged
  const int *mpos;        // [n_seq][n_new][3] or null
  float *ws;              // (G + n_units) slots of rb*6*PART_STRIDE floats
  int *cnt;               // per-unit arrival counters (zero at launch) or null: merge in a second kernel
  int *status;
  int n_seq, n_new, q_heads, kv_heads;
  int rb;                 // tokens per unit block
  int nblk;               // blocks per sequence
  int G;                  // CTAs in the grid
  int q_lo_dims;          // 0, 64 or 256: leading dims that carry a bf16 "lo" part
  float scale_log2;       // softmax scale * log2(e)
  int do_rope, do_gate;
  int q_rows_pad;         // tcgen05 kernel: rows of the Q tile that really exist in shared memory (32, 64 or 128)
  int nslot;              // tcgen05 kernel: 16 KB ring slots that fit beside that Q tile
  int sliced;             // tcgen05 kernel: all CTAs of a cut unit merge it together, a slice each (see merge_unit_sliced)
  int q_dep;              // q and gate are written by the launch before this one (fused projection rows)
  int no_causal;          // every row sees exactly pos[s] keys (a KV sub-range without the new rows)
  RopeTable rope;
};

struct UnitInfo {
  int s, blk, kvh;
  int tok0, ntok;   // first new-token index of the block and tokens in it
  int pos;          // tokens cached before the call for this sequence
  int rpos;         // position of the sequence's first new row for the RoPE angles (pos unless q_pos is given)
  int len;          // keys visible to the last row of the unit
};

__device__ __forceinline__ UnitInfo unit_info(const SplitKVParams &p, int u) {
  UnitInfo ui;
  ui.kvh = u % p.kv_heads;
  const int sb = u / p.kv_heads;
  ui.blk = sb % p.nblk;
  ui.s = sb / p.nblk;
  ui.tok0 = ui.blk * p.rb;
  ui.ntok = min(p.rb, p.n_new - ui.tok0);
  ui.pos = p.pos[ui.s];
  ui.rpos = p.q_pos ? p.q_pos[ui.s] : ui.pos;
  ui.len = p.no_causal ? ui.pos : ui.pos + ui.tok0 + ui.ntok;
  return ui;
}
template <int TK = SK_TK>
__device__ __forceinline__ int unit_tiles(const SplitKVParams &p, int u) {
  const UnitInfo ui = unit_info(p, u);
  return (ui.len + TK - 1) / TK;
}

// Warp-cooperative: total number of tiles over all units.
template <int TK = SK_TK>
__device__ __forceinline__ long long warp_total_tiles(const SplitKVParams &p, int n_units, int lane) {
  long long t = 0;
  for (int u = lane; u < n_units; u += 32) t += unit_tiles<TK>(p, u);
#pragma unroll
  for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}
// Warp-cooperative: total tiles, units that have any, and the number of CTAs to spread them over.
// When all units are equally long the grid is trimmed (by at most a fifth) to a count that divides,
// or is divided by, the unit count: every CTA then stays inside one unit, or takes whole units, and
// none pays for a change of unit that its neighbours do not have (`aligned`).
template <int TK = SK_TK>
__device__ __forceinline__ void warp_partition(const SplitKVParams &p, int n_units, int lane, long long &total, int &live,
                                               int &geff, bool &aligned) {
  total = 0;
  live = 0;
  int mn = 0x7fffffff, mx = 0;
  for (int u = lane; u < n_units; u += 32) {
    const int nt = unit_tiles<TK>(p, u);
    total += nt;
    mn = min(mn, nt);
    mx = max(mx, nt);
    live += nt > 0;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    total += __shfl_xor_sync(0xffffffffu, total, o);
    live += __shfl_xor_sync(0xffffffffu, live, o);
    mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  geff = p.G;
  aligned = false;
  if (mn == mx && mx > 0) {
    if (n_units <= p.G) {
      const int k = p.G / n_units;
      if (k * n_units * 5 >= p.G * 4) { geff = k * n_units; aligned = true; }
    } else {
      for (int d = p.G; d * 5 >= p.G * 4; --d)
        if (n_units % d == 0) { geff = d; aligned = true; break; }
    }
  }
}
// Warp-cooperative: the unit containing flat tile g and the flat index of that unit's tile 0.
template <int TK = SK_TK>
__device__ __forceinline__ void warp_find_unit(const SplitKVParams &p, int n_units, int lane, long long g,
                                               int &u_out, long long &pre_out, int extra = 0) {
  long long carry = 0;
  u_out = n_units;
  pre_out = 0;
  for (int base = 0; base < n_units; base += 32) {
    const int u = base + lane;
    long long mine = u < n_units ? unit_tiles<TK>(p, u) : 0;
    if (mine > 0) mine += extra;  // list entries that precede the unit's tiles (see splitkv_umma.cu)
    long long inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const long long v = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += v;
    }
    const long long excl = carry + inc - mine;
    const bool hit = u < n_units && mine > 0 && g >= excl && g < excl + mine;
    const unsigned ball = __ballot_sync(0xffffffffu, hit);
    if (ball) {
      const int src = __ffs(ball) - 1;
      u_out = base + src;
      pre_out = __shfl_sync(0xffffffffu, excl, src);
      return;
    }
    carry += __shfl_sync(0xffffffffu, inc, 31);
  }
}
// Warp-cooperative: flat index of tile 0 of unit u.
template <int TK = SK_TK>
__device__ __forceinline__ long long warp_unit_prefix(const SplitKVParams &p, int u_target, int lane) {
  long long t = 0;
  for (int u = lane; u < u_target; u += 32) t += unit_tiles<TK>(p, u);
#pragma unroll
  for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}
// CTA that owns flat tile g when `total` tiles are cut into G slices [c*total/G, (c+1)*total/G).
__device__ __forceinline__ int cta_of_tile(long long g, long long total, int G) {
  return (int)(((g + 1) * (long long)G - 1) / total);
}

__device__ __forceinline__ void consumer_sync(int nthreads) {
  asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}

// Offsets inside the Q staging area (also reused as the fp32 combine buffer).
// q_hi: [MT*16 rows][256] bf16, 512-byte rows, 16-byte chunk index XORed with (row & 7).
__device__ __forceinline__ uint32_t q_hi_off(int row, int d) {
  const int c16 = d >> 3;
  return (uint32_t)(row * 512 + ((c16 ^ (row & 7)) << 4) + ((d & 7) << 1));
}

// Last step of a merge: the row's partial (for a KV-range split over GPUs) or its normalised, gated
// output and log-sum-exp.  lane = 8 channels.
template <typename TOut>
__device__ __forceinline__ void merge_finish(const SplitKVParams &p, const UnitInfo &ui, int row, int lane, float mg,
                                             float lg, float (&acc)[8]) {
  const int b = row / GROUP, hh = row % GROUP;
  const size_t grow = ((size_t)ui.s * p.n_new + ui.tok0 + b) * p.q_heads + (size_t)ui.kvh * GROUP + hh;
  if (p.partial_out) {
    float *dst = p.partial_out + grow * PART_STRIDE;
    *reinterpret_cast<float4 *>(dst + lane * 8) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4 *>(dst + lane * 8 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if (lane == 0) { dst[256] = mg; dst[257] = lg; }
    return;
  }
  const float inv = 1.f / lg;
  if (p.do_gate) {
    const uint4 g4 = *reinterpret_cast<const uint4 *>(p.gate + grow * HEAD_DIM + lane * 8);
    const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[2 * j] *= inv * sigmoidf_(bf16lo(gw[j]));
      acc[2 * j + 1] *= inv * sigmoidf_(bf16hi(gw[j]));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= inv;
  }
  store8<TOut>(reinterpret_cast<TOut *>(p.out) + grow * HEAD_DIM + lane * 8, acc);
  if (lane == 0 && p.lse) p.lse[grow] = (mg + log2f(lg)) * LN2;
}

// Merges the partials of one row of unit u, written by the CTAs c_first..c_last that own tiles
// of the unit, in CTA order (fixed order => bit-stable), then normalises, gates and stores.
// One warp per row, lane = 8 channels.  Used by the merge kernel and, when arrival counters are
// available, by whichever CTA finishes the unit last.
template <typename TOut, int BATCH = 4>
__device__ __forceinline__ void merge_unit_row(const SplitKVParams &p, int u, const UnitInfo &ui, int row, int c_first,
                                               int c_last, long long total, int lane, int G,
                                               const volatile uint8_t *live_of = nullptr) {
  // Partials are fetched BATCH at a time with all their loads in flight together (a unit is
  // usually cut into two to four pieces, so this is one L2 round trip; one sequence alone is cut
  // into dozens, and the merge is then a chain of round trips: hence eight at a time there) and
  // folded in with a running maximum, strictly in CTA order.
  // When there are at least as many tiles as CTAs every CTA owns tiles, so every CTA between the
  // unit's first and last has written a part: the per-CTA test (two 64-bit divisions) is skipped.
  const bool all_live = total >= (long long)G;
  float mg = -INFINITY, lg = 0.f;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int c0 = c_first; c0 <= c_last; c0 += BATCH) {
    float mv[BATCH], lv[BATCH];
    float4 av[BATCH], bv[BATCH];
    bool live[BATCH];
#pragma unroll
    for (int k = 0; k < BATCH; ++k) {
      const int c = c0 + k;
      // CTAs without tiles wrote nothing; live_of, when given, holds that test for c_first .. c_last
      // (64-bit divisions are slow enough to dominate a merge of many parts)
      live[k] = c <= c_last && (all_live || (live_of ? live_of[c - c_first] != 0 : (total * c / G != total * (c + 1) / G)));
      const float *src = p.ws + ((size_t)((live[k] ? c : c_first) + u) * (p.rb * GROUP) + row) * PART_STRIDE;
      mv[k] = __ldcg(src + 256);
      lv[k] = __ldcg(src + 257);
      av[k] = __ldcg(reinterpret_cast<const float4 *>(src + lane * 8));
      bv[k] = __ldcg(reinterpret_cast<const float4 *>(src + lane * 8 + 4));
    }
#pragma unroll
    for (int k = 0; k < BATCH; ++k) {
      if (!live[k] || !(lv[k] > 0.f)) continue;
      const float m_new = fmaxf(mg, mv[k]);
      const float f_old = fast_exp2(mg - m_new), f = fast_exp2(mv[k] - m_new);  // mg = -inf gives f_old = 0
      mg = m_new;
      lg = lg * f_old + lv[k] * f;
      acc[0] = acc[0] * f_old + av[k].x * f; acc[1] = acc[1] * f_old + av[k].y * f;
      acc[2] = acc[2] * f_old + av[k].z * f; acc[3] = acc[3] * f_old + av[k].w * f;
      acc[4] = acc[4] * f_old + bv[k].x * f; acc[5] = acc[5] * f_old + bv[k].y * f;
      acc[6] = acc[6] * f_old + bv[k].z * f; acc[7] = acc[7] * f_old + bv[k].w * f;
    }
  }
  merge_finish<TOut>(p, ui, row, lane, mg, lg, acc);
}

// The same with eight parts in flight, as a function of its own: inlined, its registers would be taken out of the
// budget of the kernel's tile loop (168 per thread with the nine-warp block), which then spills.
template <typename TOut>
__device__ __noinline__ void merge_unit_row_wide(const SplitKVParams &p, int u, const UnitInfo &ui, int row, int c_first,
                                                 int c_last, long long total, int lane, int G) {
  merge_unit_row<TOut, 8>(p, u, ui, row, c_first, c_last, total, lane, G);
}

// Barrier over the nt threads that use named barrier 1 (the consumer warps / the softmax group) that also tells
// every one of them whether all passed true.
__device__ __forceinline__ bool group_bar_and(bool v, int nt) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)v), "r"(nt)
      : "memory");
  return r != 0;
}

// Plain (untiled) bulk copy global -> shared memory, completion counted in bytes on an mbarrier.  Both addresses
// 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Whether merge_unit_bulk can take a unit of R rows cut into nparts parts: either everything fits the buffer at once
// (parts and gate rows), or at least one part fits beside the gate rows and the running state of every item.
__device__ __forceinline__ bool merge_bulk_fits(const SplitKVParams &p, int R, int nparts, uint32_t buf_bytes) {
  const uint32_t block = (uint32_t)(R * PART_STRIDE * sizeof(float));
  const uint32_t gate = (!p.partial_out && p.do_gate) ? (uint32_t)(R * HEAD_DIM * sizeof(uint16_t)) : 0u;
  return (uint32_t)nparts * block + gate <= buf_bytes || block + gate + (uint32_t)(R * 64 * 24) <= buf_bytes;
}

// Merge of one unit's partials by all nt threads of named barrier 1 (the consumer warps of the mma.sync kernel, the
// softmax group of the tcgen05 kernel) in the CTA that arrived last.
// A dependent global load costs 0.8 to 2 us at this point of the kernel (the lines were written by other SMs long
// ago and the pages are cold for this SM), and one warp per row folding part after part is a chain of them:
// about 10 us for 24 rows x 9 parts, measured, however few the parts.  Here the copy engine fetches the parts
// instead: the R rows of one part are contiguous in the workspace (R x 1040 bytes), so one bulk copy per part
// brings everything -- o, m and l -- and the unit's gate rows (per token the six heads of the group are
// contiguous) into shared memory that is idle by then (buf) in a single round trip, and the fold runs out of
// shared memory: thread = (row, 4 channels); per wave the maximum first, then a weighted sum in CTA order, so the
// loads and exponentials of different parts do not depend on one another and the result does not depend on which
// CTA merges.  A unit with more parts than the buffer holds (one sequence alone is cut into 37) takes several such
// waves, the running (acc, m, l) of every item kept in shared memory between them; the parts area is then used as
// two halves, so that the copy engine fetches the next wave while this one is folded and only the first round trip
// is exposed.  The loops are rolled on purpose: this code runs once per CTA, from a cold instruction cache.
// Every part c_first .. c_first + nparts - 1 must exist, and merge_bulk_fits() must hold.  bars: two mbarriers
// (one arrival each); phases: bit i = parity that the next wave on bars[i] completes.  Returns false when a wait
// ran out.
template <typename TOut>
__device__ __forceinline__ bool merge_unit_bulk(const SplitKVParams &p, int u, int c_first, int nparts, int t, int nt,
                                                uint8_t *buf, uint32_t buf_bytes, uint64_t *bars, uint32_t &phases) {
  const int kvh = u % p.kv_heads, sb = u / p.kv_heads, blk = sb % p.nblk, s = sb / p.nblk;
  const int tok0 = blk * p.rb, ntok = min(p.rb, p.n_new - tok0);
  const int R = ntok * GROUP, rs = p.rb * GROUP, n_items = R * 64;
  const uint32_t block_bytes = (uint32_t)(R * PART_STRIDE * sizeof(float)), bstride = block_bytes / sizeof(float);
  const uint32_t gate_bytes = (!p.partial_out && p.do_gate) ? (uint32_t)(R * HEAD_DIM * sizeof(uint16_t)) : 0u;
  const bool single = (uint32_t)nparts * block_bytes + gate_bytes <= buf_bytes;
  const uint32_t state_bytes = single ? 0u : (uint32_t)(n_items * 24);
  uint8_t *gbuf = buf + buf_bytes - gate_bytes;                               // gate rows, then the state, at the end
  float4 *st_acc = reinterpret_cast<float4 *>(gbuf - state_bytes);            // [n_items]
  float2 *st_ml = reinterpret_cast<float2 *>(gbuf - state_bytes + n_items * 16);  // [n_items]
  // parts per wave: all of them, or what half of the parts area holds (one at least: the halves then overlap
  // and the waves simply follow one another)
  const uint32_t area = buf_bytes - gate_bytes - state_bytes;
  const int half_cap = (int)(area / 2 / block_bytes);
  const int per_wave = single ? nparts : max(half_cap, 1);
  const uint32_t half_off = half_cap >= 1 ? (uint32_t)half_cap * block_bytes : 0u;
  const float *base = p.ws + (size_t)(c_first + u) * rs * PART_STRIDE;  // part k: base + k * rs * PART_STRIDE
  auto issue = [&](int w) {  // thread 0: the copies of wave w, into half w & 1, counted on bars[w & 1]
    const int k0 = w * per_wave, n = min(per_wave, nparts - k0);
    uint64_t *bar = bars + (w & 1);
    uint8_t *dst = buf + (w & 1) * half_off;
    mbar_expect_tx(bar, (uint32_t)n * block_bytes + (w == 0 ? gate_bytes : 0u));
    for (int k = 0; k < n; ++k)
      bulk_load(dst + (size_t)k * block_bytes, base + (size_t)(k0 + k) * rs * PART_STRIDE, block_bytes, bar);
    for (int b = 0; b < ntok && w == 0 && gate_bytes; ++b)
      bulk_load(gbuf + (size_t)b * GROUP * HEAD_DIM * sizeof(uint16_t),
                p.gate + (((size_t)s * p.n_new + tok0 + b) * p.q_heads + (size_t)kvh * GROUP) * HEAD_DIM,
                (uint32_t)(GROUP * HEAD_DIM * sizeof(uint16_t)), bar);
  };
  const int n_waves = (nparts + per_wave - 1) / per_wave;
  const bool overlap = half_cap >= 1;  // the next wave may be fetched while this one is folded
  bool ok = true;
  if (t == 0) issue(0);
  for (int w = 0; w < n_waves && ok; ++w) {
    const int k0 = w * per_wave, n = min(per_wave, nparts - k0);
    const bool first = w == 0, last = w == n_waves - 1;
    if (t == 0 && overlap && !last) issue(w + 1);
    ok = mbar_wait(bars + (w & 1), (phases >> (w & 1)) & 1u);
    phases ^= 1u << (w & 1);
    if (ok) {
#pragma unroll 1
      for (int item = t; item < n_items; item += nt) {
        const int r = item >> 6, c4 = item & 63;
        const float *rowp = reinterpret_cast<const float *>(buf + (w & 1) * half_off) + r * PART_STRIDE;
        float m_prev = -INFINITY, l_run = 0.f;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        if (!first) {
          a = st_acc[item];
          const float2 ml = st_ml[item];
          m_prev = ml.x;
          l_run = ml.y;
        }
        float m_run = m_prev;
#pragma unroll 4
        for (int k = 0; k < n; ++k) {
          const float m = rowp[k * bstride + 256], l = rowp[k * bstride + 257];
          m_run = fmaxf(m_run, l > 0.f ? m : -INFINITY);
        }
        const float sp = (m_prev == -INFINITY) ? 0.f : fast_exp2(m_prev - m_run);
        l_run *= sp;
        a.x *= sp; a.y *= sp; a.z *= sp; a.w *= sp;
#pragma unroll 4
        for (int k = 0; k < n; ++k) {
          const float m = rowp[k * bstride + 256], l = rowp[k * bstride + 257];
          const float4 v = *reinterpret_cast<const float4 *>(rowp + k * bstride + c4 * 4);
          const float f = l > 0.f ? fast_exp2(m - m_run) : 0.f;
          l_run = fmaf(l, f, l_run);
          a.x = fmaf(v.x, f, a.x); a.y = fmaf(v.y, f, a.y); a.z = fmaf(v.z, f, a.z); a.w = fmaf(v.w, f, a.w);
        }
        if (!last) {
          st_acc[item] = a;
          st_ml[item] = make_float2(m_run, l_run);
          continue;
        }
        const size_t gr = ((size_t)s * p.n_new + tok0 + r / GROUP) * p.q_heads + (size_t)kvh * GROUP + r % GROUP;
        if (p.partial_out) {
          float *dst = p.partial_out + gr * PART_STRIDE;
          *reinterpret_cast<float4 *>(dst + c4 * 4) = a;
          if (c4 == 0) { dst[256] = m_run; dst[257] = l_run; }
          continue;
        }
        const float inv = __fdividef(1.f, l_run);  // 8 or 16 warps issue this epilogue: the short forms
        a.x *= inv; a.y *= inv; a.z *= inv; a.w *= inv;
        if (p.do_gate) {
          const uint2 g = *reinterpret_cast<const uint2 *>(gbuf + (size_t)r * HEAD_DIM * sizeof(uint16_t) + c4 * 8);
          a.x *= sigmoid_fast(bf16lo(g.x)); a.y *= sigmoid_fast(bf16hi(g.x));
          a.z *= sigmoid_fast(bf16lo(g.y)); a.w *= sigmoid_fast(bf16hi(g.y));
        }
        if constexpr (sizeof(TOut) == 4) {
          *reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + gr * HEAD_DIM + c4 * 4) = a;
        } else {
          *reinterpret_cast<uint2 *>(reinterpret_cast<uint16_t *>(p.out) + gr * HEAD_DIM + c4 * 4) =
              make_uint2(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w));
        }
        if (c4 == 0 && p.lse) p.lse[gr] = (m_run + log2f(l_run)) * LN2;
      }
    }
    ok = group_bar_and(ok, nt);  // this half is written again by the wave after the next, or by the next merge
    if (t == 0 && ok && !overlap && !last) issue(w + 1);
  }
  return ok;
}

// Merge of a unit cut into at most four parts, straight from the workspace: thread = (row, 8 channels), every load
// of every part in flight together -- one round trip and no set-up, where the bulk-copy merge pays for its barrier and
// its longer code (3.1 us for the two parts of a decode unit, cold).  The arithmetic is the bulk merge's, operation
// for operation, in part order: the same bits, whichever of the two is used and whichever CTA merges.
template <typename TOut>
__device__ __forceinline__ void merge_unit_direct(const SplitKVParams &p, int u, int c_first, int nparts, int t, int nt) {
  const int kvh = u % p.kv_heads, sb = u / p.kv_heads, blk = sb % p.nblk, s = sb / p.nblk;
  const int tok0 = blk * p.rb, ntok = min(p.rb, p.n_new - tok0);
  const int R = ntok * GROUP, rs = p.rb * GROUP;
  const float *base = p.ws + (size_t)(c_first + u) * rs * PART_STRIDE;
  for (int idx = t; idx < R * 32; idx += nt) {
    const int row = idx >> 5, c8 = idx & 31;
    float m[4], l[4];
    float4 va[4], vb[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      m[k] = -INFINITY;
      l[k] = 0.f;
      va[k] = vb[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k < nparts) {
        const float *src = base + ((size_t)k * rs + row) * PART_STRIDE;
        m[k] = __ldcg(src + 256);
        l[k] = __ldcg(src + 257);
        va[k] = __ldcg(reinterpret_cast<const float4 *>(src + c8 * 8));
        vb[k] = __ldcg(reinterpret_cast<const float4 *>(src + c8 * 8 + 4));
      }
    }
    const size_t gr = ((size_t)s * p.n_new + tok0 + row / GROUP) * p.q_heads + (size_t)kvh * GROUP + row % GROUP;
    uint4 g4 = make_uint4(0, 0, 0, 0);
    if (!p.partial_out && p.do_gate) g4 = *reinterpret_cast<const uint4 *>(p.gate + gr * HEAD_DIM + c8 * 8);
    float m_run = -INFINITY;
#pragma unroll
    for (int k = 0; k < 4; ++k) m_run = fmaxf(m_run, l[k] > 0.f ? m[k] : -INFINITY);
    float l_run = 0.f;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (k >= nparts) continue;
      const float f = l[k] > 0.f ? fast_exp2(m[k] - m_run) : 0.f;
      l_run = fmaf(l[k], f, l_run);
      v[0] = fmaf(va[k].x, f, v[0]); v[1] = fmaf(va[k].y, f, v[1]); v[2] = fmaf(va[k].z, f, v[2]); v[3] = fmaf(va[k].w, f, v[3]);
      v[4] = fmaf(vb[k].x, f, v[4]); v[5] = fmaf(vb[k].y, f, v[5]); v[6] = fmaf(vb[k].z, f, v[6]); v[7] = fmaf(vb[k].w, f, v[7]);
    }
    if (p.partial_out) {
      float *dst = p.partial_out + gr * PART_STRIDE;
      *reinterpret_cast<float4 *>(dst + c8 * 8) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4 *>(dst + c8 * 8 + 4) = make_float4(v[4], v[5], v[6], v[7]);
      if (c8 == 0) { dst[256] = m_run; dst[257] = l_run; }
      continue;
    }
    const float inv = __fdividef(1.f, l_run);
    const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[j] *= inv;
      if (p.do_gate) v[j] *= sigmoid_fast((j & 1) ? bf16hi(gw[j >> 1]) : bf16lo(gw[j >> 1]));
    }
    store8<TOut>(reinterpret_cast<TOut *>(p.out) + gr * HEAD_DIM + c8 * 8, v);
    if (c8 == 0 && p.lse) p.lse[gr] = (m_run + log2f(l_run)) * LN2;
  }
}

// Merge of one unit by ALL the CTAs that hold a part of it, each taking a slice of the (row, 4-channel) items: for
// a unit cut into dozens of parts (one sequence alone on the whole device: 37) a single merging CTA has to pull every
// part -- 231 KB -- through one SM, which costs more than the streaming of the sequence's KV; sliced, a CTA reads
// 1/nparts of every part.  The caller has waited until every part has arrived.  A group of 8, 16 or 32 lanes (the
// power of two that holds the parts; beyond 32 a lane takes up to five) serves one item, a warp 4, 2 or 1 items at a
// time and several such rounds per iteration: all loads of an iteration are in flight together, then the row maximum,
// the weights and the weighted sums are reduced across the group's lanes in a fixed tree, so the result does not
// depend on timing.  j: this CTA's index among the unit's nparts CTAs (nparts <= 160).
// LG: lanes per item (a power of two that holds the parts, or 32); PL: parts per lane; UN: rounds per iteration
// (their loads are all in flight together).
template <typename TOut, int LG, int PL, int UN>
__device__ __forceinline__ void merge_unit_sliced_t(const SplitKVParams &p, int u, int c_first, int nparts, int j, int warp,
                                                    int lane, int nwarps) {
  const int kvh = u % p.kv_heads, sb = u / p.kv_heads, blk = sb % p.nblk, s = sb / p.nblk;
  const int tok0 = blk * p.rb, ntok = min(p.rb, p.n_new - tok0);
  const int R = ntok * GROUP, rs = p.rb * GROUP, n_items = R * 64;
  const int lo = (int)((long long)n_items * j / nparts), hi = (int)((long long)n_items * (j + 1) / nparts);
  const float *base = p.ws + (size_t)(c_first + u) * rs * PART_STRIDE;  // part k, row r: base + (k * rs + r) * PART_STRIDE
  constexpr int g = LG, per_round = 32 / LG;
  const int sub = lane / g, pl = lane % g;
  for (int it0 = lo + warp * UN * per_round; it0 < hi; it0 += nwarps * UN * per_round) {
    float m[UN][PL], l[UN][PL];
    float4 v[UN][PL];
    uint2 g2[UN];
#pragma unroll
    for (int e = 0; e < UN; ++e) {
      const int item = it0 + e * per_round + sub, r = item >> 6, c4 = item & 63;
      g2[e] = make_uint2(0, 0);
#pragma unroll
      for (int q2 = 0; q2 < PL; ++q2) {
        const int k = pl + g * q2;
        m[e][q2] = -INFINITY;
        l[e][q2] = 0.f;
        v[e][q2] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (item < hi && k < nparts && (q2 == 0 || g == 32)) {
          const float *src = base + ((size_t)k * rs + r) * PART_STRIDE;
          m[e][q2] = __ldcg(src + 256);
          l[e][q2] = __ldcg(src + 257);
          v[e][q2] = __ldcg(reinterpret_cast<const float4 *>(src + c4 * 4));
        }
      }
      if (item < hi && pl == 0 && !p.partial_out && p.do_gate) {
        const size_t gr = ((size_t)s * p.n_new + tok0 + r / GROUP) * p.q_heads + (size_t)kvh * GROUP + r % GROUP;
        g2[e] = *reinterpret_cast<const uint2 *>(p.gate + gr * HEAD_DIM + c4 * 4);
      }
    }
#pragma unroll
    for (int e = 0; e < UN; ++e) {
      const int item = it0 + e * per_round + sub, r = item >> 6, c4 = item & 63;
      // every lane takes part in the shuffles, whether its group's item exists or not
      float m_run = -INFINITY;
#pragma unroll
      for (int q2 = 0; q2 < PL; ++q2) m_run = fmaxf(m_run, l[e][q2] > 0.f ? m[e][q2] : -INFINITY);
#pragma unroll
      for (int o = g >> 1; o; o >>= 1) m_run = fmaxf(m_run, __shfl_xor_sync(0xffffffffu, m_run, o));
      float l_run = 0.f;
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int q2 = 0; q2 < PL; ++q2) {
        const float f = l[e][q2] > 0.f ? fast_exp2(m[e][q2] - m_run) : 0.f;
        l_run = fmaf(l[e][q2], f, l_run);
        a.x = fmaf(v[e][q2].x, f, a.x); a.y = fmaf(v[e][q2].y, f, a.y);
        a.z = fmaf(v[e][q2].z, f, a.z); a.w = fmaf(v[e][q2].w, f, a.w);
      }
#pragma unroll
      for (int o = g >> 1; o; o >>= 1) {
        l_run += __shfl_xor_sync(0xffffffffu, l_run, o);
        a.x += __shfl_xor_sync(0xffffffffu, a.x, o); a.y += __shfl_xor_sync(0xffffffffu, a.y, o);
        a.z += __shfl_xor_sync(0xffffffffu, a.z, o); a.w += __shfl_xor_sync(0xffffffffu, a.w, o);
      }
      if (item >= hi || pl != 0) continue;  // (no shuffle follows in this round)
      const size_t gr = ((size_t)s * p.n_new + tok0 + r / GROUP) * p.q_heads + (size_t)kvh * GROUP + r % GROUP;
      if (p.partial_out) {
        float *dst = p.partial_out + gr * PART_STRIDE;
        *reinterpret_cast<float4 *>(dst + c4 * 4) = a;
        if (c4 == 0) { dst[256] = m_run; dst[257] = l_run; }
        continue;
      }
      const float inv = __fdividef(1.f, l_run);
      a.x *= inv; a.y *= inv; a.z *= inv; a.w *= inv;
      if (p.do_gate) {
        a.x *= sigmoid_fast(bf16lo(g2[e].x)); a.y *= sigmoid_fast(bf16hi(g2[e].x));
        a.z *= sigmoid_fast(bf16lo(g2[e].y)); a.w *= sigmoid_fast(bf16hi(g2[e].y));
      }
      if constexpr (sizeof(TOut) == 4) {
        *reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + gr * HEAD_DIM + c4 * 4) = a;
      } else {
        *reinterpret_cast<uint2 *>(reinterpret_cast<uint16_t *>(p.out) + gr * HEAD_DIM + c4 * 4) =
            make_uint2(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w));
      }
      if (c4 == 0 && p.lse) p.lse[gr] = (m_run + log2f(l_run)) * LN2;
    }
  }
}
template <typename TOut>
__device__ __forceinline__ void merge_unit_sliced(const SplitKVParams &p, int u, int c_first, int nparts, int j, int warp,
                                                  int lane, int nwarps) {
  if (nparts > 16) merge_unit_sliced_t<TOut, 32, 5, 2>(p, u, c_first, nparts, j, warp, lane, nwarps);
  else if (nparts > 8) merge_unit_sliced_t<TOut, 16, 1, 2>(p, u, c_first, nparts, j, warp, lane, nwarps);
  else merge_unit_sliced_t<TOut, 8, 1, 2>(p, u, c_first, nparts, j, warp, lane, nwarps);
}

// FOLD = false: a dedicated producer warp (warp NCW).  FOLD = true: lane 0 of consumer warp 0 also
// issues the TMA loads, STAGES - 1 tiles ahead of the tile it is about to consume; the block is then
// exactly 8 warps and every thread may use up to 255 registers (with a ninth warp the register file
// is carved as if for twelve, which caps a thread at 168 and makes the two-row-tile variant spill).
// SLICED: units cut across CTAs are merged by all of their CTAs together, each a slice of the channels (see
// merge_unit_sliced), instead of by the CTA that arrives last.  Every CTA then waits (bounded) for the unit's arrival
// counter to reach the number of parts, which needs all CTAs of the grid resident at once -- one per SM, as the grid
// is sized -- so the host selects this variant only where it pays: few long units, each cut into eight parts or more.
template <int MT, int DS, int STAGES, int LOK, bool FOLD, typename TIn, typename TOut, bool SLICED = false>
__global__ void __launch_bounds__((SK_KS * DS + (FOLD ? 0 : 1)) * 32, 1)
splitkv_kernel(const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
               const __grid_constant__ SplitKVParams p) {
  constexpr int NCW = SK_KS * DS;          // consumer warps
  constexpr int NCT = NCW * 32;            // consumer threads
  constexpr int ROWS = MT * 16;            // padded rows
  constexpr int DW = HEAD_DIM / DS;        // output channels per warp
  constexpr int NT_O = DW / 8;             // 8-wide output n-tiles per warp
  constexpr int QREGION = ROWS * 1024;     // q_hi + q_lo (bf16) or combine buffer (fp32)
  // With one 16-row tile and the 8-warp block there are registers to spare: the Q fragments of all
  // k-steps then live in registers for the whole segment instead of being re-read per KV tile.
  constexpr bool QREG = FOLD && MT == 1 && LOK <= 4;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *stage_base = smem;
  uint8_t *qregion = smem + STAGES * SK_STAGE_BYTES;
  float *mx = reinterpret_cast<float *>(qregion + QREGION);  // [SK_KS][ROWS]
  float *lx = mx + SK_KS * ROWS;                             // [SK_KS][ROWS]
  uint64_t *full = reinterpret_cast<uint64_t *>(lx + SK_KS * ROWS);
  uint64_t *empty = full + STAGES;
  long long *seg = reinterpret_cast<long long *>(empty + STAGES);  // [0]=total [1]=pre(u_first) [2]=u_first
  volatile int *ticket = reinterpret_cast<volatile int *>(seg + 3);
  uint64_t *merge_bar = reinterpret_cast<uint64_t *>(seg + 4);  // two: bulk copies of a merge's parts land on them
  // MT == 1: 16 KB more, so that the four key slices of a unit of at most eight rows have a buffer each in any segment
  float *comb_extra = reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(seg) + 120 + 15) & ~uintptr_t(15));
  volatile int *pend = reinterpret_cast<volatile int *>(seg + 6);  // units this CTA is to merge: 5 ints each, [10] their count, [11] scratch

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_units = p.n_seq * p.nblk * p.kv_heads;
  const int cta = blockIdx.x;
  // a kernel launched behind this one as a programmatic dependent (this library's append kernel is) may become
  // resident now; it waits for this grid's completion before it touches memory
  grid_dep_launch_dependents();

  if (tid == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], NCW); }
    mbar_init(merge_bar, 1);
    mbar_init(merge_bar + 1, 1);
    pend[10] = 0;
    fence_barrier_init();
    prefetch_tensormap(&mapK);
    prefetch_tensormap(&mapV);
  }
  if (warp == 0) {
    long long total; int live, geff; bool aligned;
    warp_partition(p, n_units, lane, total, live, geff, aligned);
    int u0 = n_units; long long pre0 = 0;
    if (cta < geff) warp_find_unit(p, n_units, lane, total * cta / geff, u0, pre0);
    if (lane == 0) { seg[0] = total; seg[1] = pre0; seg[2] = (long long)u0 | ((long long)geff << 32); }
  }
  __syncthreads();
  const long long total = seg[0];
  const int G = (int)(seg[2] >> 32);                  // CTAs in use (the rest of the grid leaves here)
  const long long g0 = cta < G ? total * cta / G : 0, g1 = cta < G ? total * (cta + 1) / G : 0;
  if (g0 >= g1) return;  // uniform for the whole CTA

  // ---------------- producer: one lane streams the tiles of every segment, in order -----------
  int pu = (int)(seg[2] & 0xffffffffll);                              // unit of the next tile to load
  long long ppre = seg[1];                           // flat index of that unit's tile 0
  int pt = (int)(max(g0, ppre) - ppre);              // next tile within the unit
  uint32_t pit = 0;                                  // tiles issued so far
  bool pok = true, dep_waited = false;
  int cached_u = -1;                                 // unit whose description and base row are held below:
  UnitInfo cached_ui;                                // loads issued while the SM streams K/V are slow, so the
  long long cached_base = 0;                         // producer reads them once per unit, not once per tile
  auto produce_one = [&]() -> bool {
    while (ppre < g1 && pu < n_units) {
      if (pu != cached_u) {
        cached_ui = unit_info(p, pu);
        cached_base = p.cache_row ? p.cache_row[cached_ui.s] : 0;
        cached_u = pu;
      }
      const UnitInfo &ui = cached_ui;
      const int nt = (ui.len + SK_TK - 1) / SK_TK;
      const int t1 = (int)(min(g1, ppre + nt) - ppre);
      if (pt < t1) {
        const int st = pit % STAGES;
        if (pit >= STAGES && !mbar_wait(&empty[st], ((pit / STAGES) - 1) & 1)) {
          if (p.status) *p.status = DEV_ERR_EMPTY_WAIT;
          pok = false;
          return false;
        }
        // the first tile that holds rows written by the append kernel of this step: wait for that kernel
        if (!dep_waited && (pt + 1) * SK_TK > ui.pos) {
          grid_dep_wait();
          dep_waited = true;
        }
        uint8_t *kd = stage_base + st * SK_STAGE_BYTES, *vd = kd + SK_TILE_BYTES;
        mbar_expect_tx(&full[st], SK_STAGE_BYTES);
        const int r = (int)cache_row_at(p.pages, cached_base, ui.s, pt * SK_TK);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          tma_load_2d(kd + c * (SK_TK * 128), &mapK, &full[st], ui.kvh * HEAD_DIM + c * 64, r);
          tma_load_2d(vd + c * (SK_TK * 128), &mapV, &full[st], ui.kvh * HEAD_DIM + c * 64, r);
        }
        ++pt;
        ++pit;
        return true;
      }
      ppre += nt;
      ++pu;
      pt = 0;
    }
    return false;
  };
  if (!FOLD && warp == NCW) {
    if (lane == 0)
      while (produce_one()) { }
    return;
  }
  // folded producer: keep the ring full up to STAGES - 1 tiles past the one about to be consumed
  auto produce_ahead = [&](uint32_t consume_it) {
    if (FOLD && warp == 0) {
      if (lane == 0)
        while (pok && pit < consume_it + STAGES && produce_one()) { }
      __syncwarp();
    }
  };
  produce_ahead(0);

  // ---------------------------- consumers ---------------------------------------------------
  const int ks = warp % SK_KS, ds = warp / SK_KS;
  const int qd = lane >> 2, ql = lane & 3;  // row-in-8 and column pair of the mma fragments
  bool ok = true;
  uint32_t it = 0;
  int u = (int)(seg[2] & 0xffffffffll);
  long long pre = seg[1];
  const uint32_t qhi_s = smem_u32(qregion);
  // Per-lane ldmatrix addresses.  The swizzle XORs the 16-byte column (d / 8) & 7 with row & 7,
  // so for a fixed lane only four distinct column offsets occur; the rest is a constant stride.
  uint32_t klane[4], vlane[4], qlane[MT][4];
  {
    const int krow = ks * 16 + (lane & 7) + ((lane >> 4) << 3);  // K: matrices (keys lo/hi) x (d lo/hi)
    const int kc_sel = (lane >> 3) & 1;
    const int vrow = ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);  // V (transposed load)
    const int vc_sel = lane >> 4;
    const int arow = (lane & 7) + (((lane >> 3) & 1) << 3);  // Q: A-fragment row within 16
    const int ac_sel = lane >> 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      klane[j] = krow * 128 + (((j * 2 + kc_sel) ^ (krow & 7)) << 4);
      vlane[j] = (ds * DW / 64) * (SK_TK * 128) + vrow * 128 + (((j * 2 + vc_sel) ^ (vrow & 7)) << 4);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
        qlane[mt][j] = qhi_s + (mt * 16 + arow) * 512 + (((j * 2 + ac_sel) ^ (arow & 7)) << 4);
    }
  }

  while (pre < g1 && u < n_units) {
    const UnitInfo ui = unit_info(p, u);
    const int nt_unit = (ui.len + SK_TK - 1) / SK_TK;
    const int t0 = (int)(max(g0, pre) - pre), t1 = (int)(min(g1, pre + nt_unit) - pre);
    const int R = ui.ntok * GROUP;
    const bool whole = (t0 == 0 && t1 == nt_unit);

    // ---- stage Q: rotate, split into bf16 hi (+ lo), zero the padding rows ----
    if (p.q_dep) grid_dep_wait();  // q comes out of the launch before this one
    consumer_sync(NCT);  // the previous segment is done with this region
    // All global loads of the staging are issued before the first one is used: one memory round trip
    // for the segment instead of one per loop iteration.
    constexpr int QIT = (ROWS * 32 + NCT - 1) / NCT;
    float xq[QIT][8], rx[QIT], ry[QIT];
#pragma unroll
    for (int qi = 0; qi < QIT; ++qi) {
      const int idx = tid + qi * NCT;
      const int row = idx >> 5, c16 = idx & 31;  // 8 channels d = c16*8 .. +7
#pragma unroll
      for (int j = 0; j < 8; ++j) xq[qi][j] = 0.f;
      if (idx < ROWS * 32 && row < R && !(p.do_rope && c16 < 8)) {
        const int b = row / GROUP, hh = row % GROUP;
        const size_t grow = ((size_t)ui.s * p.n_new + ui.tok0 + b) * p.q_heads + (size_t)ui.kvh * GROUP + hh;
        load8<TIn>(reinterpret_cast<const TIn *>(p.q) + grow * HEAD_DIM + c16 * 8, xq[qi]);
      }
      rx[qi] = ry[qi] = 0.f;
      if (p.do_rope && idx < ROWS * ROT_PAIRS) {
        const int rrow = idx / ROT_PAIRS, i = idx % ROT_PAIRS;  // pair (i, i + 32) of this row
        if (rrow < R) {
          const size_t grow = ((size_t)ui.s * p.n_new + ui.tok0 + rrow / GROUP) * p.q_heads + (size_t)ui.kvh * GROUP + rrow % GROUP;
          const TIn *src = reinterpret_cast<const TIn *>(p.q) + grow * HEAD_DIM;
          rx[qi] = load_as_f32<TIn>(src + i);
          ry[qi] = load_as_f32<TIn>(src + i + ROT_PAIRS);
        }
      }
    }
#pragma unroll
    for (int qi = 0; qi < QIT; ++qi) {
      const int idx = tid + qi * NCT;
      const int row = idx >> 5, c16 = idx & 31;
      if (idx >= ROWS * 32 || (p.do_rope && c16 < 8)) continue;  // rotary channels are written pair-wise below
      uint32_t hi[4], lo[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        hi[j] = pack_bf16(xq[qi][2 * j], xq[qi][2 * j + 1]);
        lo[j] = pack_bf16(xq[qi][2 * j] - bf16lo(hi[j]), xq[qi][2 * j + 1] - bf16hi(hi[j]));
      }
      *reinterpret_cast<uint4 *>(qregion + q_hi_off(row, c16 * 8)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      if (c16 * 8 < p.q_lo_dims)
        *reinterpret_cast<uint4 *>(qregion + ROWS * 512 + q_hi_off(row, c16 * 8)) =
            make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
    if (p.do_rope) {
#pragma unroll
      for (int qi = 0; qi < QIT; ++qi) {
        const int idx = tid + qi * NCT;
        if (idx >= ROWS * ROT_PAIRS) continue;
        const int row = idx / ROT_PAIRS, i = idx % ROT_PAIRS;
        float xr = 0.f, yr = 0.f;
        if (row < R) {
          const size_t trow = (size_t)ui.s * p.n_new + ui.tok0 + row / GROUP;
          const int pz = p.mpos ? p.mpos[trow * 3 + mrope_component(i)] : ui.rpos + ui.tok0 + row / GROUP;
          float c, sn;
          rope_sincos_reduced(pz, p.rope.inv_freq[i], c, sn);  // angle reduced in double, then the fast sincos
          xr = rx[qi] * c - ry[qi] * sn;
          yr = rx[qi] * sn + ry[qi] * c;
        }
        const uint16_t xh = f32_to_bf16_bits(xr), yh = f32_to_bf16_bits(yr);
        *reinterpret_cast<uint16_t *>(qregion + q_hi_off(row, i)) = xh;
        *reinterpret_cast<uint16_t *>(qregion + q_hi_off(row, i + ROT_PAIRS)) = yh;
        if (p.q_lo_dims) {
          *reinterpret_cast<uint16_t *>(qregion + ROWS * 512 + q_hi_off(row, i)) =
              f32_to_bf16_bits(xr - bf16_bits_to_f32(xh));
          *reinterpret_cast<uint16_t *>(qregion + ROWS * 512 + q_hi_off(row, i + ROT_PAIRS)) =
              f32_to_bf16_bits(yr - bf16_bits_to_f32(yh));
        }
      }
    }
    consumer_sync(NCT);
    uint32_t qf[QREG ? 16 : 1][4], qlf[QREG && LOK > 0 ? LOK : 1][4];
    if (QREG) {
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) ldsm_x4(qlane[0][kk & 3] + (kk >> 2) * 128, qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
#pragma unroll
      for (int kk = 0; kk < LOK; ++kk)
        ldsm_x4(qlane[0][kk & 3] + (kk >> 2) * 128 + ROWS * 512, qlf[kk][0], qlf[kk][1], qlf[kk][2], qlf[kk][3]);
    }

    // ---- per-row state ----
    float o[MT][NT_O][4];
    float m_run[MT][2], l_run[MT][2];
    int lim[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        m_run[mt][h2] = -INFINITY;
        l_run[mt][h2] = 0.f;
        const int row = mt * 16 + h2 * 8 + qd;
        const int b = min(row / GROUP, ui.ntok - 1);
        lim[mt][h2] = p.no_causal ? ui.pos : ui.pos + ui.tok0 + b + 1;  // keys visible to this row
      }
#pragma unroll
      for (int n = 0; n < NT_O; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[mt][n][j] = 0.f;
    }
    const int lim_min = p.no_causal ? ui.pos : ui.pos + ui.tok0 + 1;

    for (int t = t0; t < t1; ++t, ++it) {
      const int st = it % STAGES;
      produce_ahead(it);
      if (ok) {
        // every lane polls; the verdict is made warp-uniform before any warp-wide operation
        const bool got = mbar_wait(&full[st], (it / STAGES) & 1);
        if (!__all_sync(0xffffffffu, got)) {
          ok = false;
          if (lane == 0 && p.status) *p.status = DEV_ERR_FULL_WAIT;
        }
      }
      if (ok) {
        const uint32_t kbase = smem_u32(stage_base + st * SK_STAGE_BYTES);
        const uint32_t vbase = kbase + SK_TILE_BYTES;
        const int key0 = t * SK_TK + ks * 16;  // first key of this warp's slice

        // S = Q K^T on the 16-key slice, two accumulator sets to shorten the dependency chain
        float s[MT][2][4], s2[MT][2][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int j = 0; j < 4; ++j) { s[mt][n][j] = 0.f; s2[mt][n][j] = 0.f; }

        uint32_t kb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) kb[j] = kbase + klane[j];
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4(kb[kk & 3] + (kk >> 2) * (SK_TK * 128), b0, b1, b2, b3);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            uint32_t a0, a1, a2, a3;
            if (QREG) { a0 = qf[kk][0]; a1 = qf[kk][1]; a2 = qf[kk][2]; a3 = qf[kk][3]; }
            else ldsm_x4(qlane[mt][kk & 3] + (kk >> 2) * 128, a0, a1, a2, a3);
            if (kk & 1) {
              mma_bf16_16816(s2[mt][0], a0, a1, a2, a3, b0, b1);
              mma_bf16_16816(s2[mt][1], a0, a1, a2, a3, b2, b3);
            } else {
              mma_bf16_16816(s[mt][0], a0, a1, a2, a3, b0, b1);
              mma_bf16_16816(s[mt][1], a0, a1, a2, a3, b2, b3);
            }
            if (kk < LOK) {  // the bf16 "lo" part of Q against the same K fragment
              if (QREG) { a0 = qlf[kk][0]; a1 = qlf[kk][1]; a2 = qlf[kk][2]; a3 = qlf[kk][3]; }
              else ldsm_x4(qlane[mt][kk & 3] + (kk >> 2) * 128 + ROWS * 512, a0, a1, a2, a3);
              if (kk & 1) {
                mma_bf16_16816(s[mt][0], a0, a1, a2, a3, b0, b1);
                mma_bf16_16816(s[mt][1], a0, a1, a2, a3, b2, b3);
              } else {
                mma_bf16_16816(s2[mt][0], a0, a1, a2, a3, b0, b1);
                mma_bf16_16816(s2[mt][1], a0, a1, a2, a3, b2, b3);
              }
            }
          }
        }

        const bool need_mask = (t * SK_TK + SK_TK > lim_min);
        // A partially valid last tile: rows of V past the unit's length may hold anything
        // (even NaN patterns), and 0 * NaN would poison the accumulators -- zero them.
        if (t == nt_unit - 1 && key0 + 16 > ui.len) {
          const int valid = max(0, ui.len - key0);
          for (int idx = lane; idx < 16 * (DW / 8); idx += 32) {
            const int kr = idx / (DW / 8), c = idx % (DW / 8);
            if (kr >= valid)
              *reinterpret_cast<uint4 *>(stage_base + st * SK_STAGE_BYTES + SK_TILE_BYTES +
                                         kv_tile_off<SK_TK>(ks * 16 + kr, ds * DW + c * 8)) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async();
          __syncwarp();
        }

        uint32_t phi[MT][4], plo[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {
            float v[4];
            v[0] = s[mt][0][2 * h2] + s2[mt][0][2 * h2];
            v[1] = s[mt][0][2 * h2 + 1] + s2[mt][0][2 * h2 + 1];
            v[2] = s[mt][1][2 * h2] + s2[mt][1][2 * h2];
            v[3] = s[mt][1][2 * h2 + 1] + s2[mt][1][2 * h2 + 1];
            if (need_mask) {
              const int kcol = key0 + ql * 2;
              if (kcol >= lim[mt][h2]) v[0] = -INFINITY;
              if (kcol + 1 >= lim[mt][h2]) v[1] = -INFINITY;
              if (kcol + 8 >= lim[mt][h2]) v[2] = -INFINITY;
              if (kcol + 9 >= lim[mt][h2]) v[3] = -INFINITY;
            }
            float mxv = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
            mxv = fmaxf(mxv, __shfl_xor_sync(0xffffffffu, mxv, 1));
            mxv = fmaxf(mxv, __shfl_xor_sync(0xffffffffu, mxv, 2));
            const float m_new = fmaxf(m_run[mt][h2], mxv * p.scale_log2);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = fast_exp2(m_run[mt][h2] - m_use);
            m_run[mt][h2] = m_new;
            float pv[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) pv[j] = fast_exp2(fmaf(v[j], p.scale_log2, -m_use));
            l_run[mt][h2] = l_run[mt][h2] * alpha + ((pv[0] + pv[1]) + (pv[2] + pv[3]));
            if (alpha != 1.f) {
#pragma unroll
              for (int n = 0; n < NT_O; ++n) { o[mt][n][2 * h2] *= alpha; o[mt][n][2 * h2 + 1] *= alpha; }
            }
            // A fragment of P: a0/a2 = rows qd (h2 = 0), a1/a3 = rows qd + 8 (h2 = 1)
            const uint32_t h01 = pack_bf16(pv[0], pv[1]), h23 = pack_bf16(pv[2], pv[3]);
            phi[mt][h2] = h01;
            phi[mt][2 + h2] = h23;
            plo[mt][h2] = pack_bf16(pv[0] - bf16lo(h01), pv[1] - bf16hi(h01));
            plo[mt][2 + h2] = pack_bf16(pv[2] - bf16lo(h23), pv[3] - bf16hi(h23));
          }
        }

        // O += P V on this warp's 16 keys and DW output channels
        uint32_t vb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) vb[j] = vbase + vlane[j];
#pragma unroll
        for (int n2 = 0; n2 < NT_O / 2; ++n2) {
          uint32_t v0, v1, v2, v3;
          ldsm_x4_trans(vb[n2 & 3] + (n2 >> 2) * (SK_TK * 128), v0, v1, v2, v3);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_bf16_16816(o[mt][2 * n2], phi[mt][0], phi[mt][1], phi[mt][2], phi[mt][3], v0, v1);
            mma_bf16_16816(o[mt][2 * n2 + 1], phi[mt][0], phi[mt][1], phi[mt][2], phi[mt][3], v2, v3);
            mma_bf16_16816(o[mt][2 * n2], plo[mt][0], plo[mt][1], plo[mt][2], plo[mt][3], v0, v1);
            mma_bf16_16816(o[mt][2 * n2 + 1], plo[mt][0], plo[mt][1], plo[mt][2], plo[mt][3], v2, v3);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);
    }

    // ---- merge the SK_KS key-slice warps of each channel group, in slice order ----
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        float l = l_run[mt][h2];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        l_run[mt][h2] = l;
        if (ds == 0 && ql == 0) {
          mx[ks * ROWS + mt * 16 + h2 * 8 + qd] = m_run[mt][h2];
          lx[ks * ROWS + mt * 16 + h2 * 8 + qd] = l;
        }
      }
    consumer_sync(NCT);  // also: every warp is past its last tile, the Q area may be reused
    float *comb = reinterpret_cast<float *>(qregion);  // [ROWS][256] fp32, 8-float groups XOR (row & 7)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const int row = mt * 16 + h2 * 8 + qd;
        float mg = -INFINITY;
#pragma unroll
        for (int k = 0; k < SK_KS; ++k) mg = fmaxf(mg, mx[k * ROWS + row]);
        const float m_use = (mg == -INFINITY) ? 0.f : mg;
        const float f = fast_exp2(m_run[mt][h2] - m_use);
#pragma unroll
        for (int n = 0; n < NT_O; ++n) { o[mt][n][2 * h2] *= f; o[mt][n][2 * h2 + 1] *= f; }
      }
    // In the CTA's last segment the K/V ring is idle: every key slice writes its sums into a buffer of its own
    // there and the finishing loop adds the four up, in slice order -- the same additions in the same order as the
    // rounds below, so the same bits -- with one barrier instead of four rounds through one buffer.
    const bool last_seg = pre + nt_unit >= g1;
    if (last_seg) {
      float *cb = reinterpret_cast<float *>(stage_base) + ks * (ROWS * HEAD_DIM);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          const int row = mt * 16 + h2 * 8 + qd;
#pragma unroll
          for (int n = 0; n < NT_O; ++n) {
            const int d = ds * DW + n * 8 + ql * 2;
            *reinterpret_cast<float2 *>(cb + row * HEAD_DIM + (d ^ ((row & 7) << 3))) =
                make_float2(o[mt][n][2 * h2], o[mt][n][2 * h2 + 1]);
          }
        }
      consumer_sync(NCT);
    }
    // Earlier segments of a CTA (it takes several units, or the tail of one and the head of the next): the ring
    // already holds the next segment's tiles.  A unit of at most eight rows (one new token per sequence: six) still
    // gets a buffer per slice -- two in the Q region, which is idle until the next segment stages its rows, two in
    // 16 KB set aside for this -- and so one barrier here as well.  Same additions, same order, same bits.
    const bool small = MT == 1 && !last_seg && R <= 8;
    float *const sb = ks < 2 ? comb + ks * (8 * HEAD_DIM) : comb_extra + (ks - 2) * (8 * HEAD_DIM);
    if (small) {
      if (MT == 1) {
#pragma unroll
        for (int n = 0; n < NT_O; ++n) {
          const int d = ds * DW + n * 8 + ql * 2;
          *reinterpret_cast<float2 *>(sb + qd * HEAD_DIM + (d ^ ((qd & 7) << 3))) = make_float2(o[0][n][0], o[0][n][1]);
        }
      }
      consumer_sync(NCT);
    }
    for (int k = 0; k < SK_KS && !last_seg && !small; ++k) {
      if (ks == k) {
        // all loads of the round first, then all stores: read-add-write per element would serialise on
        // shared-memory latency (32 dependent round trips per thread and round)
        if (k) {
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              const int row = mt * 16 + h2 * 8 + qd;
#pragma unroll
              for (int n = 0; n < NT_O; ++n) {
                const int d = ds * DW + n * 8 + ql * 2;
                const float2 w = *reinterpret_cast<const float2 *>(comb + row * HEAD_DIM + (d ^ ((row & 7) << 3)));
                o[mt][n][2 * h2] += w.x;
                o[mt][n][2 * h2 + 1] += w.y;
              }
            }
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {
            const int row = mt * 16 + h2 * 8 + qd;
#pragma unroll
            for (int n = 0; n < NT_O; ++n) {
              const int d = ds * DW + n * 8 + ql * 2;
              *reinterpret_cast<float2 *>(comb + row * HEAD_DIM + (d ^ ((row & 7) << 3))) =
                  make_float2(o[mt][n][2 * h2], o[mt][n][2 * h2 + 1]);
            }
          }
      }
      consumer_sync(NCT);
    }

    // ---- finish the segment: final output, or a partial for the merge kernel ----
    for (int idx = tid; idx < R * 32; idx += NCT) {
      const int row = idx >> 5, c8 = idx & 31;  // channels c8*8 .. +7
      float mg = -INFINITY;
#pragma unroll
      for (int k = 0; k < SK_KS; ++k) mg = fmaxf(mg, mx[k * ROWS + row]);
      const float m_use = (mg == -INFINITY) ? 0.f : mg;
      float lg = 0.f;
#pragma unroll
      for (int k = 0; k < SK_KS; ++k) lg += lx[k * ROWS + row] * fast_exp2(mx[k * ROWS + row] - m_use);
      const float4 *srcp = reinterpret_cast<const float4 *>((last_seg ? reinterpret_cast<const float *>(stage_base) : comb) +
                                                            row * HEAD_DIM + ((c8 * 8) ^ ((row & 7) << 3)));
      float4 a = srcp[0], bq = srcp[1];
      if (small) {
        const int off = row * HEAD_DIM + ((c8 * 8) ^ ((row & 7) << 3));
#pragma unroll
        for (int k = 1; k < SK_KS; ++k) {
          const float4 *wp = reinterpret_cast<const float4 *>((k < 2 ? comb + k * (8 * HEAD_DIM) : comb_extra + (k - 2) * (8 * HEAD_DIM)) + off);
          const float4 wa = wp[0], wb = wp[1];
          a.x += wa.x; a.y += wa.y; a.z += wa.z; a.w += wa.w;
          bq.x += wb.x; bq.y += wb.y; bq.z += wb.z; bq.w += wb.w;
        }
      }
      if (last_seg) {
#pragma unroll
        for (int k = 1; k < SK_KS; ++k) {
          const float4 wa = srcp[k * (ROWS * HEAD_DIM / 4)], wb = srcp[k * (ROWS * HEAD_DIM / 4) + 1];
          a.x += wa.x; a.y += wa.y; a.z += wa.z; a.w += wa.w;
          bq.x += wb.x; bq.y += wb.y; bq.z += wb.z; bq.w += wb.w;
        }
      }
      float v[8] = {a.x, a.y, a.z, a.w, bq.x, bq.y, bq.z, bq.w};
      const int b = row / GROUP, hh = row % GROUP;
      const size_t grow = ((size_t)ui.s * p.n_new + ui.tok0 + b) * p.q_heads + (size_t)ui.kvh * GROUP + hh;
      if (whole && !p.partial_out) {
        const float inv = 1.f / lg;
        if (p.do_gate) {
          const uint4 g4 = *reinterpret_cast<const uint4 *>(p.gate + grow * HEAD_DIM + c8 * 8);
          const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            v[2 * j] *= inv * sigmoidf_(bf16lo(gw[j]));
            v[2 * j + 1] *= inv * sigmoidf_(bf16hi(gw[j]));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] *= inv;
        }
        store8<TOut>(reinterpret_cast<TOut *>(p.out) + grow * HEAD_DIM + c8 * 8, v);
        if (c8 == 0 && p.lse) p.lse[grow] = (mg + log2f(lg)) * LN2;
      } else {
        float *dst = (whole && p.partial_out)
                         ? p.partial_out + grow * PART_STRIDE
                         : p.ws + ((size_t)(cta + u) * (p.rb * GROUP) + row) * PART_STRIDE;
        *reinterpret_cast<float4 *>(dst + c8 * 8) = a;
        *reinterpret_cast<float4 *>(dst + c8 * 8 + 4) = bq;
        if (c8 == 0) { dst[256] = mg; dst[257] = lg; }
      }
    }
    // ---- with arrival counters: the CTA that completes a unit last merges it (after its own last tile) ----
    if (!whole && p.cnt) {
      // Release: the barrier orders every thread's partial stores before thread 0's fence, which is cumulative,
      // so one fence + atomic publishes the whole CTA's partial.  Acquire: the fence after the atomic, then the
      // barrier, order the merge's loads (which bypass L1) after the other CTAs' tickets.
      consumer_sync(NCT);
      if (tid == 0) {
        __threadfence();
        grid_dep_wait();  // the append kernel of this step clears the counters
        *ticket = atomicAdd(&p.cnt[u], 1);
        __threadfence();
        // the parts may be fetched by the copy engine: order its reads after this thread's acquire as well
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      consumer_sync(NCT);
      const int c_first = cta_of_tile(pre, total, G), c_last = cta_of_tile(pre + nt_unit - 1, total, G);
      // how many CTAs hold a part of the unit: all of c_first .. c_last when there are at least as many tiles as
      // CTAs (the usual case); otherwise count the ones that own tiles (two 64-bit divisions each: slow)
      int nparts = c_last - c_first + 1;
      if (total < (long long)G) {
        nparts = 0;
        for (int c = c_first; c <= c_last; ++c) nparts += (total * c / G != total * (c + 1) / G) ? 1 : 0;
      }
      // The merge itself waits until this CTA has no tiles left: the K/V ring is idle then and takes the parts by
      // bulk copy (one sequence alone is cut into dozens of parts: folding them row by row from global memory is
      // a chain of round trips several times longer than the streaming of its KV).  Which way a unit is merged
      // must not depend on which CTA happens to arrive last -- the two ways round differently -- and with the
      // merge deferred it depends on the shapes alone.  A slice has at most two cut units: its first and its last.
      // The notes -- (unit, first CTA, last CTA, parts, arrived last) each and their count -- live in shared memory:
      // the tile loop has no register to spare for them.  The sliced variant notes every cut unit: all of a unit's
      // CTAs take part in its merge.
      const bool sliced = SLICED && total >= (long long)G && nparts <= 160;
      if (tid == 0 && (sliced || *ticket == nparts - 1) && pend[10] < 2) {
        const int n = pend[10];
        pend[5 * n] = u; pend[5 * n + 1] = c_first; pend[5 * n + 2] = c_last; pend[5 * n + 3] = nparts;
        pend[5 * n + 4] = (*ticket == nparts - 1) ? 1 : 0;
        pend[10] = n + 1;
      }
    }
    pre += nt_unit;
    ++u;
  }
  consumer_sync(NCT);  // thread 0's notes above
  const int n_pend = pend[10];
  uint32_t merge_phase = 0;
  for (int k = 0; k < n_pend; ++k) {
    constexpr uint32_t MERGE_BUF = (uint32_t)(STAGES * SK_STAGE_BYTES + QREGION);
    const int um = pend[5 * k], cf = pend[5 * k + 1], cl = pend[5 * k + 2], np = pend[5 * k + 3];
    const int R = min(p.rb, p.n_new - ((um / p.kv_heads) % p.nblk) * p.rb) * GROUP;
    if (SLICED && total >= (long long)G && np <= 160) {
      // every CTA of the unit has taken its ticket before it waits here, so the count is reached as soon as the
      // slowest of them is through its tiles; the wait is bounded all the same
      if (tid == 0) {
        const uint64_t t0 = global_timer_ns();
        int got = 1;
        for (;;) {
          int v;
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p.cnt + um) : "memory");
          if (v >= np) break;
          if (global_timer_ns() - t0 > WAIT_LIMIT_NS) { got = 0; break; }
        }
        pend[11] = got;
      }
      consumer_sync(NCT);
      if (pend[11]) merge_unit_sliced<TOut>(p, um, cf, np, cta - cf, warp, lane, NCW);
      else if (tid == 0 && p.status) *p.status = DEV_ERR_FULL_WAIT;
      consumer_sync(NCT);  // pend[11] is written again for the next unit
      continue;            // the counter is left as it is: other CTAs of the unit may still be reading it
    }
    if (!pend[5 * k + 4]) continue;  // (sliced variant, unit merged the plain way: not this CTA's)
    if (total >= (long long)G && np <= 4) {
      merge_unit_direct<TOut>(p, um, cf, np, tid, NCT);
    } else if (total >= (long long)G && merge_bulk_fits(p, R, np, MERGE_BUF)) {
      if (!merge_unit_bulk<TOut>(p, um, cf, np, tid, NCT, smem, MERGE_BUF, merge_bar, merge_phase) && tid == 0 && p.status)
        *p.status = DEV_ERR_FULL_WAIT;
    } else {
      const UnitInfo ui = unit_info(p, um);
      for (int row = warp; row < R; row += NCW) merge_unit_row<TOut>(p, um, ui, row, cf, cl, total, lane, G);
    }
    if (tid == 0) p.cnt[um] = 0;  // leave the counter clean for a caller that does not reset it
  }
}

// Merge the partials of every unit that was cut across CTAs.  One block per unit, one warp per
// row, lane = 8 channels; partials are visited in CTA order so the sum order is fixed.
template <typename TOut>
__global__ void __launch_bounds__(256) splitkv_merge_kernel(const __grid_constant__ SplitKVParams p) {
  const int u = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_units = p.n_seq * p.nblk * p.kv_heads;
  __shared__ long long sh[3];
  if (warp == 0) {
    long long total; int live, geff; bool aligned;
    warp_partition(p, n_units, lane, total, live, geff, aligned);
    const long long pre = warp_unit_prefix(p, u, lane);
    if (lane == 0) { sh[0] = total; sh[1] = pre; sh[2] = geff; }
  }
  __syncthreads();
  const long long total = sh[0], pre = sh[1];
  const int G = (int)sh[2];
  const UnitInfo ui = unit_info(p, u);
  const int nt = (ui.len + SK_TK - 1) / SK_TK;
  if (nt == 0 || total == 0) return;
  const int c_first = cta_of_tile(pre, total, G), c_last = cta_of_tile(pre + nt - 1, total, G);
  if (c_first == c_last) return;  // the main kernel already wrote this unit
  const int R = ui.ntok * GROUP;
  for (int row = warp; row < R; row += 8) merge_unit_row_wide<TOut>(p, u, ui, row, c_first, c_last, total, lane, G);
}

// Merge n_parts partial sets [n_parts][n][PART_STRIDE] (n = rows * q_heads) in index order, then
// normalise and gate.  One warp per (row, head), lane = 8 channels.
template <typename TOut>
__global__ void __launch_bounds__(256) combine_partials_kernel(const float *parts, int n_parts, long long n,
                                                               const uint16_t *gate, TOut *out, float *lse) {
  const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= n) return;
  float mg = -INFINITY;
  for (int k = 0; k < n_parts; ++k) {
    const float *src = parts + ((size_t)k * n + r) * PART_STRIDE;
    if (src[257] > 0.f) mg = fmaxf(mg, src[256]);
  }
  const float m_use = (mg == -INFINITY) ? 0.f : mg;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  float lg = 0.f;
  for (int k = 0; k < n_parts; ++k) {
    const float *src = parts + ((size_t)k * n + r) * PART_STRIDE;
    const float l = src[257];
    if (!(l > 0.f)) continue;
    const float f = fast_exp2(src[256] - m_use);
    lg += l * f;
    const float4 a = *reinterpret_cast<const float4 *>(src + lane * 8);
    const float4 b = *reinterpret_cast<const float4 *>(src + lane * 8 + 4);
    acc[0] += a.x * f; acc[1] += a.y * f; acc[2] += a.z * f; acc[3] += a.w * f;
    acc[4] += b.x * f; acc[5] += b.y * f; acc[6] += b.z * f; acc[7] += b.w * f;
  }
  const float inv = 1.f / lg;
  if (gate) {
    float g[8];
    load8<uint16_t>(gate + r * HEAD_DIM + lane * 8, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= inv * sigmoidf_(g[j]);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= inv;
  }
  store8<TOut>(out + r * HEAD_DIM + lane * 8, acc);
  if (lane == 0 && lse) lse[r] = (mg + log2f(lg)) * LN2;
}

// The same merge with the exchange inside the kernel, over NVLink peer memory: rank k's partials are read
// straight from rank k's buffer (part_ptrs[k], a peer mapping of symmetric memory) -- no collective, no
// staging copy.  Every block publishes this rank's step number in its own flag word (release, system scope;
// the kernel that produced the partials ran before this one on the stream) and waits until every peer's flag
// has reached the step (acquire, system scope).  The wait is bounded (PEER_WAIT_NS): on expiry the block
// writes DEV_ERR_PEER_WAIT to *status and leaves without touching the output.  Buffers and flags alternate
// by step parity, which is enough to keep a fast rank from overwriting what a slow one still reads: a rank
// can publish step s + 2 only after its own combine of step s + 1, which waited for every peer to have
// finished step s.
constexpr unsigned long long PEER_WAIT_NS = 2000000000ull;
template <typename TOut>
__global__ void __launch_bounds__(256) combine_partials_peer_kernel(const float *const *part_ptrs, int *const *flag_ptrs,
                                                                    int rank, int n_parts, int step, long long n,
                                                                    const uint16_t *gate, TOut *out, float *lse,
                                                                    int *status) {
  __shared__ int failed;
  if (threadIdx.x == 0) {
    failed = 0;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag_ptrs[rank]), "r"(step) : "memory");
  }
  __syncthreads();
  // one thread per peer: the polls (a round trip over NVLink each) run side by side, not one peer after the other
  for (int k = threadIdx.x; k < n_parts; k += blockDim.x) {
    if (k == rank) continue;
    const int *f = flag_ptrs[k];
    const uint64_t t0 = global_timer_ns();
    for (;;) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if (v - step >= 0) break;  // the peer is at this step (or already past it)
      if (global_timer_ns() - t0 > PEER_WAIT_NS) {
        failed = 1;
        if (status) *status = DEV_ERR_PEER_WAIT;
        break;
      }
    }
  }
  __syncthreads();
  if (failed) return;
  const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= n) return;
  // A load from a peer's memory is a round trip over NVLink (2 to 3 us); chained one after the other -- the test of
  // l, then m, then the row, per part -- they made this kernel 31 us at two ranks and 76 us at four.  All loads of up
  // to eight parts are issued together, then folded in rank order with the arithmetic of combine_partials_kernel.
  float mg = -INFINITY, lg = 0.f;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (n_parts <= 8) {
    float mv[8], lv[8];
    float4 av[8], bv[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (k < n_parts) {
        const float *src = part_ptrs[k] + (size_t)r * PART_STRIDE;
        mv[k] = src[256];
        lv[k] = src[257];
        av[k] = *reinterpret_cast<const float4 *>(src + lane * 8);
        bv[k] = *reinterpret_cast<const float4 *>(src + lane * 8 + 4);
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < n_parts && lv[k] > 0.f) mg = fmaxf(mg, mv[k]);
    const float m_use = (mg == -INFINITY) ? 0.f : mg;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (k >= n_parts || !(lv[k] > 0.f)) continue;
      const float f = fast_exp2(mv[k] - m_use);
      lg += lv[k] * f;
      acc[0] += av[k].x * f; acc[1] += av[k].y * f; acc[2] += av[k].z * f; acc[3] += av[k].w * f;
      acc[4] += bv[k].x * f; acc[5] += bv[k].y * f; acc[6] += bv[k].z * f; acc[7] += bv[k].w * f;
    }
  } else {
    for (int k = 0; k < n_parts; ++k) {
      const float *src = part_ptrs[k] + (size_t)r * PART_STRIDE;
      if (src[257] > 0.f) mg = fmaxf(mg, src[256]);
    }
    const float m_use = (mg == -INFINITY) ? 0.f : mg;
    for (int k = 0; k < n_parts; ++k) {  // rank order, as in combine_partials_kernel: same bits
      const float *src = part_ptrs[k] + (size_t)r * PART_STRIDE;
      const float l = src[257];
      if (!(l > 0.f)) continue;
      const float f = fast_exp2(src[256] - m_use);
      lg += l * f;
      const float4 a4 = *reinterpret_cast<const float4 *>(src + lane * 8);
      const float4 b4 = *reinterpret_cast<const float4 *>(src + lane * 8 + 4);
      acc[0] += a4.x * f; acc[1] += a4.y * f; acc[2] += a4.z * f; acc[3] += a4.w * f;
      acc[4] += b4.x * f; acc[5] += b4.y * f; acc[6] += b4.z * f; acc[7] += b4.w * f;
    }
  }
  const float inv = 1.f / lg;
  if (gate) {
    float g[8];
    load8<uint16_t>(gate + r * HEAD_DIM + lane * 8, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= inv * sigmoidf_(g[j]);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= inv;
  }
  store8<TOut>(out + r * HEAD_DIM + lane * 8, acc);
  if (lane == 0 && lse) lse[r] = (mg + log2f(lg)) * LN2;
}

template <int MT, int DS, int STAGES>
constexpr size_t splitkv_smem_bytes() {
  return 1024 + (size_t)STAGES * SK_STAGE_BYTES + (size_t)MT * 16 * 1024 + 2 * SK_KS * MT * 16 * 4 +
         2 * STAGES * 8 + 3 * 8 + 96 + (MT == 1 ? 16 + 16384 : 0);
}

}  // namespace qwb
