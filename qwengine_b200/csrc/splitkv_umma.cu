// Split-KV attention for decode / speculative verify / short chunks on the tcgen05 tensor cores.
//
// Same work model as splitkv.cuh (units = (sequence, block of new tokens, KV head); all KV tiles of
// all units in one flat list cut evenly over a persistent grid; partials merged in CTA order by the
// CTA that completes a unit last), but the tile arithmetic runs on UMMA instead of mma.sync:
// a unit's query rows (token b, head hh) -> row 6 b + hh fill the first R <= 126 rows of a 128-row
// Q tile, S = Q K^T is a 128 x 128 x 256 tcgen05.mma per 128-key tile and O += P V a 128 x 256 x 128
// one with P (bf16 hi + lo) in tensor memory.  The rows beyond R are padding: the tensor pipe has
// the slack (3.3k cycles of MMA per 128 KB tile against ~5.4k cycles of HBM time per SM), and in
// exchange the per-tile instruction stream of the CUDA cores shrinks to the softmax of R rows, so
// the kernel stays HBM-bound for 24-row verify batches where the mma.sync kernel is issue-bound.
//
// Layout and roles follow prefill_umma2.cu: TMEM O | S0 | S1 (P over S), K/V through a ring of
// eight 16 KB TMA slots released by tcgen05.commit, warp 0 = producer, warp 1 = MMA issuer and
// TMEM owner, warps 2..17 = four softmax warpgroups (thread = row, warpgroup = 32-key column group
// and 64-channel output group).  Differences: Q is staged by the softmax threads themselves (plain
// loads, RoPE in double, bf16 hi + lo, written in the swizzled UMMA layout); each row has its own
// causal limit; a CTA walks several segments (unit, tile range), so every barrier phase is tracked
// with CTA-cumulative counters; a segment ends in a final store or in a partial + arrival ticket.
#include <atomic>
#include <cstring>

#include "splitkv.cuh"
#include "splitkv_umma.cuh"
#include "umma_common.cuh"

namespace qwb {

namespace {

constexpr int DU_BN = 128;                 // keys per tile
constexpr int DU_SLOT = 32768;             // half a K tile (128 keys x 128 channels) or half a V tile (64 keys x 256)
constexpr int DU_MAX_SLOT = 6;             // ring slots when the Q tile is smallest
constexpr int DU_SMEM_TOTAL = 232448 - 1024;   // dynamic shared memory left after the alignment slack
constexpr int DU_NWG = 4;
constexpr int DU_MAX_PARTS = 256;         // CTAs of one unit whose liveness is tabulated for the merge
constexpr int DU_SWITCH_TILES = 12;        // tiles of time charged to a CTA whose slice crosses into the next unit
constexpr int DU_SM_THREADS = DU_NWG * 128;
constexpr int DU_CTL_THREADS = 128;        // control warpgroup: TMA producer, MMA issuer, the partition warp, one idle warp
constexpr int DU_THREADS = DU_CTL_THREADS + DU_SM_THREADS;
constexpr int DU_CTL_REGS = 64, DU_SM_REGS = 104;  // after setmaxnreg: 128 x 64 + 512 x 104 = the 640 x 96 registers the block starts with

struct DecCtl {
  uint64_t q_ready, o_free, s_full[2], p_full[2], o_done[2];
  uint64_t slot_full[DU_MAX_SLOT], slot_empty[DU_MAX_SLOT];
  uint64_t merge_bar[2];         // bulk copies of a merge's parts land on them
  uint32_t tmem_base;
  volatile int abort_flag;
  volatile int ticket[2];
  volatile int merge_go;
  volatile int merge_parts[2];   // CTAs that hold a part of each pending unit
  volatile uint8_t merge_live[2][DU_MAX_PARTS];
  long long part[5];             // total tiles, flat index of the first unit's tile 0, first unit, CTAs in use, lead entries per unit
  float mxbuf[2][DU_NWG][128];
  float lbuf[DU_NWG][128];
};

// Byte offset of element (row, d) of the Q tile: 64-channel sub-tiles (sub_bytes apart) of 128-byte
// rows, 16-byte column XOR (row & 7) -- the K-major 128-byte-swizzle operand layout.
//
// Only the first q_rows_pad (32, 64 or 128) rows of the 128-row MMA tile exist in shared memory.
// The operand descriptor still spans 128 rows; the rows past q_rows_pad read whatever follows (the
// next sub-tile, the ring), which is valid shared memory whose contents only reach accumulator rows
// that nobody reads.  That shrinks Q from 80 KB to 20 KB for decode and verify and gives the bytes
// to the K/V ring, where an HBM-bound kernel needs them (bytes in flight = bandwidth x latency).
__device__ __forceinline__ uint32_t q_tile_off(int row, int d, int sub_bytes) {
  return (uint32_t)((d >> 6) * sub_bytes + row * 128 + ((((d >> 3) & 7) ^ (row & 7)) << 4) + ((d & 7) << 1));
}

template <typename TOut>
__global__ void __launch_bounds__(DU_THREADS, 1)
splitkv_umma_kernel(const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                    const __grid_constant__ SplitKVParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int QSUB = p.q_rows_pad * 128;      // bytes of one 64-channel Q sub-tile
  const int DU_NSLOT = p.nslot;
  uint8_t *q_smem = smem;
  uint8_t *ring = smem + 5 * QSUB;          // four sub-tiles + the rotary "lo" sub-tile; a multiple of 1 KB
  DecCtl *ctl = reinterpret_cast<DecCtl *>(smem + DU_SMEM_TOTAL - sizeof(DecCtl));

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_units = p.n_seq * p.nblk * p.kv_heads;
  const int cta = blockIdx.x;
  // a kernel launched behind this one as a programmatic dependent (this library's append kernel is) may become
  // resident now; it waits for this grid's completion before it touches memory
  grid_dep_launch_dependents();

  if (tid == 0) {
    // the softmax warps signal once per warp (each lane's fence, __syncwarp, then lane 0 arrives): 512 arrivals on
    // one barrier per signal cost more than the work between two signals
    mbar_init(&ctl->q_ready, DU_SM_THREADS / 32);
    mbar_init(&ctl->o_free, DU_SM_THREADS / 32);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl->s_full[i], 1);
      mbar_init(&ctl->p_full[i], DU_SM_THREADS / 32);
      mbar_init(&ctl->o_done[i], 1);
    }
    for (int i = 0; i < DU_MAX_SLOT; ++i) { mbar_init(&ctl->slot_full[i], 1); mbar_init(&ctl->slot_empty[i], 1); }
    mbar_init(&ctl->merge_bar[0], 1);
    mbar_init(&ctl->merge_bar[1], 1);
    ctl->abort_flag = (p.status && *reinterpret_cast<volatile int *>(p.status) != 0) ? 1 : 0;
    fence_barrier_init();
    prefetch_tensormap(&mapK);
    prefetch_tensormap(&mapV);
  }
  if (warp == 2) {
    long long total; int live, geff; bool aligned;
    warp_partition<DU_BN>(p, n_units, lane, total, live, geff, aligned);
    const int lead = aligned ? 0 : DU_SWITCH_TILES + (p.rb * GROUP) / 16;
    // Where the grid could not be aligned with the units, a CTA whose slice runs over a unit boundary
    // loses time there (the pipeline drains: last P V, read-out of O, new Q tile): about 11 us, three
    // to four tiles, measured; and it is usually the last to arrive at both of its units, so it merges
    // both, one after the other, at the very end of the kernel.  The flat list charges for it: every unit
    // is preceded by `lead` entries that stand for no tile, so such a CTA receives that many tiles less.
    // Measured on the ragged verify batch (kernel, two boxes): 5 entries 0.140 ms, 7 0.137-0.139, 9 0.131-0.135,
    // 11 0.135, 13 0.131-0.133, 15 0.129-0.130, 17 0.129-0.131, 21 0.133.  13 is used: beyond it the gain is the
    // batch's own (its boundary CTAs stop being the last at both of their units), and a batch of many short
    // units would be charged more than a boundary costs.
    total += (long long)lead * live;
    int u0 = n_units; long long pre0 = 0;
    if (cta < geff) warp_find_unit<DU_BN>(p, n_units, lane, total * cta / geff, u0, pre0, lead);
    if (lane == 0) { ctl->part[0] = total; ctl->part[1] = pre0; ctl->part[2] = u0; ctl->part[3] = geff; ctl->part[4] = lead; }
  } else if (warp == 1) {  // meanwhile: tensor memory
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  const long long total = ctl->part[0];
  const int G = (int)ctl->part[3], LEAD = (int)ctl->part[4];
  const long long g0 = cta < G ? total * cta / G : 0, g1 = cta < G ? total * (cta + 1) / G : 0;
  if (g0 >= g1 || ctl->abort_flag) {  // uniform: nothing to do, or the launch already failed
    if (warp == 1) tmem_dealloc(tmem, 512);
    return;
  }
  // Advance (u, pre) to the next unit that has tiles inside this CTA's slice [g0, g1) of the flat
  // list; t0 / t1 bound those tiles.  The first LEAD entries of a unit stand for no tile.
  auto find_live = [&](int &u, long long &pre, int &nt, int &t0, int &t1) -> bool {
    while (u < n_units && pre < g1) {
      nt = unit_tiles<DU_BN>(p, u);
      const int vt = nt > 0 ? nt + LEAD : 0;
      t0 = max((int)(max(g0, pre) - pre) - LEAD, 0);
      t1 = max((int)(min(g1, pre + vt) - pre) - LEAD, 0);
      if (t0 < t1) return true;
      pre += vt;
      ++u;
    }
    return false;
  };
  volatile int *abort_flag = &ctl->abort_flag;
  auto fail = [&](int code) {
    if (!*abort_flag && p.status) *p.status = code;
    *abort_flag = 1;
  };

  // Registers: five warpgroups start with 96 per thread; the control warpgroup hands a third of its share to
  // the four softmax warpgroups (setmaxnreg, first thing in each branch: the compiler changes the register
  // budget only for code that the instruction dominates), so the softmax loop holds its 64 values of S and P
  // per thread without spilling.
  if (warp == 0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(DU_CTL_REGS));
    // =============================== TMA producer ===========================================
    // Per segment the slot stream is  K_t0 | K_t0+1 V_t0 | ... | V_t1-1 ; segments follow each
    // other without a gap.  A K slot is two 64-channel sub-tiles of 128 keys, a V slot 64 keys x 256 channels
    // (32 KB each: fewer, larger slots keep the issuing thread's waits and commits off the tensor pipe's path).
    if (elect_one()) {
      int u = (int)ctl->part[2];
      long long pre = ctl->part[1];
      int sl = 0;            // ring position: slot, and the parity of the slot's current use
      uint32_t ph = 0;
      bool wrapped = false, ok = true, dep_waited = false;
      auto slot_ready = [&]() -> bool {
        if (wrapped && !wait_or_abort(&ctl->slot_empty[sl], ph ^ 1, abort_flag)) {
          fail(DEV_ERR_EMPTY_WAIT);
          ok = false;
          return false;
        }
        mbar_expect_tx(&ctl->slot_full[sl], DU_SLOT);
        return true;
      };
      auto advance = [&]() {
        if (++sl == DU_NSLOT) { sl = 0; ph ^= 1; wrapped = true; }
      };
      int nt, t0, t1;
      while (ok && find_live(u, pre, nt, t0, t1)) {
        const UnitInfo ui = unit_info(p, u);
        const long long base = p.cache_row ? p.cache_row[ui.s] : 0;
        for (int j = t0; j <= t1 && ok; ++j) {
          if (j < t1) {
            if (!dep_waited && (j + 1) * DU_BN > ui.pos) {  // first tile with rows of this step's append kernel
              grid_dep_wait();
              dep_waited = true;
            }
            const int krow = (int)cache_row_at(p.pages, base, ui.s, j * DU_BN);  // a tile never straddles a page
            for (int c2 = 0; c2 < 2 && ok; ++c2) {  // two 64-channel sub-tiles per slot
              if (!slot_ready()) break;
#pragma unroll
              for (int a = 0; a < 2; ++a)
                tma_load_2d(ring + sl * DU_SLOT + a * 16384, &mapK, &ctl->slot_full[sl],
                            ui.kvh * HEAD_DIM + (2 * c2 + a) * 64, krow);
              advance();
            }
          }
          if (j > t0 && ok) {
            const int vrow = (int)cache_row_at(p.pages, base, ui.s, (j - 1) * DU_BN);
            for (int g = 0; g < 2 && ok; ++g) {
              if (!slot_ready()) break;
#pragma unroll
              for (int c = 0; c < 4; ++c)  // 64 keys x 64 channels each, channel atoms 8 KB apart
                tma_load_2d(ring + sl * DU_SLOT + c * 8192, &mapV, &ctl->slot_full[sl], ui.kvh * HEAD_DIM + c * 64,
                            vrow + g * 64);
              advance();
            }
          }
        }
        pre += nt + LEAD;
        ++u;
      }
    }
  } else if (warp == 1) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(DU_CTL_REGS));
    // =============================== MMA issuer ==============================================
    // One elected thread walks the tile sequence and issues everything.  J counts tiles over all segments of this CTA: S / P buffer J & 1,
    // barrier phase J >> 1.
    if (elect_one()) {
    const uint32_t idesc_qk = make_idesc(128, 128, 1, 1, 0, 0);
    const uint32_t idesc_pv = make_idesc(128, 256, 1, 1, 0, 1);
    const uint64_t qdesc0 = smem_desc(smem_u32(q_smem), 16, 1024);
    const uint64_t kdesc0 = smem_desc(smem_u32(ring), 16, 1024);
    const uint64_t vdesc0 = smem_desc(smem_u32(ring), 8192, 1024);  // channel atoms 8 KB apart, 8-key groups 1 KB
    const uint32_t qsub16 = (uint32_t)(QSUB >> 4);
    int u = (int)ctl->part[2];
    long long pre = ctl->part[1];
    int sl = 0;
    uint32_t ph = 0;
    int J = 0, seg = 0;
    bool ok = true;
    auto wait_all = [&](uint64_t *bar, uint32_t parity, int code) {
      const bool got = wait_or_abort(bar, parity, abort_flag);
      if (!got) {
        fail(code);
        ok = false;
      }
      return got;
    };
    auto advance = [&]() {
      if (++sl == DU_NSLOT) { sl = 0; ph ^= 1; }
    };
    int nt, t0, t1;
    while (ok && find_live(u, pre, nt, t0, t1)) {
      if (!wait_all(&ctl->q_ready, seg & 1, DEV_ERR_MMA_WAIT)) break;
      tc_fence_after();
      for (int j = t0; j <= t1 && ok; ++j) {
        const int Jt = J + (j - t0);
        if (j < t1) {
          // ---- S[Jt & 1] = Q K_j^T ----
          const uint32_t d_s = tmem + ((Jt & 1) ? TMEM_S1 : TMEM_S0);
          for (int c2 = 0; c2 < 2 && ok; ++c2) {  // a slot = two 64-channel sub-tiles of the K tile
            if (!wait_all(&ctl->slot_full[sl], ph, DEV_ERR_MMA_WAIT)) break;
            tc_fence_after();
#pragma unroll
            for (int a = 0; a < 2; ++a) {
              const int c = 2 * c2 + a;
              const uint64_t kd = kdesc0 + (uint64_t)((sl * DU_SLOT + a * 16384) >> 4);
              const uint64_t qd = qdesc0 + (uint64_t)(c * qsub16);
#pragma unroll
              for (int k = 0; k < 4; ++k) umma_ss(d_s, qd + (uint64_t)(k * 2), kd + (uint64_t)(k * 2), idesc_qk, (c | k) != 0);
              if (c == 0 && p.q_lo_dims) {  // low-order part of the rotated channels against the same K sub-tile
                const uint64_t ql = qdesc0 + (uint64_t)(4 * qsub16);
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_ss(d_s, ql + (uint64_t)(k * 2), kd + (uint64_t)(k * 2), idesc_qk, 1);
              }
            }
            umma_commit(&ctl->slot_empty[sl]);
            if (c2 == 1) umma_commit(&ctl->s_full[Jt & 1]);
            advance();
          }
        }
        if (j > t0 && ok) {
          // ---- O (+)= P_{j-1} V_{j-1} ----
          const int jj = j - 1, Jp = Jt - 1;
          if (!wait_all(&ctl->p_full[Jp & 1], (Jp >> 1) & 1, DEV_ERR_SOFTMAX_WAIT)) break;
          // the first P V of a segment overwrites O: the previous segment must have read it out
          if (jj == t0 && seg > 0 && !wait_all(&ctl->o_free, (seg - 1) & 1, DEV_ERR_SOFTMAX_WAIT)) break;
          tc_fence_after();
          const uint32_t a_p = tmem + ((Jp & 1) ? TMEM_S1 : TMEM_S0);
          for (int g = 0; g < 2 && ok; ++g) {  // a slot = 64 keys of the V tile
            if (!wait_all(&ctl->slot_full[sl], ph, DEV_ERR_MMA_WAIT)) break;
            tc_fence_after();
            const uint64_t vd = vdesc0 + (uint64_t)(sl * (DU_SLOT >> 4));
            const uint32_t first = (uint32_t)(jj != t0) | (uint32_t)g;
#pragma unroll
            for (int k = 0; k < 4; ++k) {  // 16 keys per step: 2 KB further in every channel atom
              umma_ts(tmem + TMEM_O, a_p + (g * 4 + k) * 8, vd + (uint64_t)(k * 128), idesc_pv, first | (uint32_t)k);
              umma_ts(tmem + TMEM_O, a_p + 64 + (g * 4 + k) * 8, vd + (uint64_t)(k * 128), idesc_pv, 1);
            }
            umma_commit(&ctl->slot_empty[sl]);
            if (g == 1) umma_commit(&ctl->o_done[Jp & 1]);
            advance();
          }
        }
      }
      J += t1 - t0;
      ++seg;
      pre += nt + LEAD;
      ++u;
    }
    }
  } else if (warp < DU_CTL_THREADS / 32) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(DU_CTL_REGS));  // the other two warps of the control warpgroup
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(DU_SM_REGS));
    // ============ softmax / correction / epilogue: thread = (row, 32-key column group) ============
    const int wg = (warp - DU_CTL_THREADS / 32) >> 2;
    const int row = (warp & 3) * 32 + lane;
    const int st_tid = tid - DU_CTL_THREADS;              // 0 .. 511
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    int u = (int)ctl->part[2];
    long long pre = ctl->part[1];
    int J = 0, o_seen = 0;
    bool ok = true;
    // P V completions are observed strictly in order (tile t: o_done[t & 1], phase t / 2)
    auto wait_pv_done = [&](int upto) {
      while (ok && o_seen <= upto) {
        ok = wait_or_abort(&ctl->o_done[o_seen & 1], (o_seen >> 1) & 1, abort_flag);
        ++o_seen;
      }
    };
    // ---- stage Q of one unit: rows (token b, head hh) -> 6 b + hh, zero padding above R ----
    // The rotary channels are rotated on the way (angle reduced in double) and split into a bf16
    // value and its bf16 remainder.
    auto stage_q = [&](const UnitInfo &ui) {
      const int R = ui.ntok * GROUP;
      if (p.q_dep) grid_dep_wait();  // q comes out of the launch before this one
      // Two passes of the thread group at a time, with every global load of both issued before the first is
      // used: a 32-row tile (decode, verify) is staged in one memory round trip instead of four.
      const int n_items = p.q_rows_pad * 32;  // 8-channel chunks, and as many rotary pairs
      for (int base = 0; base < n_items; base += 2 * DU_SM_THREADS) {
        uint4 xq[2];
        uint16_t rx[2], ry[2];
#pragma unroll
        for (int it = 0; it < 2; ++it) {
          const int idx = base + it * DU_SM_THREADS + st_tid;
          const int r = idx >> 5, c16 = idx & 31;           // 8 channels c16*8 .. +7
          xq[it] = make_uint4(0, 0, 0, 0);
          rx[it] = ry[it] = 0;
          if (idx < n_items && r < R) {
            const size_t grow = ((size_t)ui.s * p.n_new + ui.tok0 + r / GROUP) * p.q_heads + (size_t)ui.kvh * GROUP + r % GROUP;
            const uint16_t *src = reinterpret_cast<const uint16_t *>(p.q) + grow * HEAD_DIM;
            if (!(p.do_rope && c16 < 8)) xq[it] = *reinterpret_cast<const uint4 *>(src + c16 * 8);
            if (p.do_rope) {  // the same index also names rotary pair (i, i + 32) = (c16, c16 + 32) of row r
              rx[it] = src[c16];
              ry[it] = src[c16 + ROT_PAIRS];
            }
          }
        }
#pragma unroll
        for (int it = 0; it < 2; ++it) {
          const int idx = base + it * DU_SM_THREADS + st_tid;
          if (idx >= n_items) continue;
          const int r = idx >> 5, c16 = idx & 31;
          if (!(p.do_rope && c16 < 8))                      // rotary channels are written pair-wise below
            *reinterpret_cast<uint4 *>(q_smem + q_tile_off(r, c16 * 8, QSUB)) = xq[it];
          if (!p.do_rope) continue;
          const int i = c16;
          float xr = 0.f, yr = 0.f;
          if (r < R) {
            const size_t trow = (size_t)ui.s * p.n_new + ui.tok0 + r / GROUP;
            const int pz = p.mpos ? p.mpos[trow * 3 + mrope_component(i)] : ui.rpos + ui.tok0 + r / GROUP;
            float c, sn;
            rope_sincos_reduced(pz, p.rope.inv_freq[i], c, sn);
            const float x = bf16_bits_to_f32(rx[it]), y = bf16_bits_to_f32(ry[it]);
            xr = x * c - y * sn;
            yr = x * sn + y * c;
          }
          const uint16_t xh = f32_to_bf16_bits(xr), yh = f32_to_bf16_bits(yr);
          *reinterpret_cast<uint16_t *>(q_smem + q_tile_off(r, i, QSUB)) = xh;
          *reinterpret_cast<uint16_t *>(q_smem + q_tile_off(r, i + ROT_PAIRS, QSUB)) = yh;
          *reinterpret_cast<uint16_t *>(q_smem + 4 * QSUB + q_tile_off(r, i, QSUB)) = f32_to_bf16_bits(xr - bf16_bits_to_f32(xh));
          *reinterpret_cast<uint16_t *>(q_smem + 4 * QSUB + q_tile_off(r, i + ROT_PAIRS, QSUB)) =
              f32_to_bf16_bits(yr - bf16_bits_to_f32(yh));
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->q_ready);
    };
    // units cut across CTAs: their merge is settled after this CTA's last tile
    // (first and last CTA of each such unit are worked out right away, in the warm part of the kernel: two 64-bit
    // divisions each, which would otherwise sit on the path between the last tile and the merge)
    int pend_u[2] = {0, 0}, pend_cf[2] = {0, 0}, pend_cl[2] = {0, 0}, n_pend = 0;
    int nt, t0, t1;
    bool have = find_live(u, pre, nt, t0, t1);
    if (have) stage_q(unit_info(p, u));
    while (have) {
      const UnitInfo ui = unit_info(p, u);
      // the unit this CTA works on next, if any: its Q tile is staged ahead of time (below)
      int u_next = u + 1, nt_next, t0_next, t1_next;
      long long pre_next = pre + nt + LEAD;
      const bool have_next = find_live(u_next, pre_next, nt_next, t0_next, t1_next);
      const int R = ui.ntok * GROUP;
      const bool whole = (t0 == 0 && t1 == nt);
      const bool warp_live = (warp & 3) * 32 < R;         // this warp holds at least one real row

      // keys visible to this row; padding rows see none
      const int lim = row < R ? (p.no_causal ? ui.pos : ui.pos + ui.tok0 + row / GROUP + 1) : 0;
      const int lim_min = p.no_causal ? ui.pos : ui.pos + ui.tok0 + 1;
      float m_used = -INFINITY, l_run = 0.f;
      for (int j = t0; j < t1; ++j) {
        const int Jt = J + (j - t0);
        const uint32_t t_s = tmem + lane_sel + ((Jt & 1) ? TMEM_S1 : TMEM_S0);
        if (ok) ok = wait_or_abort(&ctl->s_full[Jt & 1], (Jt >> 1) & 1, abort_flag);
        tc_fence_after();
        uint32_t sr[32];
        float mx = -INFINITY;
        if (warp_live) {
          tmem_ld32(t_s + wg * 32, sr);
          tmem_wait_ld();
          const int key0 = j * DU_BN + wg * 32;
          if (j * DU_BN + DU_BN > lim_min || row >= R) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float v = __uint_as_float(sr[i]);
              v = (key0 + i < lim) ? v : -INFINITY;
              sr[i] = __float_as_uint(v);
              mx = fmaxf(mx, v);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(sr[i]));
          }
        }
        ctl->mxbuf[Jt & 1][wg][row] = mx;
        asm volatile("bar.sync 1, %0;" ::"n"(DU_SM_THREADS) : "memory");
#pragma unroll
        for (int w2 = 0; w2 < DU_NWG; ++w2) mx = fmaxf(mx, ctl->mxbuf[Jt & 1][w2][row]);
        const float m_new = fmaxf(m_used, mx * p.scale_log2);
        if (__any_sync(0xffffffffu, m_new - m_used > PF_RESCALE_THRESHOLD)) {
          if (j > t0) {
            const float alpha = fast_exp2(m_used - m_new);
            l_run *= alpha;
            wait_pv_done(Jt - 1);  // O may only be touched once the previous P V has retired
            if (__all_sync(0xffffffffu, ok)) {
              tc_fence_after();
              const uint32_t t_o = tmem + lane_sel + TMEM_O + wg * 64;
#pragma unroll 1
              for (int c = 0; c < 2; ++c) {
                uint32_t orow[32];
                tmem_ld32(t_o + c * 32, orow);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
                tmem_st32(t_o + c * 32, orow);
              }
              tmem_wait_st();
            }
          }
          m_used = m_new;
        }
        if (warp_live) {
          const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
          float lsum = 0.f;
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {  // 16 keys at a time: fewer packed values live at once
            uint32_t hi[8], lo[8];
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              const float p0 = fast_exp2(fmaf(__uint_as_float(sr[h2 * 16 + i]), p.scale_log2, -m_sub));
              const float p1 = fast_exp2(fmaf(__uint_as_float(sr[h2 * 16 + i + 1]), p.scale_log2, -m_sub));
              lsum += p0 + p1;
              const uint32_t h = pack_bf16(p0, p1);
              hi[i >> 1] = h;
              lo[i >> 1] = pack_bf16(p0 - bf16lo(h), p1 - bf16hi(h));
            }
            tmem_st8(t_s + wg * 16 + h2 * 8, hi);
            tmem_st8(t_s + 64 + wg * 16 + h2 * 8, lo);
          }
          l_run += lsum;
          tmem_wait_st();
        }
        // Keys past the end of the unit may hold anything in V; P is zero there but 0 * NaN is NaN,
        // so those rows are cleared before the tensor core reads them.  The ragged tile is the
        // unit's last, hence the last of its segment: its V slots are the two that follow the
        // 4 Jt + 2 slots consumed before them.
        if (j * DU_BN + DU_BN > ui.len) {
          for (int g = 0; g < 2; ++g) {
            const int key_lo = j * DU_BN + g * 64;
            if (key_lo + 64 <= ui.len) continue;
            const uint32_t itv = 4u * (uint32_t)Jt + 2u + (uint32_t)g;
            const int sl = (int)(itv % (uint32_t)DU_NSLOT);
            if (ok) ok = wait_or_abort(&ctl->slot_full[sl], (itv / (uint32_t)DU_NSLOT) & 1u, abort_flag);
            const int valid = max(0, ui.len - key_lo);
            for (int idx = st_tid; idx < 64 * 32; idx += DU_SM_THREADS) {
              const int kr = idx >> 5, c16 = idx & 31;
              if (kr >= valid)
                *reinterpret_cast<uint4 *>(ring + sl * DU_SLOT + (c16 >> 3) * 8192 + kr * 128 + (((c16 & 7) ^ (kr & 7)) << 4)) =
                    make_uint4(0, 0, 0, 0);
            }
          }
          fence_proxy_async();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->p_full[Jt & 1]);
        // Last tile of the segment: every Q K^T of this unit has completed (s_full above), so the Q
        // tile is free -- stage the next unit's rows while the tensor core runs this tile's P V.
        if (j == t1 - 1 && have_next) stage_q(unit_info(p, u_next));
        if (j > t0) wait_pv_done(Jt - 1);
      }
      // ---- end of the segment: read O out, release it, then store the result or a partial ----
      wait_pv_done(J + (t1 - t0) - 1);
      ctl->lbuf[wg][row] = l_run;
      asm volatile("bar.sync 1, %0;" ::"n"(DU_SM_THREADS) : "memory");
      float l_tot = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < DU_NWG; ++w2) l_tot += ctl->lbuf[w2][row];
      const bool all_ok = __all_sync(0xffffffffu, ok);
      const size_t grow = ((size_t)ui.s * p.n_new + ui.tok0 + row / GROUP) * p.q_heads + (size_t)ui.kvh * GROUP + row % GROUP;
      const bool final_store = whole && !p.partial_out;
      float *part_dst = (whole ? p.partial_out + grow * PART_STRIDE
                               : p.ws + ((size_t)(cta + u) * (p.rb * GROUP) + row) * PART_STRIDE) + wg * 64;
      if (warp_live && all_ok) {
        tc_fence_after();
        const uint32_t t_o = tmem + lane_sel + TMEM_O + wg * 64;
        const float inv = 1.f / l_tot;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t orow[32];
          tmem_ld32(t_o + c * 32, orow);
          tmem_wait_ld();
          if (row < R) {
            if (final_store) {
              const size_t off = grow * HEAD_DIM + wg * 64 + c * 32;
#pragma unroll
              for (int v8 = 0; v8 < 4; ++v8) {
                float o8[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) o8[e] = __uint_as_float(orow[v8 * 8 + e]) * inv;
                if (p.do_gate) {
                  float g8[8];
                  load8<uint16_t>(p.gate + off + v8 * 8, g8);
#pragma unroll
                  for (int e = 0; e < 8; ++e) o8[e] *= sigmoid_fast(g8[e]);
                }
                store8<TOut>(reinterpret_cast<TOut *>(p.out) + off + v8 * 8, o8);
              }
            } else {
#pragma unroll
              for (int v4 = 0; v4 < 8; ++v4)
                *reinterpret_cast<uint4 *>(part_dst + c * 32 + v4 * 4) =
                    make_uint4(orow[v4 * 4], orow[v4 * 4 + 1], orow[v4 * 4 + 2], orow[v4 * 4 + 3]);
            }
          }
        }
        if (row < R && wg == 0) {
          if (final_store) {
            if (p.lse) p.lse[grow] = (m_used + log2f(l_tot)) * LN2;
          } else {
            part_dst[256] = m_used;
            part_dst[257] = l_tot;
          }
        }
      }
      // O has been read (or is abandoned): the next segment's first P V may overwrite it
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->o_free);
      if (!all_ok) {
        if (lane == 0) fail(DEV_ERR_SOFTMAX_WAIT);
        break;
      }
      if (!whole) {  // at most the first and the last segment of a CTA
        pend_u[n_pend] = u;
        pend_cf[n_pend] = cta_of_tile(pre + LEAD, total, G);
        pend_cl[n_pend] = cta_of_tile(pre + LEAD + nt - 1, total, G);
        ++n_pend;
      }
      J += t1 - t0;
      have = have_next;
      u = u_next; pre = pre_next; nt = nt_next; t0 = t0_next; t1 = t1_next;
    }
    // ---- units cut across CTAs are merged by whichever of their CTAs arrives last ----
    if (n_pend > 0) {  // n_pend is the same in all softmax threads
      // which CTAs of c_first .. c_last hold a part (one thread per CTA: the test is two 64-bit divisions)
      // (with at least as many entries as CTAs every CTA of the span owns some and has written its part)
      const bool all_live = total >= (long long)G;
      for (int k = 0; k < n_pend && !all_live; ++k) {
        const int c_first = pend_cf[k], c_last = pend_cl[k];
        for (int i = st_tid; i <= c_last - c_first && i < DU_MAX_PARTS; i += DU_SM_THREADS)
          ctl->merge_live[k][i] = (total * (c_first + i) / G != total * (c_first + i + 1) / G) ? 1 : 0;
      }
      // release / acquire through one thread: the barrier orders every thread's partial stores before that
      // thread's (cumulative) fence and ticket; its second fence and the next barrier order the merge's loads
      // (which bypass L1) after the other CTAs' tickets
      asm volatile("bar.sync 1, %0;" ::"n"(DU_SM_THREADS) : "memory");
      if (st_tid == 0) {  // one thread decides, so that a failure flagged meanwhile cannot split the group
        const int go = *abort_flag ? 0 : 1;
        __threadfence();
        grid_dep_wait();  // the append kernel of this step clears the counters
        for (int k = 0; k < n_pend && go; ++k) {
          const int c_first = pend_cf[k], c_last = pend_cl[k];
          int nparts = all_live ? c_last - c_first + 1 : 0;
          for (int i = 0; i <= c_last - c_first && !all_live; ++i)
            nparts += i < DU_MAX_PARTS ? ctl->merge_live[k][i] : ((total * (c_first + i) / G != total * (c_first + i + 1) / G) ? 1 : 0);
          ctl->merge_parts[k] = nparts;
        }
        // both tickets in flight together (one memory round trip), not one after the other
        const int tk0 = (go && n_pend > 0) ? atomicAdd(&p.cnt[pend_u[0]], 1) : 0;
        const int tk1 = (go && n_pend > 1) ? atomicAdd(&p.cnt[pend_u[1]], 1) : 0;
        ctl->ticket[0] = tk0;
        ctl->ticket[1] = tk1;
        __threadfence();
        // the parts are fetched by the copy engine: order its reads after this thread's acquire as well
        asm volatile("fence.proxy.async;" ::: "memory");
        ctl->merge_go = go;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(DU_SM_THREADS) : "memory");
      uint32_t merge_phase = 0;
      for (int k = 0; k < n_pend && ctl->merge_go; ++k) {
        if (p.sliced && all_live && ctl->merge_parts[k] <= 160) {
          // Few long units (one sequence's draft tokens on the whole device): every CTA of the unit merges a slice
          // of its channels once all parts have arrived.  All of them have taken their tickets before they wait
          // here; the wait is bounded all the same.
          if (st_tid == 0) {
            const uint64_t t0 = global_timer_ns();
            int got = 1;
            for (;;) {
              int v;
              asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p.cnt + pend_u[k]) : "memory");
              if (v >= ctl->merge_parts[k]) break;
              if (*abort_flag || global_timer_ns() - t0 > WAIT_LIMIT_NS) { got = 0; break; }
            }
            ctl->merge_go = got;
            if (!got) fail(DEV_ERR_SOFTMAX_WAIT);
          }
          asm volatile("bar.sync 1, %0;" ::"n"(DU_SM_THREADS) : "memory");
          if (ctl->merge_go)
            merge_unit_sliced<TOut>(p, pend_u[k], pend_cf[k], ctl->merge_parts[k], cta - pend_cf[k],
                                    warp - DU_CTL_THREADS / 32, lane, DU_SM_THREADS / 32);
          asm volatile("bar.sync 1, %0;" ::"n"(DU_SM_THREADS) : "memory");
          continue;  // the counter is left as it is: other CTAs of the unit may still be reading it
        }
        if (ctl->ticket[k] == ctl->merge_parts[k] - 1) {
          const int c_first = pend_cf[k], c_last = pend_cl[k];
          const int blk = (pend_u[k] / p.kv_heads) % p.nblk;  // no load on the way to the merge: unit_info reads pos
          const int R = min(p.rb, p.n_new - blk * p.rb) * GROUP, span = c_last - c_first + 1;
          // the Q tile and the K/V ring are idle by now: one buffer from the start of Q to the control block
          const uint32_t buf_bytes = (uint32_t)(reinterpret_cast<uint8_t *>(ctl) - q_smem) & ~15u;
          if (all_live && merge_bulk_fits(p, R, span, buf_bytes)) {
            if (!merge_unit_bulk<TOut>(p, pend_u[k], c_first, span, st_tid, DU_SM_THREADS, q_smem, buf_bytes,
                                       ctl->merge_bar, merge_phase)) {
              if (st_tid == 0) fail(DEV_ERR_SOFTMAX_WAIT);
              break;
            }
          } else {
            const UnitInfo ui = unit_info(p, pend_u[k]);
            for (int r = warp - DU_CTL_THREADS / 32; r < R; r += DU_NWG * 4)
              merge_unit_row<TOut>(p, pend_u[k], ui, r, c_first, c_last, total, lane, G,
                                   span <= DU_MAX_PARTS ? ctl->merge_live[k] : nullptr);
          }
          if (st_tid == 0) p.cnt[pend_u[k]] = 0;
        }
      }
    }
  }

  // ---- teardown ----
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) { }
    }
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace

bool splitkv_umma_usable(int n_new) { return n_new >= 1 && n_new < 64; }
int splitkv_umma_rb(int n_new) { return n_new < 21 ? n_new : 21; }  // 21 tokens x 6 heads = 126 rows of the tile
void splitkv_umma_layout(int rb, int *q_rows_pad, int *nslot) {
  const int rows = rb * GROUP;
  *q_rows_pad = rows <= 32 ? 32 : (rows <= 64 ? 64 : 128);
  const int avail = DU_SMEM_TOTAL - (int)sizeof(DecCtl) - 5 * *q_rows_pad * 128;
  int n = avail / DU_SLOT;
  *nslot = n > DU_MAX_SLOT ? DU_MAX_SLOT : n;
}

int launch_splitkv_umma(const CUtensorMap &mk, const CUtensorMap &mv, const SplitKVParams &p, bool out_is_f32,
                        cudaStream_t st, bool dependent) {
  constexpr size_t smem = 1024 + DU_SMEM_TOTAL;
  // once per device; the step is idempotent, so an atomic flag is all that concurrent host threads need
  static std::atomic<int> configured[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
  if (dev < 0 || !configured[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(splitkv_umma_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        cudaFuncSetAttribute(splitkv_umma_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return 3;
    if (dev >= 0) configured[dev].store(1, std::memory_order_release);
  }
  if (out_is_f32)
    launch_kernel(splitkv_umma_kernel<float>, dim3(p.G), dim3(DU_THREADS), smem, st, dependent, mk, mv, p);
  else
    launch_kernel(splitkv_umma_kernel<uint16_t>, dim3(p.G), dim3(DU_THREADS), smem, st, dependent, mk, mv, p);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace qwb
