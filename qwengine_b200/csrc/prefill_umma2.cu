// Causal chunked-prefill attention, CTA-pair version (tcgen05 cta_group::2).
//
// Two CTAs of a cluster (two SMs) take the same 128 query rows of two query heads that share a
// KV head, so every K/V tile is needed by both.  With cta_group::2 one tcgen05.mma spans the pair:
// M = 256 (128 rows per CTA, each CTA's own Q / P and its own TMEM accumulators) and the B operand
// is split across the pair's shared memories -- for S = Q K^T each CTA stages 64 of the tile's 128
// keys, for O += P V each CTA stages 128 of the 256 value channels.  Per CTA and KV tile that is
// 64 KB instead of 128 KB: half the L2->SM traffic, half the shared-memory read bandwidth per MMA,
// and the same 128 KB ring holds two tiles of look-ahead instead of one.
//
// TMEM map: O | S0 | S1, P over S as bf16 hi + lo.
//
// The kernel is persistent: the grid is as many CTA pairs as the device holds at once and each
// pair walks a static list of items (sequence, query tile, head pair) dealt out heaviest first in
// rounds of alternating direction.  KV tiles are numbered through all items of a pair; the MMA
// stream is Q K_g^T, P V_{g-1}, Q K_{g+1}^T, ... straight through item boundaries and the K/V ring
// is filled in that same order.
//
// Warp roles: a control warpgroup (warp 0 = TMA producer, warp 1 = TMEM owner and -- in the leader
// CTA only -- MMA issuer, warp 2 = TMA store of finished output tiles, warp 3 idle) that gives
// registers away with setmaxnreg, and four softmax warpgroups (thread = query row x 32-key group)
// that take them.  The softmax warps also rotate the next item's Q tile in shared memory (RoPE,
// hi + lo sub-tiles) after delivering the current item's last P, and finish the PREVIOUS item
// (O out of TMEM, 1/l, sigmoid gate) after delivering the next item's first P, so the tensor pipe
// has work across the boundary.  The epilogue tile of an item lives in four ring slots behind the
// item's last V tile: the producer loads the gate rows there by TMA, the softmax warps overwrite
// them with the gated output, the store warp sends them out by TMA and returns the slots.
// Every wait is bounded; on expiry the CTA raises an abort flag and writes a status word.
//
// Cross-CTA signalling: the leader's barriers collect both CTAs.  TMA loads of either CTA complete
// on the leader's slot barrier (cp.async.bulk.tensor with .cta_group::2, no multicast); softmax
// warps of the peer arrive (one arrival per warp) on the leader's q_ready / p_full / o_drained
// barriers through mapa'd addresses; the MMA thread publishes "S_g complete" and "P_g V_g retired"
// to both CTAs with one tcgen05.commit each (arrival multicast to the same barrier in both CTAs).
// Those two signals also free the ring: the producer remembers the last occupant of each slot
// group and waits for exactly the completion that releases it (s_full for a K group, o_done for a
// V group, e_free for an epilogue tile), every completion observed in tile order because a parity
// wait cannot tell two phases apart.
//
#include "prefill_umma.cuh"

#include <atomic>
#include <cstring>

#include "umma_common.cuh"

namespace qwb {

namespace {

constexpr int P2_BM = 128;                 // query rows per CTA (256 per pair)
constexpr int P2_BN = 128;                 // keys per KV tile
constexpr int P2_SLOT = 16384;             // ring slot bytes per CTA
constexpr int P2_NSLOT = 8;                // ring slots: 2 K + 2 V per tile -> two tiles of look-ahead
constexpr int P2_QBYTES = 5 * P2_SLOT;     // four 64-channel Q sub-tiles + the rotary "lo" sub-tile
constexpr int P2_NWG = 4;
constexpr int P2_SM_THREADS = P2_NWG * 128;
constexpr int P2_CTL_THREADS = 128;         // control warpgroup: TMA producer, MMA issuer, output-store warp, one idle warp
constexpr int P2_THREADS = P2_CTL_THREADS + P2_SM_THREADS;
constexpr int P2_CTL_REGS = 64, P2_SM_REGS = 104;  // after setmaxnreg: 128 x 64 + 512 x 104 = the 640 x 96 registers the block starts with

struct PairCtl {
  uint64_t q_full, q_ready, o_drained, s_full[2], p_full[2], o_done[2];
  uint64_t slot_full[P2_NSLOT];
  uint64_t fix_bar;              // CTA-local: the ragged last V tile lands here first
  uint64_t g_full, e_ready, e_free;  // CTA-local: gate tile landed; output tile written; its ring slots are free again
  uint32_t tmem_base;
  volatile int abort_flag;
  uint32_t skip;                 // leader: the launch had already failed when this pair started
  float mxbuf[2][P2_NWG][128];
  float lbuf[P2_NWG][128];
  float mbuf[128];
  volatile int e_slot[2];       // by item parity: first ring slot the producer used for the item's epilogue tile
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
// Arrival on a barrier that may live in the other CTA.  The cluster-scope release form orders
// this thread's earlier generic-memory writes for the other CTA and costs about a thousand
// cycles; it is used once, after the RoPE prologue has rewritten Q in shared memory.  The per-tile
// "P is ready" arrivals publish tensor-memory data only, which tcgen05.wait::st and
// tcgen05.fence::before_thread_sync already order, so they use the plain form.
__device__ __forceinline__ void remote_arrive_release(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void remote_arrive(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void remote_arrive_expect_tx(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes)
               : "memory");
}
// Wait with cluster-scope acquire: the arrivals it observes may come from the other CTA.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool wait_cluster_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
  for (int i = 0; i < 32; ++i)
    if (mbar_try_wait_cluster(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 0; i < (1u << 30); ++i) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((i & 7) == 7) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > WAIT_LIMIT_NS) return false;
    }
  }
  return false;
}
// 2-D TMA load whose completion bytes are counted on a barrier that may live in the pair's other
// CTA (.cta_group::2); plain tile mode, no multicast.
__device__ __forceinline__ void tma_load_2d_pair(void *dst, const CUtensorMap *map, uint32_t bar_cluster_addr, int c0,
                                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
// 2-D tiled TMA store of one shared-memory box (same 64-element x 128-row, 128-byte-swizzled layout the loads
// produce) to global memory; completion is tracked by the issuing thread's bulk-async group.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, const void *src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(src)), "r"(c0), "r"(c1)
               : "memory");
}
// Asks the copy engine to bring one box of a tiled tensor into L2 (no shared-memory destination, no barrier).
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap *map, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(ncols) : "memory");
}
// Completion of all MMAs issued so far, signalled on the barrier at this shared-memory offset
// in BOTH CTAs of the pair (a commit is not a load: nothing is copied, two barriers get an arrival).
__device__ __forceinline__ void umma_commit_both(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3)
               : "memory");
}
__device__ __forceinline__ void umma_ss_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}

// One work item of a CTA pair: 128 query rows (one query tile) of the two heads `head` of the pair.
struct PairItem {
  int s, head, kvh;      // sequence, this CTA's query head, their KV head
  int q0, rows_valid;    // first row of the tile within the chunk, rows that exist
  int pos;               // tokens cached before the chunk
  int kv_len, nt;        // keys the tile's last row sees, and KV tiles that cover them
  long long crow;        // first cache row of the sequence (contiguous layout)
  bool ragged;           // the last KV tile is only partly inside the sequence
};

// The k-th item of cluster `cluster` out of `n_clusters`.  Items are ordered heaviest first (latest query
// tile of every sequence and head pair, then the one before, ...) and dealt out in rounds whose direction
// alternates, so that every cluster's items add up to about the same number of KV tiles without any
// run-time scheduling: the assignment is static and the result bit-stable.
__device__ __forceinline__ bool pair_item(const PrefillParams &p, int k, int cluster, int n_clusters, uint32_t rank,
                                          PairItem &w) {
  const int pairs = p.q_heads / 2;
  const long long per_level = (long long)p.n_seq * pairs;
  const long long n_items = per_level * p.n_qtiles;
  const long long e = (long long)k * n_clusters + ((k & 1) ? n_clusters - 1 - cluster : cluster);
  if (e >= n_items) return false;
  const int lvl = (int)(e / per_level), r = (int)(e % per_level);
  w.s = r / pairs;
  const int qt = p.n_qtiles - 1 - lvl;
  w.head = (r % pairs) * 2 + (int)rank;
  w.kvh = w.head / GROUP;
  w.crow = p.cache_row ? p.cache_row[w.s] : 0;
  w.q0 = qt * P2_BM;
  w.rows_valid = min(P2_BM, p.n_new - w.q0);
  w.pos = p.pos[w.s];
  w.kv_len = w.pos + w.q0 + w.rows_valid;
  w.nt = (w.kv_len + P2_BN - 1) / P2_BN;
  w.ragged = (w.kv_len % P2_BN) != 0;
  return true;
}

// First ring slot of the epilogue tile of the pair's k-th item, whose last KV tile is the pair's `tiles_through`-th.
// The ring stream is  K_0 | K_1 V_0 | K_2 V_1 | ...  and an item's epilogue tile (two groups of two slots) follows
// the V group of the item's last tile: before it the ring has seen one K and one V group per KV tile so far, the
// K group of the next item's first tile if there is a next item, and two groups per earlier epilogue tile.  Its
// four slots follow each other modulo the ring size.
__device__ __forceinline__ int epi_tile_slot(int tiles_through, int k, bool has_next) {
  return (4 * (tiles_through + k) + (has_next ? 2 : 0)) % P2_NSLOT;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P2_THREADS, 1)
prefill_umma_pair_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                         const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapG,
                         const __grid_constant__ CUtensorMap mapO, const __grid_constant__ PrefillParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *q_smem = smem;
  uint8_t *ring = smem + P2_QBYTES;
  PairCtl *ctl = reinterpret_cast<PairCtl *>(ring + P2_NSLOT * P2_SLOT);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader (issues the MMAs), 1 = peer
  const bool leader = rank == 0;
  const int cluster = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  // a kernel launched behind this one as a programmatic dependent (the append kernel of the next chunk is) may
  // become resident now; it waits for this grid's completion before it touches memory
  grid_dep_launch_dependents();

  if (tid == 0) {
    mbar_init(&ctl->q_full, 1);
    // the softmax warps signal once per warp (a lane's tcgen05 / proxy fence, __syncwarp, then lane 0 arrives): a
    // thousand arrivals per signal on one barrier, half of them from the other CTA, cost more than the work between them
    mbar_init(&ctl->q_ready, 2 * (P2_SM_THREADS / 32));
    mbar_init(&ctl->o_drained, 2 * (P2_SM_THREADS / 32));
    for (int i = 0; i < 2; ++i) { mbar_init(&ctl->s_full[i], 1); mbar_init(&ctl->p_full[i], 2 * (P2_SM_THREADS / 32)); }
    mbar_init(&ctl->o_done[0], 1);
    mbar_init(&ctl->o_done[1], 1);
    for (int i = 0; i < P2_NSLOT; ++i) mbar_init(&ctl->slot_full[i], 2);
    mbar_init(&ctl->fix_bar, 1);
    mbar_init(&ctl->g_full, 1);
    mbar_init(&ctl->e_ready, P2_SM_THREADS / 32);
    mbar_init(&ctl->e_free, 1);
    ctl->abort_flag = 0;
    ctl->skip = (p.status && *reinterpret_cast<volatile int *>(p.status) != 0) ? 1u : 0u;
    fence_barrier_init();
    prefetch_tensormap(&mapQ);
    prefetch_tensormap(&mapK);
    prefetch_tensormap(&mapV);
    if (p.tma_epi) { prefetch_tensormap(&mapG); prefetch_tensormap(&mapO); }
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc_pair(&ctl->tmem_base, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // both CTAs: barriers initialised, TMEM allocated
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  volatile int *abort_flag = &ctl->abort_flag;
  // A launch that has already failed somewhere does not keep the GPU busy with further timeouts:
  // both CTAs follow the leader's reading of the status word, taken before the cluster barrier.
  uint32_t skip;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(skip) : "r"(map_to_cta(smem_u32(&ctl->skip), 0)) : "memory");
  const bool run = skip == 0;

  // The pair is persistent: it walks its items one after the other, and KV tiles are numbered through all of
  // them (g = 0, 1, 2, ...).  Tile g uses S / P buffer g & 1 and barrier phase (g >> 1) & 1.  The tensor pipe is
  // fed  Q K_g^T, P V_{g-1}, Q K_{g+1}^T, P V_g, ...  straight through the item boundaries: the first Q K^T of the
  // next item runs before the last P V of this one, so the softmax warps can turn its scores into P while that
  // last P V and the read-out of O are under way; only the next item's first P V waits, for O to have been read
  // (o_drained).  The next item's Q tile is loaded as soon as this item's last Q K^T has retired and rotated by
  // the softmax warps right after they have delivered this item's last P.  The ring follows the same order:
  // ... K_last, V_last-1 | K'_0, V_last, E | K'_1, V'_0 | K'_2, ...
  //
  // E is the item's epilogue tile (bf16 output, p.tma_epi): four ring slots, one per 64-channel group, that the
  // producer fills with the item's gate tile by TMA; the softmax warps read their row's gate values from there,
  // overwrite them with the gated output, and an otherwise idle warp of the control warpgroup sends the four
  // slots to global memory by TMA store and returns them to the ring.  Gate loads and output stores are then
  // whole 128-byte lines moved by the copy engine instead of 32 scattered lines per warp instruction, which
  // took longer than the rest of an item's end together.

  // Registers: the block is five warpgroups that start with 96 registers per thread.  The control warpgroup
  // (producer, MMA issuer, two idle warps) gives a third of its share back and the four softmax warpgroups take
  // it, so the softmax loop with its 64 values of S and P per thread does not spill.  Every warp of a
  // warpgroup runs the same setmaxnreg, first thing in its branch: the compiler raises or lowers the register
  // budget only for code that the instruction dominates.
  if (warp == 0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(P2_CTL_REGS));
    // =============================== TMA producer (each CTA loads its halves) ================
    // The whole warp walks the stream (a ragged last V tile needs all lanes, see below); one elected lane
    // issues the copies.  The ring is used in groups of two slots (one K or V half-tile of this CTA); a group
    // may be refilled once the MMAs that read its last contents have retired, which the MMA thread publishes
    // per tile: s_full[t & 1] for the K of tile t, o_done[t & 1] for its V.  The last occupants of the four
    // groups are remembered here, oldest first, so the order of the stream may change at item boundaries.
    // Every completion is waited for in tile order, which a parity wait needs: it cannot tell apart phases
    // that lie two apart.
    bool ok = run;
    uint32_t grp = 0;   // ring groups filled so far
    uint32_t fixn = 0;  // ragged V slots handled so far (phase of fix_bar)
    int g = 0;          // KV tiles started so far, over all items
    int occ_kind[4] = {0, 0, 0, 0}, occ_tile[4] = {0, 0, 0, 0};  // 0 empty, 1 = K of tile, 2 = V of tile, 3 = epilogue tile of item; [0] is reused next
    PairItem w, pv;     // current item; item of the tile whose V is still to be loaded
    int pv_j = -1;      // that tile's index within its item (-1: none pending)
    auto producer_fail = [&]() {
      if (lane == 0) { if (!*abort_flag && p.status) *p.status = DEV_ERR_EMPTY_WAIT; *abort_flag = 1; }
      ok = false;
    };
    // Claims the next ring group for (kind, tile); returns its first slot, or -1 after a failed wait.
    auto next_group = [&](int kind, int tile) -> int {
      bool got = true;
      if (occ_kind[0] == 1) got = wait_or_abort(&ctl->s_full[occ_tile[0] & 1], (occ_tile[0] >> 1) & 1, abort_flag);
      else if (occ_kind[0] == 2) got = wait_or_abort(&ctl->o_done[occ_tile[0] & 1], (occ_tile[0] >> 1) & 1, abort_flag);
      else if (occ_kind[0] == 3) got = wait_or_abort(&ctl->e_free, occ_tile[0] & 1, abort_flag);  // "tile" = the pair's item count
      if (!__all_sync(0xffffffffu, got)) { producer_fail(); return -1; }
#pragma unroll
      for (int i = 0; i < 3; ++i) { occ_kind[i] = occ_kind[i + 1]; occ_tile[i] = occ_tile[i + 1]; }
      occ_kind[3] = kind;
      occ_tile[3] = tile;
      const int sl = (int)((2 * grp) % P2_NSLOT);
      ++grp;
      return sl;
    };
    // V of (item v, tile j), global tile t: this CTA's 128 channels, two slots of 64 keys
    auto load_v = [&](const PairItem &v, int j, int t) {
      const int sl0 = next_group(2, t);
      if (sl0 < 0) return;
      const bool ragged_tile = v.ragged && j == v.nt - 1;
      for (int gg = 0; gg < 2 && ok; ++gg) {
        const int sl = sl0 + gg;
        const int vrow = (int)cache_row_at(p.pages, v.crow, v.s, j * P2_BN + gg * 64);
        if (!ragged_tile) {
          if (elect_one()) {
            const uint32_t bar = map_to_cta(smem_u32(&ctl->slot_full[sl]), 0);
            remote_arrive_expect_tx(bar, P2_SLOT);
#pragma unroll
            for (int a = 0; a < 2; ++a)
              tma_load_2d_pair(ring + sl * P2_SLOT + a * 8192, &mapV, bar, v.kvh * HEAD_DIM + (int)rank * 128 + a * 64, vrow);
          }
          __syncwarp();
          continue;
        }
        // Ragged last tile: rows of V past the sequence's end may hold anything (even NaN bit patterns) and
        // P is an exact zero there, but 0 * NaN is NaN.  The tile is therefore loaded on a CTA-local barrier,
        // its rows past the end are cleared by the whole warp, and only then is the slot announced on the
        // leader's barrier (a plain arrival: the bytes are in).
        if (elect_one()) {
          mbar_expect_tx(&ctl->fix_bar, P2_SLOT);
#pragma unroll
          for (int a = 0; a < 2; ++a)
            tma_load_2d(ring + sl * P2_SLOT + a * 8192, &mapV, &ctl->fix_bar, v.kvh * HEAD_DIM + (int)rank * 128 + a * 64, vrow);
        }
        __syncwarp();
        if (!__all_sync(0xffffffffu, wait_or_abort(&ctl->fix_bar, fixn & 1, abort_flag))) { producer_fail(); break; }
        ++fixn;
        const int valid = max(0, v.kv_len - (j * P2_BN + gg * 64));  // rows of this slot inside the sequence
        for (int idx = lane; idx < 64 * 16; idx += 32) {
          const int kr = idx >> 4, c16 = idx & 15;  // key row, 16-byte column over the two 64-channel atoms
          if (kr >= valid)
            *reinterpret_cast<uint4 *>(ring + sl * P2_SLOT + (c16 >> 3) * 8192 + kr * 128 + (((c16 & 7) ^ (kr & 7)) << 4)) =
                make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) remote_arrive_release(map_to_cta(smem_u32(&ctl->slot_full[sl]), 0));
      }
    };
    // Epilogue tile of the pair's (k)-th item v: two ring groups; the gate tile goes into them when there is a gate.
    auto load_e = [&](const PairItem &v, int k) {
      if (!p.tma_epi) return;
      for (int h2 = 0; h2 < 2 && ok; ++h2) {
        const int sl0 = next_group(3, k);
        if (sl0 < 0) return;
        if (h2 == 0 && lane == 0) ctl->e_slot[k & 1] = sl0;   // read behind g_full, which orders it
        // g_full tells the softmax warps that the tile's slots are theirs: with a gate it completes when the
        // gate tile has landed, without one it is a plain arrival once both groups have been claimed
        if (elect_one()) {
          if (p.gate) {
            if (h2 == 0) mbar_expect_tx(&ctl->g_full, 4 * P2_SLOT);
            const int qrow = v.s * p.n_new + v.q0;
#pragma unroll
            for (int i = 0; i < 2; ++i)
              tma_load_2d(ring + (sl0 + i) * P2_SLOT, &mapG, &ctl->g_full, v.head * HEAD_DIM + (2 * h2 + i) * 64, qrow);
          } else if (h2 == 1) {
            mbar_arrive(&ctl->g_full);
          }
        }
        __syncwarp();
      }
    };
    bool pv_last = false;  // the pending tile is the last of its item: its epilogue tile follows its V
    int pv_k = 0;          // the pending tile's item
    for (int k = 0; ok && pair_item(p, k, cluster, n_clusters, rank, w); ++k) {
      // this item's Q tile: the Q region is free once every Q K^T of the previous item has completed
      if (k > 0 && !__all_sync(0xffffffffu, wait_or_abort(&ctl->s_full[(g - 1) & 1], ((g - 1) >> 1) & 1, abort_flag))) {
        producer_fail();
        break;
      }
      if (elect_one()) {
        mbar_expect_tx(&ctl->q_full, 4 * P2_SLOT);
        const int qrow = w.s * p.n_new + w.q0;
#pragma unroll
        for (int c = 0; c < 4; ++c) tma_load_2d(q_smem + c * P2_SLOT, &mapQ, &ctl->q_full, w.head * HEAD_DIM + c * 64, qrow);
      }
      __syncwarp();
      // The next item's Q tile cannot be loaded before this item's last Q K^T has retired (one Q region), and it
      // comes from HBM (q is read once): asking it into L2 now shortens that load, which sits on the path
      // between two items, to an L2 hit.
      {
        PairItem wn;
        if (pair_item(p, k + 1, cluster, n_clusters, rank, wn) && elect_one()) {
          const int qrow = wn.s * p.n_new + wn.q0;
#pragma unroll
          for (int c = 0; c < 4; ++c) tma_prefetch_l2_2d(&mapQ, wn.head * HEAD_DIM + c * 64, qrow);
        }
        __syncwarp();
      }
      for (int j = 0; j < w.nt && ok; ++j, ++g) {
        // K_g: this CTA's 64 keys, channels [128 i, 128 i + 128) per slot
        const int sl0 = next_group(1, g);
        if (sl0 < 0) break;
        if (elect_one()) {
          const int krow = (int)cache_row_at(p.pages, w.crow, w.s, j * P2_BN + (int)rank * 64);
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const uint32_t bar = map_to_cta(smem_u32(&ctl->slot_full[sl0 + i]), 0);
            remote_arrive_expect_tx(bar, P2_SLOT);
#pragma unroll
            for (int a = 0; a < 2; ++a)
              tma_load_2d_pair(ring + (sl0 + i) * P2_SLOT + a * 8192, &mapK, bar, w.kvh * HEAD_DIM + (2 * i + a) * 64, krow);
          }
        }
        __syncwarp();
        if (pv_j >= 0) {   // V of the tile before (the previous item's last one when j = 0), then that item's epilogue tile
          load_v(pv, pv_j, g - 1);
          if (ok && pv_last) load_e(pv, pv_k);
        }
        pv = w;
        pv_j = j;
        pv_last = j == w.nt - 1;
        pv_k = k;
      }
    }
    if (ok && pv_j >= 0) {
      load_v(pv, pv_j, g - 1);
      if (ok && pv_last) load_e(pv, pv_k);
    }
  } else if (warp == 1) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(P2_CTL_REGS));
    // =============================== MMA issuer (one thread of the leader CTA) ===============
    // A tcgen05.mma of this shape occupies the tensor pipe for only ~64 cycles, so the issuing
    // thread must not spend longer than that per instruction: descriptors are built once and
    // advanced by adding the (16-byte unit) offset to their start-address field.
    if (run && leader && elect_one()) {
      const uint32_t idesc_qk = make_idesc(256, 128, 1, 1, 0, 0);
      const uint32_t idesc_pv = make_idesc(256, 256, 1, 1, 0, 1);
      const uint64_t qdesc0 = smem_desc(smem_u32(q_smem), 16, 1024);
      const uint64_t kdesc0 = smem_desc(smem_u32(ring), 16, 1024);
      const uint64_t vdesc0 = smem_desc(smem_u32(ring), 8192, 1024);  // channel atoms 8 KB apart, 8-key groups 1 KB
      bool ok = true;
      auto fail = [&](int code) {
        if (!*abort_flag && p.status) *p.status = code;
        *abort_flag = 1;
        ok = false;
      };
      uint32_t it = 0;           // ring slots passed so far (K, V and epilogue tiles)
      uint32_t slot_phase = 0;   // bit sl: parity of the next completion of slot_full[sl] (epilogue tiles do not complete it)
      int g = 0;                 // KV tiles issued so far, over all items
      bool pend = false;         // tile g - 1 still lacks its P V
      bool pend_first = false;   // ... and it is the first tile of its item (O starts from zero)
      int pend_item = 0;         // ... of the pair's pend_item-th item
      // O (+)= P_t V_t for global tile t
      auto issue_pv = [&](int t, bool first, int item_k) {
        if (!wait_cluster_or_abort(&ctl->p_full[t & 1], (t >> 1) & 1, abort_flag)) { fail(DEV_ERR_SOFTMAX_WAIT); return; }
        // the first P V of an item overwrites O: the softmax warps must have read the previous item's O out
        if (first && item_k > 0 && !wait_cluster_or_abort(&ctl->o_drained, (item_k - 1) & 1, abort_flag)) {
          fail(DEV_ERR_SOFTMAX_WAIT);
          return;
        }
        tc_fence_after();
        const uint32_t a_p = tmem + ((t & 1) ? TMEM_S1 : TMEM_S0);
#pragma unroll
        for (int gg = 0; gg < 2; ++gg, ++it) {
          const int sl = it % P2_NSLOT;
          if (!ok || !wait_cluster_or_abort(&ctl->slot_full[sl], (slot_phase >> sl) & 1, abort_flag)) { if (ok) fail(DEV_ERR_MMA_WAIT); continue; }
          slot_phase ^= 1u << sl;
          tc_fence_after();
          const uint64_t vd = vdesc0 + (uint64_t)(sl * (P2_SLOT >> 4));
#pragma unroll
          for (int k = 0; k < 4; ++k) {  // 16 keys per step
            umma_ts_pair(tmem + TMEM_O, a_p + (gg * 4 + k) * 8, vd + (uint64_t)((k * 2048) >> 4), idesc_pv,
                         !(first && gg == 0 && k == 0));
            if (!p.fast_p)
              umma_ts_pair(tmem + TMEM_O, a_p + 64 + (gg * 4 + k) * 8, vd + (uint64_t)((k * 2048) >> 4), idesc_pv, 1);
          }
        }
        if (ok) umma_commit_both(&ctl->o_done[t & 1]);  // O updated; the tile's V slots are free
      };
      bool pend_last = false;    // ... and the last of its item: that item's epilogue tile follows its V in the ring
      PairItem w;
      for (int k = 0; ok && pair_item(p, k, cluster, n_clusters, rank, w); ++k) {
        if (!wait_cluster_or_abort(&ctl->q_ready, k & 1, abort_flag)) { fail(DEV_ERR_MMA_WAIT); break; }
        tc_fence_after();
        for (int j = 0; j < w.nt && ok; ++j, ++g) {
          // ---- S[g & 1] = Q K_j^T for both CTAs' rows ----
          const uint32_t d_s = tmem + ((g & 1) ? TMEM_S1 : TMEM_S0);
#pragma unroll
          for (int i = 0; i < 2; ++i, ++it) {
            const int sl = it % P2_NSLOT;
            if (!ok || !wait_cluster_or_abort(&ctl->slot_full[sl], (slot_phase >> sl) & 1, abort_flag)) { if (ok) fail(DEV_ERR_MMA_WAIT); continue; }
            slot_phase ^= 1u << sl;
            tc_fence_after();
            const uint64_t kd = kdesc0 + (uint64_t)(sl * (P2_SLOT >> 4));
#pragma unroll
            for (int a = 0; a < 2; ++a) {
              const int c = 2 * i + a;  // 64-channel sub-tile
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                umma_ss_pair(d_s, qdesc0 + (uint64_t)((c * P2_SLOT + kk * 32) >> 4),
                             kd + (uint64_t)((a * 8192 + kk * 32) >> 4), idesc_qk, !(c == 0 && kk == 0));
              if (c == 0 && p.do_rope) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                  umma_ss_pair(d_s, qdesc0 + (uint64_t)((4 * P2_SLOT + kk * 32) >> 4), kd + (uint64_t)((kk * 32) >> 4),
                               idesc_qk, 1);
              }
            }
          }
          if (!ok) break;
          // one completion point for the whole S tile, seen by the softmax warps (S is ready) and
          // by both producers (the tile's K slots are free)
          umma_commit_both(&ctl->s_full[g & 1]);
          // ---- O (+)= P V of the tile before; at j = 0 that is the previous item's last tile ----
          if (pend) {
            issue_pv(g - 1, pend_first, pend_item);
            if (pend_last && p.tma_epi) it += 4;  // that item's epilogue tile sits in the ring here
          }
          pend = true;
          pend_first = j == 0;
          pend_item = k;
          pend_last = j == w.nt - 1;
        }
      }
      if (ok && pend) issue_pv(g - 1, pend_first, pend_item);
    }
  } else if (warp < P2_CTL_THREADS / 32) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(P2_CTL_REGS));
    // =============================== output store (warp 2; warp 3 idles) =====================
    // Per item: once the softmax warps have written the gated bf16 output into the epilogue tile, send its four
    // 64-channel slots to global memory by TMA store, wait until the copy engine has read them, and return the
    // slots to the ring.  A tile that reaches past the chunk's end was stored row by row by the softmax warps
    // (a TMA store would overwrite the rows that follow): its slots are returned as they are.
    if (warp == 2 && run && p.tma_epi) {
      PairItem w, wn;
      int G = 0;
      bool have = pair_item(p, 0, cluster, n_clusters, rank, w);
      for (int k = 0; have; ++k) {
        const bool has_next = pair_item(p, k + 1, cluster, n_clusters, rank, wn);
        if (!__all_sync(0xffffffffu, wait_or_abort(&ctl->e_ready, k & 1, abort_flag))) break;
        if (elect_one()) {
          if (w.rows_valid == P2_BM) {
            const int base = epi_tile_slot(G + w.nt, k, has_next);
            const int qrow = w.s * p.n_new + w.q0;
#pragma unroll
            for (int c = 0; c < 4; ++c)
              tma_store_2d(&mapO, ring + (size_t)((base + c) % P2_NSLOT) * P2_SLOT, w.head * HEAD_DIM + c * 64, qrow);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          }
          mbar_arrive(&ctl->e_free);
        }
        __syncwarp();
        G += w.nt;
        have = has_next;
        w = wn;
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // every store has landed before the CTA may exit
    }
  } else if (run) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(P2_SM_REGS));
    // ============ softmax / correction / epilogue: thread = (query row, 32-key column group) =========
    const int wg = (warp - P2_CTL_THREADS / 32) >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t q_ready_addr = map_to_cta(smem_u32(&ctl->q_ready), 0);
    const uint32_t o_drained_addr = map_to_cta(smem_u32(&ctl->o_drained), 0);
    const uint32_t p_full_addr[2] = {map_to_cta(smem_u32(&ctl->p_full[0]), 0), map_to_cta(smem_u32(&ctl->p_full[1]), 0)};
    bool ok = true;
    // RoPE of item w's Q tile (already in shared memory by TMA), in place: hi + lo sub-tiles for the 64
    // rotary channels; then the tile is handed to the MMA thread.  k = the pair's k-th item.
    auto stage_q = [&](const PairItem &w, int k) {
      if (ok) ok = wait_or_abort(&ctl->q_full, k & 1, abort_flag);
      if (ok && p.do_rope) {
        const size_t trow = (size_t)w.s * p.n_new + w.q0 + row;
        const bool live = row < w.rows_valid;
        const int rope_pos = (p.q_pos ? p.q_pos[w.s] : w.pos) + w.q0 + row;
        uint8_t *base = q_smem + row * 128;
        uint8_t *lo_base = q_smem + 4 * P2_SLOT + row * 128;
        const int c = wg;
        uint4 *px = reinterpret_cast<uint4 *>(base + ((c ^ (row & 7)) << 4));
        uint4 *py = reinterpret_cast<uint4 *>(base + (((c + 4) ^ (row & 7)) << 4));
        const uint4 xv = *px, yv = *py;
        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, yw[4] = {yv.x, yv.y, yv.z, yv.w};
        uint32_t xh[4], yh[4], xl[4], yl[4];
#pragma unroll
        for (int w2 = 0; w2 < 4; ++w2) {
          float xr[2], yr[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int i = c * 8 + w2 * 2 + e;
            const float x = e ? bf16hi(xw[w2]) : bf16lo(xw[w2]);
            const float y = e ? bf16hi(yw[w2]) : bf16lo(yw[w2]);
            const int pz = (p.mpos && live) ? p.mpos[trow * 3 + mrope_component(i)] : rope_pos;
            float cs, sn;
            rope_sincos_reduced(pz, p.rope.inv_freq[i], cs, sn);
            xr[e] = x * cs - y * sn;
            yr[e] = x * sn + y * cs;
          }
          xh[w2] = pack_bf16(xr[0], xr[1]);
          yh[w2] = pack_bf16(yr[0], yr[1]);
          xl[w2] = pack_bf16(xr[0] - bf16lo(xh[w2]), xr[1] - bf16hi(xh[w2]));
          yl[w2] = pack_bf16(yr[0] - bf16lo(yh[w2]), yr[1] - bf16hi(yh[w2]));
        }
        *px = make_uint4(xh[0], xh[1], xh[2], xh[3]);
        *py = make_uint4(yh[0], yh[1], yh[2], yh[3]);
        *reinterpret_cast<uint4 *>(lo_base + ((c ^ (row & 7)) << 4)) = make_uint4(xl[0], xl[1], xl[2], xl[3]);
        *reinterpret_cast<uint4 *>(lo_base + (((c + 4) ^ (row & 7)) << 4)) = make_uint4(yl[0], yl[1], yl[2], yl[3]);
      }
      fence_proxy_async();   // each lane publishes its rows to the tensor core's proxy; then one arrival per warp
      __syncwarp();
      if (lane == 0) remote_arrive_release(q_ready_addr);
    };

    int o_seen = 0;  // P V completions observed so far, in order (tile t: o_done[t & 1], phase t / 2)
    auto wait_pv_done = [&](int upto) {
      while (ok && o_seen <= upto) {
        ok = wait_or_abort(&ctl->o_done[o_seen & 1], (o_seen >> 1) & 1, abort_flag);
        ++o_seen;
      }
    };
    // End of an item: 1/l, gate, store.  O is read out of tensor memory, a row per thread, 64 channels per
    // warpgroup.  With an epilogue tile in the ring (bf16 output, a full tile of 128 rows) the row's gate values
    // are read from shared memory and the gated output is written over them for the TMA store; otherwise
    // (fp32 output, or a tile that reaches past the chunk's last row) gate and output move by plain loads and
    // stores, one 128-byte run per thread.
    // kf: the finished item (the pair's kf-th); tiles_through: KV tiles of the pair up to and including its last.
    // The item's row sums and maxima were left in lbuf / mbuf when the softmax warps moved on to the next item.
    auto epilogue = [&](int kf, int tiles_through, bool has_next) {
      PairItem f;
      pair_item(p, kf, cluster, n_clusters, rank, f);
      const bool live_row = row < f.rows_valid;
      const bool via_tile = p.tma_epi && f.rows_valid == P2_BM;
      const size_t grow = ((size_t)f.s * p.n_new + f.q0 + row) * p.q_heads + f.head;
      const size_t elem0 = grow * HEAD_DIM + wg * 64;
      const uint4 *gp = reinterpret_cast<const uint4 *>(p.gate + elem0);
      if (!via_tile && p.gate && live_row) asm volatile("prefetch.global.L2 [%0];" ::"l"(gp));
      // this warpgroup's slot of the epilogue tile
      uint8_t *e_row = ring + (size_t)((epi_tile_slot(tiles_through, kf, has_next) + wg) % P2_NSLOT) * P2_SLOT + row * 128;
      wait_pv_done(tiles_through - 1);
      if (ok && p.tma_epi) ok = wait_or_abort(&ctl->g_full, kf & 1, abort_flag);  // the epilogue tile is ours (and holds the gate)
      asm volatile("bar.sync 1, %0;" ::"n"(P2_SM_THREADS) : "memory");
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0 && !*abort_flag && p.status) *p.status = DEV_ERR_SOFTMAX_WAIT;
        *abort_flag = 1;
        ok = false;
        return;
      }
      tc_fence_after();
      float l_tot = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < P2_NWG; ++w2) l_tot += ctl->lbuf[w2][row];
      const float m_row = ctl->mbuf[row];
      // lbuf / mbuf are single buffers: nobody may run on to the end of the next item (a one-tile item ends right
      // after this epilogue) and overwrite them before every thread has read its row
      asm volatile("bar.sync 1, %0;" ::"n"(P2_SM_THREADS) : "memory");
      const float inv = 1.f / l_tot;
      const uint32_t t_o = tmem + lane_sel + TMEM_O + wg * 64;
      // both halves of the row's 64 channels go to registers first: the accumulator is then free for the next
      // item's first P V while the gate arithmetic below runs
      uint32_t orow[2][32];
      tmem_ld32(t_o, orow[0]);
      tmem_ld32(t_o + 32, orow[1]);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) remote_arrive(o_drained_addr);
      // the producer's ring bookkeeping and the arithmetic above must agree on where the tile is
      if (p.tma_epi && ctl->e_slot[kf & 1] != epi_tile_slot(tiles_through, kf, has_next)) {
        if (!*abort_flag && p.status) *p.status = DEV_ERR_RING;
        *abort_flag = 1;
        ok = false;
        return;
      }
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        if (via_tile || live_row) {
#pragma unroll
          for (int v8 = 0; v8 < 4; ++v8) {
            float o8[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) o8[e] = __uint_as_float(orow[c][v8 * 8 + e]) * inv;
            if (p.gate) {
              const uint4 gv = via_tile ? *reinterpret_cast<const uint4 *>(e_row + (((c * 4 + v8) ^ (row & 7)) << 4)) : __ldg(gp + c * 4 + v8);
              const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                o8[2 * e] *= sigmoid_tanh(bf16lo(gw[e]));
                o8[2 * e + 1] *= sigmoid_tanh(bf16hi(gw[e]));
              }
            }
            if (via_tile)
              *reinterpret_cast<uint4 *>(e_row + (((c * 4 + v8) ^ (row & 7)) << 4)) =
                  make_uint4(pack_bf16(o8[0], o8[1]), pack_bf16(o8[2], o8[3]), pack_bf16(o8[4], o8[5]), pack_bf16(o8[6], o8[7]));
            else if (p.out_is_f32) store8<float>(reinterpret_cast<float *>(p.out) + elem0 + c * 32 + v8 * 8, o8);
            else store8<uint16_t>(reinterpret_cast<uint16_t *>(p.out) + elem0 + c * 32 + v8 * 8, o8);
          }
        }
      }
      if (p.tma_epi) {  // the tile (written or not) goes back to the warp that stores it and frees its slots
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->e_ready);
      }

      if (wg == 0 && live_row && p.lse) p.lse[grow] = (m_row + log2f(l_tot)) * LN2;
    };
    int G = 0;  // KV tiles of the items before the current one
    PairItem w;
    bool have = pair_item(p, 0, cluster, n_clusters, rank, w);
    if (have) stage_q(w, 0);
    for (int k = 0; have && ok; ++k) {
      const int nt = w.nt, pos = w.pos, q0 = w.q0;
      // Causal limit: keys 0 .. qpos.  Rows past the chunk's end take the last row's limit, so that no score of a
      // key outside the sequence enters a row maximum: the rescale vote below is per warp, and the result would
      // otherwise depend, in its last bits, on whatever lies behind the sequence's rows in the cache.
      const int qpos = pos + q0 + min(row, w.rows_valid - 1);
      float m_used = -INFINITY, l_run = 0.f;
      for (int j = 0; j < nt; ++j) {
        const int g = G + j;
        const uint32_t t_s = tmem + lane_sel + ((g & 1) ? TMEM_S1 : TMEM_S0);
        if (ok) ok = wait_or_abort(&ctl->s_full[g & 1], (g >> 1) & 1, abort_flag);
        tc_fence_after();
        uint32_t sr[32];
        tmem_ld32(t_s + wg * 32, sr);
        tmem_wait_ld();
        const int key0 = j * P2_BN + wg * 32;
        const bool need_mask = j * P2_BN + P2_BN - 1 > pos + q0;
        float mx = -INFINITY;
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float v = __uint_as_float(sr[i]);
            v = (key0 + i <= qpos) ? v : -INFINITY;
            sr[i] = __float_as_uint(v);
            mx = fmaxf(mx, v);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(sr[i]));
        }
        ctl->mxbuf[g & 1][wg][row] = mx;
        asm volatile("bar.sync 1, %0;" ::"n"(P2_SM_THREADS) : "memory");
#pragma unroll
        for (int w2 = 0; w2 < P2_NWG; ++w2) mx = fmaxf(mx, ctl->mxbuf[g & 1][w2][row]);
        const float m_new = fmaxf(m_used, mx * p.scale_log2);
        if (__any_sync(0xffffffffu, m_new - m_used > PF_RESCALE_THRESHOLD)) {
          if (j > 0) {
            const float alpha = fast_exp2(m_used - m_new);
            l_run *= alpha;
            wait_pv_done(g - 1);
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
          if (!p.fast_p) tmem_st8(t_s + 64 + wg * 16 + h2 * 8, lo);
        }
        l_run += lsum;
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) remote_arrive(p_full_addr[g & 1]);
        // Last tile of the item: every Q K^T of it has completed (s_full above), so the producer has already
        // asked for the next item's Q tile -- rotate it while the tensor core runs this item's last P V.
        if (j == nt - 1) {
          PairItem wn;  // looked up again at the item's end rather than kept in registers through the epilogue
          if (pair_item(p, k + 1, cluster, n_clusters, rank, wn)) stage_q(wn, k + 1);
        }
        // The first P of this item is on its way: now finish the previous item (its last P V was issued right
        // after this item's first Q K^T).  This item's first P V waits until O has been read out.
        if (j == 0 && k > 0) epilogue(k - 1, G, true);
        if (j > 0) wait_pv_done(g - 1);
      }
      // the row's sum and maximum wait in shared memory for the item's epilogue (single buffers: the epilogue of
      // the item before has run by now, at this item's first tile)
      ctl->lbuf[wg][row] = l_run;
      if (wg == 0) ctl->mbuf[row] = m_used;

      G += nt;
      have = pair_item(p, k + 1, cluster, n_clusters, rank, w);
      if (!have && ok) epilogue(k, G, false);   // the pair's last item
    }
  }

  // ---- teardown: both CTAs meet (no signal may target a CTA that has left), then free TMEM ----
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && warp == 1) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) { }
  }
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem, 512);
  }
}

}  // namespace

bool prefill_umma_supported(int n_new) { return n_new >= 64; }

int launch_prefill_umma_pair(const PrefillCall &c, cudaStream_t st, int *n_launched) {
  *n_launched = 0;
  if ((reinterpret_cast<uintptr_t>(c.q) | reinterpret_cast<uintptr_t>(c.kc) | reinterpret_cast<uintptr_t>(c.vc)) & 15)
    return 1;
  if (c.q_heads % 2) return 2;
  PrefillParams p;
  memset(&p, 0, sizeof(p));
  p.gate = c.gate; p.out = c.out; p.lse = c.lse; p.cache_row = c.cache_row; p.pages = c.pages; p.pos = c.pos; p.q_pos = c.q_pos; p.mpos = c.mpos;
  p.status = c.status; p.n_seq = c.n_seq; p.n_new = c.n_new; p.q_heads = c.q_heads; p.kv_heads = c.kv_heads;
  p.n_qtiles = (c.n_new + P2_BM - 1) / P2_BM;
  p.scale_log2 = c.scale * LOG2E;
  p.do_rope = c.do_rope; p.out_is_f32 = c.out_is_f32;
  p.fast_p = c.fast_p;
  p.rope = c.rope;
  CUtensorMap mq, mk, mv;
  if (encode_map(&mq, c.q, (int64_t)c.n_seq * c.n_new, c.q_heads * HEAD_DIM, P2_BM) != CUDA_SUCCESS) return 3;
  if (encode_map(&mk, c.kc, c.cache_rows, c.kv_heads * HEAD_DIM, 64) != CUDA_SUCCESS) return 3;
  if (encode_map(&mv, c.vc, c.cache_rows, c.kv_heads * HEAD_DIM, 64) != CUDA_SUCCESS) return 3;
  // bf16 output goes out by TMA store from an epilogue tile in the K/V ring, where the gate tile is loaded first
  p.tma_epi = (!c.out_is_f32 && !(reinterpret_cast<uintptr_t>(c.out) & 15) && !(reinterpret_cast<uintptr_t>(c.gate) & 15)) ? 1 : 0;
  CUtensorMap mg = mq, mo = mq;
  if (p.tma_epi) {
    if (c.gate && encode_map(&mg, c.gate, (int64_t)c.n_seq * c.n_new, c.q_heads * HEAD_DIM, P2_BM) != CUDA_SUCCESS) return 3;
    if (encode_map(&mo, c.out, (int64_t)c.n_seq * c.n_new, c.q_heads * HEAD_DIM, P2_BM) != CUDA_SUCCESS) return 3;
  }
  constexpr size_t smem = 1024 + P2_QBYTES + P2_NSLOT * P2_SLOT + sizeof(PairCtl);
  // Once per device: the shared-memory attribute and the number of CTA pairs the device holds at once (the
  // grid is persistent: that many pairs walk a static list of items).  The steps are idempotent, so atomics
  // are all that concurrent host threads need.
  static std::atomic<int> resident_pairs[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
  int pairs_resident = dev >= 0 ? resident_pairs[dev].load(std::memory_order_acquire) : 0;
  if (pairs_resident <= 0) {
    if (cudaFuncSetAttribute(prefill_umma_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return 3;
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev < 0 ? 0 : dev) != cudaSuccess || sms < 2) sms = 148;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(sms & ~1));
    cfg.blockDim = dim3(P2_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, prefill_umma_pair_kernel, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sms / 2;
    }
    pairs_resident = n;
    if (dev >= 0) resident_pairs[dev].store(n, std::memory_order_release);
  }
  const long long n_items = (long long)c.n_seq * p.n_qtiles * (c.q_heads / 2);  // (sequence, query tile, head pair)
  if (n_items > 0x3fffffffll) return 2;
  const long long n_pairs = n_items < pairs_resident ? n_items : pairs_resident;
  prefill_umma_pair_kernel<<<(unsigned)(2 * n_pairs), P2_THREADS, smem, st>>>(mq, mk, mv, mg, mo, p);
  *n_launched = 1;
  return cudaPeekAtLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace qwb
