// Causal chunked-prefill attention, CTA-pair version (tcgen05 cta_group::2).
//
// Two CTAs of a cluster (two SMs) take the same 128 query rows of two query heads that share a
// KV head, so every K/V tile is needed by both.  With cta_group::2 one tcgen05.mma spans the pair:
// M = 256 (128 rows per CTA, each CTA's own Q / P and its own TMEM accumulators) and the B operand
// is split across the pair's shared memories -- for S = Q K^T each CTA stages 64 of the tile's 128
// keys, for O += P V each CTA stages 128 of the 256 value channels.  Per CTA and KV tile that is
// 64 KB instead of 128 KB: half the L2->SM traffic, half the shared-memory read bandwidth per MMA,
// and the same 128 KB ring now holds two tiles of look-ahead instead of one, which is what hides
// the load latency the single-CTA kernel is bound by.
//
// TMEM map: O | S0 | S1, P over
// S as bf16 hi + lo; warp roles (0 = TMA producer, 1 = TMEM owner and -- in the leader CTA only --
// MMA issuer, 2..17 = four softmax warpgroups), RoPE(q) prologue in shared memory, 1/l * sigmoid
// epilogue out of TMEM, bounded waits with an abort flag and a status word.
//
// Cross-CTA signalling: the leader's barriers collect both CTAs.  TMA loads of either CTA complete
// on the leader's slot barrier (cp.async.bulk.tensor with .cta_group::2, no multicast); softmax
// threads of the peer arrive on the leader's q_ready / p_full barriers through mapa'd addresses;
// the MMA thread publishes "S_j complete" and "P_j V_j retired" to both CTAs with one
// tcgen05.commit each (arrival multicast to the same barrier in both CTAs); those two signals also
// free the ring slots: K slots are reused every second tile and V slots every second tile, so the
// producers wait for s_full / o_done of the tile that last used the slot instead of per-slot
// barriers.
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
constexpr int P2_THREADS = 64 + P2_SM_THREADS;

struct PairCtl {
  uint64_t q_full, q_ready, s_full[2], p_full[2], o_done[2];
  uint64_t slot_full[P2_NSLOT];
  uint64_t fix_bar;              // CTA-local: the ragged last V tile lands here first
  uint32_t tmem_base;
  volatile int abort_flag;
  uint32_t skip;                 // leader: the launch had already failed when this pair started
  float mxbuf[2][P2_NWG][128];
  float lbuf[P2_NWG][128];
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

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P2_THREADS, 1)
prefill_umma_pair_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                         const __grid_constant__ CUtensorMap mapV, const __grid_constant__ PrefillParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *q_smem = smem;
  uint8_t *ring = smem + P2_QBYTES;
  PairCtl *ctl = reinterpret_cast<PairCtl *>(ring + P2_NSLOT * P2_SLOT);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader (issues the MMAs), 1 = peer
  const bool leader = rank == 0;

  // ---- which tile: heaviest (latest) query tiles first; a pair = two heads of one KV head ----
  const int pairs_per_seq = p.n_qtiles * (p.q_heads / 2);
  const int cid = blockIdx.x >> 1;
  const int s = cid / pairs_per_seq;
  const int rem = cid % pairs_per_seq;
  const int qt = p.n_qtiles - 1 - rem / (p.q_heads / 2);
  const int head = (rem % (p.q_heads / 2)) * 2 + (int)rank;
  const int kvh = head / GROUP;
  const long long crow = p.cache_row ? p.cache_row[s] : 0;  // first cache row of the sequence (contiguous layout)
  const int q0 = qt * P2_BM;
  const int rows_valid = min(P2_BM, p.n_new - q0);
  const int pos = p.pos[s];
  const int kv_len = pos + q0 + rows_valid;
  const int nt = (kv_len + P2_BN - 1) / P2_BN;

  if (tid == 0) {
    mbar_init(&ctl->q_full, 1);
    mbar_init(&ctl->q_ready, 2 * P2_SM_THREADS);
    for (int i = 0; i < 2; ++i) { mbar_init(&ctl->s_full[i], 1); mbar_init(&ctl->p_full[i], 2 * P2_SM_THREADS); }
    mbar_init(&ctl->o_done[0], 1);
    mbar_init(&ctl->o_done[1], 1);
    for (int i = 0; i < P2_NSLOT; ++i) mbar_init(&ctl->slot_full[i], 2);
    mbar_init(&ctl->fix_bar, 1);
    ctl->abort_flag = 0;
    ctl->skip = (p.status && *reinterpret_cast<volatile int *>(p.status) != 0) ? 1u : 0u;
    fence_barrier_init();
    prefetch_tensormap(&mapQ);
    prefetch_tensormap(&mapK);
    prefetch_tensormap(&mapV);
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

  const bool partial_last = (kv_len % P2_BN) != 0;
  // The ring slots that V_t goes into last held V_{t-2} (K_0 for t = 1).  P V completion
  // alternates between two barriers by tile parity, so the phase waited for here is always the
  // one right before the phase this very load enables: a parity wait cannot tell phases two
  // apart, and a producer that runs ahead of the MMAs would otherwise lag that far.
  auto wait_v_slots_free = [&](int t) -> bool {
    if (t == 1) return wait_or_abort(&ctl->s_full[0], 0, abort_flag);
    if (t >= 2) return wait_or_abort(&ctl->o_done[t & 1], ((t - 2) >> 1) & 1, abort_flag);
    return true;
  };

  if (warp == 0) {
    // =============================== TMA producer (each CTA loads its halves) ================
    int producer_ok = 1;
    if (run && elect_one()) {
      mbar_expect_tx(&ctl->q_full, 4 * P2_SLOT);
      const int qrow = s * p.n_new + q0;
#pragma unroll
      for (int c = 0; c < 4; ++c) tma_load_2d(q_smem + c * P2_SLOT, &mapQ, &ctl->q_full, head * HEAD_DIM + c * 64, qrow);
      uint32_t it = 0;
      bool ok = true;
      // Ring slots in consumption order.  Per slot: wait until the MMAs that read its previous
      // contents have retired, announce this CTA's 16 KB on the leader's barrier, then two 8 KB boxes.
      for (int j = 0; j <= nt && ok; ++j) {
        if (j < nt) {
          for (int i = 0; i < 2 && ok; ++i, ++it) {  // K slot i: channels [128 i, 128 i + 128) of this CTA's 64 keys
            const int sl = it % P2_NSLOT;
            // K slots alternate between ring positions {0,1} and {4,5}: this slot last held K_{j-2},
            // which is free once S_{j-2} is complete (s_full[j & 1], phase (j - 2) / 2)
            if (i == 0 && j >= 2 && !wait_or_abort(&ctl->s_full[j & 1], ((j - 2) >> 1) & 1, abort_flag)) {
              if (!*abort_flag && p.status) *p.status = DEV_ERR_EMPTY_WAIT;
              *abort_flag = 1;
              ok = false;
              break;
            }
            const uint32_t bar = map_to_cta(smem_u32(&ctl->slot_full[sl]), 0);
            remote_arrive_expect_tx(bar, P2_SLOT);
            const int krow = (int)cache_row_at(p.pages, crow, s, j * P2_BN + (int)rank * 64);
#pragma unroll
            for (int a = 0; a < 2; ++a)
              tma_load_2d_pair(ring + sl * P2_SLOT + a * 8192, &mapK, bar, kvh * HEAD_DIM + (2 * i + a) * 64, krow);
          }
        }
        if (j >= 1 && !(partial_last && j == nt)) {  // a ragged last V tile is loaded by the whole warp below
          for (int g = 0; g < 2 && ok; ++g, ++it) {  // V slot g: keys [64 g, 64 g + 64), this CTA's 128 channels
            const int sl = it % P2_NSLOT;
            if (g == 0 && !wait_v_slots_free(j - 1)) {
              if (!*abort_flag && p.status) *p.status = DEV_ERR_EMPTY_WAIT;
              *abort_flag = 1;
              ok = false;
              break;
            }
            const uint32_t bar = map_to_cta(smem_u32(&ctl->slot_full[sl]), 0);
            remote_arrive_expect_tx(bar, P2_SLOT);
            const int vrow = (int)cache_row_at(p.pages, crow, s, (j - 1) * P2_BN + g * 64);
#pragma unroll
            for (int a = 0; a < 2; ++a)
              tma_load_2d_pair(ring + sl * P2_SLOT + a * 8192, &mapV, bar, kvh * HEAD_DIM + (int)rank * 128 + a * 64, vrow);
          }
        }
      }
      if (!ok) producer_ok = 0;
    }
    // ---- ragged last tile: rows of V past the sequence's end may hold anything (even NaN bit
    // patterns) and P is an exact zero there, but 0 * NaN is NaN.  The last V tile is therefore
    // loaded on a CTA-local barrier, its rows past the end are cleared by the whole warp, and only
    // then is the slot announced on the leader's barrier (a plain arrival: the bytes are in). ----
    producer_ok = __shfl_sync(0xffffffffu, producer_ok, 0);
    if (run && partial_last && producer_ok) {
      bool ok = true;
      for (int g = 0; g < 2; ++g) {
        const uint32_t itv = 4u * (uint32_t)nt - 2u + (uint32_t)g;  // the two last ring slots of this tile sequence
        const int sl = itv % P2_NSLOT;
        if (g == 0) ok = wait_v_slots_free(nt - 1);
        ok = __all_sync(0xffffffffu, ok);
        if (ok && elect_one()) {
          mbar_expect_tx(&ctl->fix_bar, P2_SLOT);
          const int vrow = (int)cache_row_at(p.pages, crow, s, (nt - 1) * P2_BN + g * 64);
#pragma unroll
          for (int a = 0; a < 2; ++a)
            tma_load_2d(ring + sl * P2_SLOT + a * 8192, &mapV, &ctl->fix_bar, kvh * HEAD_DIM + (int)rank * 128 + a * 64, vrow);
        }
        if (ok) ok = wait_or_abort(&ctl->fix_bar, g & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) { if (!*abort_flag && p.status) *p.status = DEV_ERR_EMPTY_WAIT; *abort_flag = 1; }
          break;
        }
        const int valid = max(0, kv_len - ((nt - 1) * P2_BN + g * 64));  // rows of this slot inside the sequence
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
    }
  } else if (warp == 1) {
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
      auto fail = [&](int code) {
        if (!*abort_flag && p.status) *p.status = code;
        *abort_flag = 1;
      };
      bool ok = wait_cluster_or_abort(&ctl->q_ready, 0, abort_flag);
      if (!ok) fail(DEV_ERR_MMA_WAIT);
      tc_fence_after();
      uint32_t it = 0;
      for (int j = 0; j <= nt && ok; ++j) {
        if (j < nt) {
          // ---- S[j & 1] = Q K_j^T for both CTAs' rows ----
          const uint32_t d_s = tmem + ((j & 1) ? TMEM_S1 : TMEM_S0);
#pragma unroll
          for (int i = 0; i < 2; ++i, ++it) {
            const int sl = it % P2_NSLOT;
            ok = ok && wait_cluster_or_abort(&ctl->slot_full[sl], (it / P2_NSLOT) & 1, abort_flag);
            if (!ok) { fail(DEV_ERR_MMA_WAIT); break; }
            tc_fence_after();
            const uint64_t kd = kdesc0 + (uint64_t)(sl * (P2_SLOT >> 4));
#pragma unroll
            for (int a = 0; a < 2; ++a) {
              const int c = 2 * i + a;  // 64-channel sub-tile
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma_ss_pair(d_s, qdesc0 + (uint64_t)((c * P2_SLOT + k * 32) >> 4),
                             kd + (uint64_t)((a * 8192 + k * 32) >> 4), idesc_qk, !(c == 0 && k == 0));
              if (c == 0 && p.do_rope) {
#pragma unroll
                for (int k = 0; k < 4; ++k)
                  umma_ss_pair(d_s, qdesc0 + (uint64_t)((4 * P2_SLOT + k * 32) >> 4), kd + (uint64_t)((k * 32) >> 4),
                               idesc_qk, 1);
              }
            }
          }
          // one completion point for the whole S tile, seen by the softmax warps (S is ready) and
          // by both producers (the tile's K slots are free)
          if (ok) umma_commit_both(&ctl->s_full[j & 1]);
        }
        if (j >= 1 && ok) {
          // ---- O += P_{j-1} V_{j-1} ----
          const int jj = j - 1;
          ok = wait_cluster_or_abort(&ctl->p_full[jj & 1], (jj >> 1) & 1, abort_flag);
          if (!ok) { fail(DEV_ERR_SOFTMAX_WAIT); break; }
          tc_fence_after();
          const uint32_t a_p = tmem + ((jj & 1) ? TMEM_S1 : TMEM_S0);
#pragma unroll
          for (int g = 0; g < 2; ++g, ++it) {
            const int sl = it % P2_NSLOT;
            ok = ok && wait_cluster_or_abort(&ctl->slot_full[sl], (it / P2_NSLOT) & 1, abort_flag);
            if (!ok) { fail(DEV_ERR_MMA_WAIT); break; }
            tc_fence_after();
            const uint64_t vd = vdesc0 + (uint64_t)(sl * (P2_SLOT >> 4));
#pragma unroll
            for (int k = 0; k < 4; ++k) {  // 16 keys per step
              umma_ts_pair(tmem + TMEM_O, a_p + (g * 4 + k) * 8, vd + (uint64_t)((k * 2048) >> 4), idesc_pv,
                           !(jj == 0 && g == 0 && k == 0));
              if (!p.fast_p)
                umma_ts_pair(tmem + TMEM_O, a_p + 64 + (g * 4 + k) * 8, vd + (uint64_t)((k * 2048) >> 4), idesc_pv, 1);
            }
          }
          if (ok) umma_commit_both(&ctl->o_done[jj & 1]);  // O updated; the tile's V slots are free
        }
      }
    }
  } else if (run) {
    // ============ softmax / correction / epilogue: thread = (query row, 32-key column group) =========
    const int wg = (warp - 2) >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const int qpos = pos + q0 + row;                                   // causal limit: keys 0 .. qpos
    const int rope_pos = (p.q_pos ? p.q_pos[s] : pos) + q0 + row;    // RoPE angle
    const uint32_t q_ready_addr = map_to_cta(smem_u32(&ctl->q_ready), 0);
    const uint32_t p_full_addr[2] = {map_to_cta(smem_u32(&ctl->p_full[0]), 0), map_to_cta(smem_u32(&ctl->p_full[1]), 0)};
    bool ok = wait_or_abort(&ctl->q_full, 0, abort_flag);
    if (ok && p.do_rope) {
      const size_t trow = (size_t)s * p.n_new + q0 + row;
      const bool live = row < rows_valid;
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
    fence_proxy_async();
    remote_arrive_release(q_ready_addr);

    float m_used = -INFINITY, l_run = 0.f;
    int o_seen = 0;  // P V completions observed so far, in order (tile t: o_done[t & 1], phase t / 2)
    auto wait_pv_done = [&](int upto) {
      while (ok && o_seen <= upto) {
        ok = wait_or_abort(&ctl->o_done[o_seen & 1], (o_seen >> 1) & 1, abort_flag);
        ++o_seen;
      }
    };
    for (int j = 0; j < nt; ++j) {
      const uint32_t t_s = tmem + lane_sel + ((j & 1) ? TMEM_S1 : TMEM_S0);
      if (ok) ok = wait_or_abort(&ctl->s_full[j & 1], (j >> 1) & 1, abort_flag);
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
      ctl->mxbuf[j & 1][wg][row] = mx;
      asm volatile("bar.sync 1, %0;" ::"n"(P2_SM_THREADS) : "memory");
#pragma unroll
      for (int w2 = 0; w2 < P2_NWG; ++w2) mx = fmaxf(mx, ctl->mxbuf[j & 1][w2][row]);
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      if (__any_sync(0xffffffffu, m_new - m_used > PF_RESCALE_THRESHOLD)) {
        if (j > 0) {
          const float alpha = fast_exp2(m_used - m_new);
          l_run *= alpha;
          wait_pv_done(j - 1);
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
      uint32_t hi[16], lo[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float p0 = fast_exp2(fmaf(__uint_as_float(sr[i]), p.scale_log2, -m_sub));
        const float p1 = fast_exp2(fmaf(__uint_as_float(sr[i + 1]), p.scale_log2, -m_sub));
        lsum += p0 + p1;
        const uint32_t h = pack_bf16(p0, p1);
        hi[i >> 1] = h;
        lo[i >> 1] = pack_bf16(p0 - bf16lo(h), p1 - bf16hi(h));
      }
      l_run += lsum;
      tmem_st16(t_s + wg * 16, hi);
      if (!p.fast_p) tmem_st16(t_s + 64 + wg * 16, lo);
      tmem_wait_st();
      tc_fence_before();
      remote_arrive(p_full_addr[j & 1]);
      if (j > 0) wait_pv_done(j - 1);
    }

    ctl->lbuf[wg][row] = l_run;
    wait_pv_done(nt - 1);
    asm volatile("bar.sync 1, %0;" ::"n"(P2_SM_THREADS) : "memory");
    if (!__all_sync(0xffffffffu, ok)) {
      if (lane == 0 && !*abort_flag && p.status) *p.status = DEV_ERR_SOFTMAX_WAIT;
      *abort_flag = 1;
    } else {
      tc_fence_after();
      float l_tot = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < P2_NWG; ++w2) l_tot += ctl->lbuf[w2][row];
      const float inv = 1.f / l_tot;
      const size_t grow = ((size_t)s * p.n_new + q0 + row) * p.q_heads + head;
      // O leaves TMEM one row per thread, but a row's 64 channels are one contiguous 128-byte
      // run in `out` and `gate`.  Each warp therefore transposes its 32 rows x 64 channels through
      // a padded staging area (Q and the K/V ring are idle by now: every MMA has retired) and then
      // walks the rows with the lanes across the channels, two per lane: every gate load and every
      // output store is one full coalesced line, and all 32 gate loads are in flight at once.
      float *stage = reinterpret_cast<float *>(smem) + (warp - 2) * (32 * 65);
      const uint32_t t_o = tmem + lane_sel + TMEM_O + wg * 64;
      const int row0 = (warp & 3) * 32;
      const int nrows = min(32, rows_valid - row0);
      const size_t elem0 = (((size_t)s * p.n_new + q0 + row0) * p.q_heads + head) * HEAD_DIM + wg * 64 + 2 * lane;
      const size_t row_stride = (size_t)p.q_heads * HEAD_DIM;
      uint32_t gw[32];
      {
        const uint16_t *gp = p.gate ? p.gate + elem0 : nullptr;
#pragma unroll
        for (int rr = 0; rr < 32; ++rr) {
          gw[rr] = (gp && rr < nrows) ? *reinterpret_cast<const uint32_t *>(gp) : 0u;
          gp += gp ? row_stride : 0;
        }
      }
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t orow[32];
        tmem_ld32(t_o + c * 32, orow);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) stage[lane * 65 + c * 32 + i] = __uint_as_float(orow[i]) * inv;
      }
      __syncwarp();
      if (p.out_is_f32) {
        float *op = reinterpret_cast<float *>(p.out) + elem0;
#pragma unroll
        for (int rr = 0; rr < 32; ++rr, op += row_stride) {
          if (rr < nrows) {
            float v0 = stage[rr * 65 + 2 * lane], v1 = stage[rr * 65 + 2 * lane + 1];
            if (p.gate) { v0 *= sigmoid_fast(bf16lo(gw[rr])); v1 *= sigmoid_fast(bf16hi(gw[rr])); }
            *reinterpret_cast<float2 *>(op) = make_float2(v0, v1);
          }
        }
      } else {
        uint16_t *op = reinterpret_cast<uint16_t *>(p.out) + elem0;
#pragma unroll
        for (int rr = 0; rr < 32; ++rr, op += row_stride) {
          if (rr < nrows) {
            float v0 = stage[rr * 65 + 2 * lane], v1 = stage[rr * 65 + 2 * lane + 1];
            if (p.gate) { v0 *= sigmoid_fast(bf16lo(gw[rr])); v1 *= sigmoid_fast(bf16hi(gw[rr])); }
            *reinterpret_cast<uint32_t *>(op) = pack_bf16(v0, v1);
          }
        }
      }
      if (wg == 0 && row < rows_valid && p.lse) p.lse[grow] = (m_used + log2f(l_tot)) * LN2;
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
  constexpr size_t smem = 1024 + P2_QBYTES + P2_NSLOT * P2_SLOT + sizeof(PairCtl);
  // once per device; the step is idempotent, so an atomic flag is all that concurrent host threads need
  static std::atomic<int> configured[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
  if (dev < 0 || !configured[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(prefill_umma_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return 3;
    if (dev >= 0) configured[dev].store(1, std::memory_order_release);
  }
  const long long grid = (long long)c.n_seq * p.n_qtiles * c.q_heads;  // CTAs; two per cluster
  if (grid > 0x7fffffffll) return 2;
  prefill_umma_pair_kernel<<<(unsigned)grid, P2_THREADS, smem, st>>>(mq, mk, mv, p);
  *n_launched = 1;
  return cudaPeekAtLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace qwb
