// Causal chunked-prefill attention for head_dim 256 on the 5th-generation tensor cores.
//
// One CTA owns 128 consecutive query rows of one query head.  S = Q K^T and O += P V are
// tcgen05.mma (UMMA) contractions, 128 x 128 x 256 and 128 x 256 x 128 per KV tile of 128 keys,
// with all accumulators in tensor memory:
//     TMEM columns   0..255  O  (128 rows x 256 fp32)
//                  256..383  S0 (128 x 128 fp32)   P0 reuses it: bf16 "hi" in columns 0..63,
//                  384..511  S1                     bf16 "lo" (p - hi) in columns 64..127; P1 likewise
// so the whole 512-column TMEM of the SM is in use and S is double buffered: while the softmax
// warps turn S_j into P_j, the tensor pipe already computes S_{j+1} and then P_{j-1} V_{j-1}.
//
// Shared memory: the Q tile (64 KB, four 128-byte-swizzled sub-tiles of 64 channels, plus a
// 16 KB sub-tile with the bf16 "lo" part of the 64 rotated channels, which keeps the scores and
// the LSE at fp32-level accuracy) stays resident; K and V stream through a ring of 16 KB slots filled by TMA (no multicast) in the exact order the MMA
// warp consumes them:  K_0 | K_1 V_0 | K_2 V_1 | ...   A K slot is one 64-channel sub-tile of
// 128 keys (K-major operand), a V slot is 32 keys x 256 channels (MN-major operand).  Each slot
// is released by a tcgen05.commit as soon as the MMAs that read it have retired.
//
// Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer (one elected lane) and TMEM owner,
// warps 2..17 = four softmax / correction / epilogue warpgroups.  Warpgroup w owns key columns
// [32w, 32w+32) of every S tile and output channels [64w, 64w+64); within a warpgroup a thread is
// one query row (TMEM lane).  The four threads of a row exchange their partial row maxima through
// shared memory once per tile, so a tile's softmax is 32 exponentials per thread and its latency
// stays under the tensor time of a tile.
// P is fed to the tensor core as a bf16 hi + lo pair (two passes over V): a single bf16 P has a
// relative error of 2^-9 per key, which alone puts the output 1.2e-3 (rel-L2) from the fp32
// result; the pair brings it to 6e-4 (left over from rounding the rotated Q to bf16).  The "fast"
// mode skips the lo pass.  Mixed fp16 x bf16 operands are not an option: kind::f16 with different
// A and B formats raises an illegal-instruction error on this part.
// Partial RoPE is applied to the Q tile in shared memory before the first MMA (prologue) and
// 1/l * sigmoid(gate) is applied while O is read out of TMEM (epilogue).
// Every wait is bounded: when one runs out the CTA raises a shared abort flag, records an error
// code in the caller's status word, drains and frees its TMEM.
#include "prefill_umma.cuh"

#include <cstring>

#include "umma_common.cuh"

namespace qwb {

namespace {

constexpr int PF_BM = 128;                 // query rows per CTA
constexpr int PF_BN = 128;                 // keys per KV tile
constexpr int PF_SLOT = 16384;             // ring slot bytes
constexpr int PF_NSLOT = 8;                // ring slots
constexpr int PF_QBYTES = 5 * PF_SLOT;     // four 64-channel sub-tiles + the rotary "lo" sub-tile
constexpr int PF_NWG = 4;                  // softmax warpgroups
constexpr int PF_SM_THREADS = PF_NWG * 128;
constexpr int PF_THREADS = 64 + PF_SM_THREADS;


struct SharedCtl {
  uint64_t q_full, q_ready, s_full[2], p_full[2], o_done;
  uint64_t slot_full[PF_NSLOT], slot_empty[PF_NSLOT];
  uint32_t tmem_base;
  volatile int abort_flag;
  float mxbuf[2][PF_NWG][128];   // partial row maxima of the tile, double buffered by tile parity
  float lbuf[PF_NWG][128];       // partial row sums, combined in the epilogue
};

__global__ void __launch_bounds__(PF_THREADS, 1)
prefill_umma_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                    const __grid_constant__ CUtensorMap mapV, const __grid_constant__ PrefillParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *q_smem = smem;                       // 5 x 16 KB
  uint8_t *ring = smem + PF_QBYTES;             // PF_NSLOT x 16 KB
  SharedCtl *ctl = reinterpret_cast<SharedCtl *>(ring + PF_NSLOT * PF_SLOT);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---- which tile: heaviest (latest) query tiles first ----
  const int per_seq = p.n_qtiles * p.q_heads;
  const int s = blockIdx.x / per_seq;
  const int rem = blockIdx.x % per_seq;
  const int qt = p.n_qtiles - 1 - rem / p.q_heads;
  const int head = rem % p.q_heads;
  const int kvh = head / GROUP;
  const long long crow = p.cache_row ? p.cache_row[s] : 0;  // first cache row of the sequence (contiguous layout)
  const int q0 = qt * PF_BM;
  const int rows_valid = min(PF_BM, p.n_new - q0);
  const int pos = p.pos[s];
  const int kv_len = pos + q0 + rows_valid;           // keys visible to the last row of the tile
  const int nt = (kv_len + PF_BN - 1) / PF_BN;        // KV tiles

  // A launch that has already failed somewhere does not keep the GPU busy with further timeouts.
  // One thread reads the status word so that the whole CTA takes the same decision.
  if (tid == 0) ctl->abort_flag = (p.status && *reinterpret_cast<volatile int *>(p.status) != 0) ? 1 : 0;
  __syncthreads();
  if (ctl->abort_flag) return;
  __syncthreads();

  if (tid == 0) {
    mbar_init(&ctl->q_full, 1);
    mbar_init(&ctl->q_ready, PF_SM_THREADS);
    for (int i = 0; i < 2; ++i) { mbar_init(&ctl->s_full[i], 1); mbar_init(&ctl->p_full[i], PF_SM_THREADS); }
    mbar_init(&ctl->o_done, 1);
    for (int i = 0; i < PF_NSLOT; ++i) { mbar_init(&ctl->slot_full[i], 1); mbar_init(&ctl->slot_empty[i], 1); }
    ctl->abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&mapQ);
    prefetch_tensormap(&mapK);
    prefetch_tensormap(&mapV);
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  volatile int *abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // =============================== TMA producer ===========================================
    if (elect_one()) {
      mbar_expect_tx(&ctl->q_full, 4 * PF_SLOT);
      const int qrow = s * p.n_new + q0;
#pragma unroll
      for (int c = 0; c < 4; ++c) tma_load_2d(q_smem + c * PF_SLOT, &mapQ, &ctl->q_full, head * HEAD_DIM + c * 64, qrow);
      // slot stream: K_0 | K_1 V_0 | K_2 V_1 | ... | V_{nt-1}
      uint32_t it = 0;
      bool ok = true;
      auto load_k = [&](int j) {
        for (int c = 0; c < 4 && ok; ++c, ++it) {
          const int sl = it % PF_NSLOT;
          if (it >= PF_NSLOT && !wait_or_abort(&ctl->slot_empty[sl], ((it / PF_NSLOT) - 1) & 1, abort_flag)) {
            if (!*abort_flag && p.status) *p.status = DEV_ERR_EMPTY_WAIT;
            *abort_flag = 1;
            ok = false;
            break;
          }
          mbar_expect_tx(&ctl->slot_full[sl], PF_SLOT);
          tma_load_2d(ring + sl * PF_SLOT, &mapK, &ctl->slot_full[sl], kvh * HEAD_DIM + c * 64, (int)cache_row_at(p.pages, crow, s, j * PF_BN));
        }
      };
      auto load_v = [&](int j) {
        for (int g = 0; g < 4 && ok; ++g, ++it) {
          const int sl = it % PF_NSLOT;
          if (it >= PF_NSLOT && !wait_or_abort(&ctl->slot_empty[sl], ((it / PF_NSLOT) - 1) & 1, abort_flag)) {
            if (!*abort_flag && p.status) *p.status = DEV_ERR_EMPTY_WAIT;
            *abort_flag = 1;
            ok = false;
            break;
          }
          mbar_expect_tx(&ctl->slot_full[sl], PF_SLOT);
#pragma unroll
          for (int c = 0; c < 4; ++c)  // 32 keys x 64 channels each, channel atoms 4 KB apart
            tma_load_2d(ring + sl * PF_SLOT + c * 4096, &mapV, &ctl->slot_full[sl], kvh * HEAD_DIM + c * 64,
                        (int)cache_row_at(p.pages, crow, s, j * PF_BN + g * 32));
        }
      };
      for (int j = 0; j <= nt && ok; ++j) {
        if (j < nt) load_k(j);
        if (j >= 1) load_v(j - 1);
      }
    }
  } else if (warp == 1) {
    // =============================== MMA issuer (one thread) =================================
    // Descriptors are built once and advanced by adding the (16-byte unit) offset to their
    // start-address field: a tcgen05.mma of this shape keeps the tensor pipe busy for only ~64
    // cycles, so the issuing thread has to be quicker than that per instruction.
    const uint32_t idesc_qk = make_idesc(128, 128, 1, 1, 0, 0);
    const uint32_t idesc_pv = make_idesc(128, 256, 1, 1, 0, 1);
    const uint64_t qdesc0 = smem_desc(smem_u32(q_smem), 16, 1024);
    const uint64_t kdesc0 = smem_desc(smem_u32(ring), 16, 1024);
    const uint64_t vdesc0 = smem_desc(smem_u32(ring), 4096, 1024);
    bool ok = wait_or_abort(&ctl->q_ready, 0, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok && lane == 0) { if (!*abort_flag && p.status) *p.status = DEV_ERR_MMA_WAIT; *abort_flag = 1; }
    tc_fence_after();
    uint32_t it = 0;
    for (int j = 0; j <= nt && ok; ++j) {
      if (j < nt) {
        // ---- S[j & 1] = Q K_j^T ----
        const uint32_t d_s = tmem + ((j & 1) ? TMEM_S1 : TMEM_S0);
        for (int c = 0; c < 4 && ok; ++c, ++it) {
          const int sl = it % PF_NSLOT;
          ok = wait_or_abort(&ctl->slot_full[sl], (it / PF_NSLOT) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) { if (lane == 0) { if (!*abort_flag && p.status) *p.status = DEV_ERR_MMA_WAIT; *abort_flag = 1; } break; }
          tc_fence_after();
          if (elect_one()) {
            const uint64_t kd = kdesc0 + (uint64_t)(sl * (PF_SLOT >> 4));
            const uint64_t qd = qdesc0 + (uint64_t)(c * (PF_SLOT >> 4));
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_ss(d_s, qd + (uint64_t)(k * 2), kd + (uint64_t)(k * 2), idesc_qk, !(c == 0 && k == 0));
            if (c == 0 && p.do_rope) {  // low-order part of the rotated channels against the same K sub-tile
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma_ss(d_s, qdesc0 + (uint64_t)(4 * (PF_SLOT >> 4) + k * 2), kd + (uint64_t)(k * 2), idesc_qk, 1);
            }
            umma_commit(&ctl->slot_empty[sl]);
            if (c == 3) umma_commit(&ctl->s_full[j & 1]);
          }
          __syncwarp();
        }
      }
      if (j >= 1 && ok) {
        // ---- O += P_{j-1} V_{j-1} ----
        const int jj = j - 1;
        ok = wait_or_abort(&ctl->p_full[jj & 1], (jj >> 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { if (lane == 0) { if (!*abort_flag && p.status) *p.status = DEV_ERR_SOFTMAX_WAIT; *abort_flag = 1; } break; }
        tc_fence_after();
        const uint32_t a_p = tmem + ((jj & 1) ? TMEM_S1 : TMEM_S0);
        for (int g = 0; g < 4 && ok; ++g, ++it) {
          const int sl = it % PF_NSLOT;
          ok = wait_or_abort(&ctl->slot_full[sl], (it / PF_NSLOT) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) { if (lane == 0) { if (!*abort_flag && p.status) *p.status = DEV_ERR_MMA_WAIT; *abort_flag = 1; } break; }
          // keys past the end of the sequence may hold anything in V; P is zero there but
          // 0 * NaN is NaN, so clear those rows before the tensor core reads them
          const int key_lo = jj * PF_BN + g * 32;
          if (key_lo + 32 > kv_len) {
            const int valid = max(0, kv_len - key_lo);
            for (int idx = lane; idx < 32 * 32; idx += 32) {
              const int kr = idx >> 5, c16 = idx & 31;  // key row, 16-byte column (8 channels)
              if (kr >= valid)
                *reinterpret_cast<uint4 *>(ring + sl * PF_SLOT + (c16 >> 3) * 4096 + kr * 128 + (((c16 & 7) ^ (kr & 7)) << 4)) =
                    make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async();
            __syncwarp();
          }
          tc_fence_after();
          if (elect_one()) {
            const uint64_t vd = vdesc0 + (uint64_t)(sl * (PF_SLOT >> 4));
#pragma unroll
            for (int k = 0; k < 2; ++k) {
              umma_ts(tmem + TMEM_O, a_p + (g * 2 + k) * 8, vd + (uint64_t)(k * 128), idesc_pv, !(jj == 0 && g == 0 && k == 0));
              if (!p.fast_p) umma_ts(tmem + TMEM_O, a_p + 64 + (g * 2 + k) * 8, vd + (uint64_t)(k * 128), idesc_pv, 1);
            }
            umma_commit(&ctl->slot_empty[sl]);
            if (g == 3) umma_commit(&ctl->o_done);
          }
          __syncwarp();
        }
      }
    }
  } else {
    // ============ softmax / correction / epilogue: thread = (query row, 32-key column group) =========
    const int wg = (warp - 2) >> 2;                 // column group / output channel group
    const int row = (warp & 3) * 32 + lane;         // TMEM lane quarter of a warp is warp % 4
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const int qpos = pos + q0 + row;                // absolute position = last visible key
    bool ok = wait_or_abort(&ctl->q_full, 0, abort_flag);
    // ---- prologue: rotate the 64 rotary channels in shared memory; warpgroup w takes the pairs
    //      (8w + i, 8w + i + 32), i < 8, of every row and writes their bf16 hi and lo parts ----
    if (ok && p.do_rope) {
      const size_t trow = (size_t)s * p.n_new + q0 + row;
      const bool live = row < rows_valid;
      uint8_t *base = q_smem + row * 128;
      uint8_t *lo_base = q_smem + 4 * PF_SLOT + row * 128;
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
          const int pz = (p.mpos && live) ? p.mpos[trow * 3 + mrope_component(i)] : qpos;
          float cs, sn;
          rope_sincos_fast(pz, p.rope.inv_freq[i], cs, sn);
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
    mbar_arrive(&ctl->q_ready);

    float m_used = -INFINITY, l_run = 0.f;
    // o_done completes one phase per P V.  A parity wait can only tell the current phase from
    // the one before it, so the phases are observed strictly in order: o_seen counts them.
    int o_seen = 0;
    auto wait_pv_done = [&](int upto) {
      while (ok && o_seen <= upto) {
        ok = wait_or_abort(&ctl->o_done, o_seen & 1, abort_flag);
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
      const int key0 = j * PF_BN + wg * 32;
      const bool need_mask = j * PF_BN + PF_BN - 1 > pos + q0;  // some row of the tile cannot see its last key
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
      // exchange the partial maxima of the row.  Passing this barrier also means every thread has
      // finished reading its S columns, so P may now overwrite the S buffer.
      ctl->mxbuf[j & 1][wg][row] = mx;
      asm volatile("bar.sync 1, %0;" ::"n"(PF_SM_THREADS) : "memory");
#pragma unroll
      for (int w2 = 0; w2 < PF_NWG; ++w2) mx = fmaxf(mx, ctl->mxbuf[j & 1][w2][row]);
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      // Lazy rescale: only when the running max of some row of this warp grew by more than 2^8.
      // The decision is made per warp (tcgen05.ld/st are warp-wide); the four warps that share
      // these 32 rows see the same maxima and decide alike.
      if (__any_sync(0xffffffffu, m_new - m_used > PF_RESCALE_THRESHOLD)) {
        if (j > 0) {
          const float alpha = fast_exp2(m_used - m_new);
          l_run *= alpha;
          wait_pv_done(j - 1);  // O may only be touched once the previous P V has retired
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
      mbar_arrive(&ctl->p_full[j & 1]);
      if (j > 0) wait_pv_done(j - 1);  // long retired by now; keeps the phase count in step
    }

    // ---- epilogue: O / l * sigmoid(gate) -> out; warpgroup w writes channels [64w, 64w+64) ----
    ctl->lbuf[wg][row] = l_run;
    wait_pv_done(nt - 1);
    asm volatile("bar.sync 1, %0;" ::"n"(PF_SM_THREADS) : "memory");
    if (!__all_sync(0xffffffffu, ok)) {
      if (lane == 0 && !*abort_flag && p.status) *p.status = DEV_ERR_SOFTMAX_WAIT;
      *abort_flag = 1;
    } else {
      tc_fence_after();
      float l_tot = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < PF_NWG; ++w2) l_tot += ctl->lbuf[w2][row];
      const float inv = 1.f / l_tot;
      const size_t grow = ((size_t)s * p.n_new + q0 + row) * p.q_heads + head;
      const uint32_t t_o = tmem + lane_sel + TMEM_O + wg * 64;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t orow[32];
        tmem_ld32(t_o + c * 32, orow);
        tmem_wait_ld();
        if (row < rows_valid) {
          const size_t off = grow * HEAD_DIM + wg * 64 + c * 32;
#pragma unroll
          for (int v8 = 0; v8 < 4; ++v8) {
            float o8[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) o8[e] = __uint_as_float(orow[v8 * 8 + e]) * inv;
            if (p.gate) {
              float g8[8];
              load8<uint16_t>(p.gate + off + v8 * 8, g8);
#pragma unroll
              for (int e = 0; e < 8; ++e) o8[e] *= sigmoidf_(g8[e]);
            }
            if (p.out_is_f32)
              store8<float>(reinterpret_cast<float *>(p.out) + off + v8 * 8, o8);
            else
              store8<uint16_t>(reinterpret_cast<uint16_t *>(p.out) + off + v8 * 8, o8);
          }
        }
      }
      if (wg == 0 && row < rows_valid && p.lse) p.lse[grow] = (m_used + log2f(l_tot)) * LN2;
    }
  }

  // ---- teardown: everyone meets, then the allocating warp frees TMEM ----
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      // give TMA writes and tensor-core work in flight a moment to land before the CTA's
      // shared and tensor memory go away
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) { }
    }
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace

bool prefill_umma_supported(int n_new) { return n_new >= 64; }

int launch_prefill_umma(const PrefillCall &c, cudaStream_t st, int *n_launched) {
  *n_launched = 0;
  if ((reinterpret_cast<uintptr_t>(c.q) | reinterpret_cast<uintptr_t>(c.kc) | reinterpret_cast<uintptr_t>(c.vc)) & 15)
    return 1;
  PrefillParams p;
  memset(&p, 0, sizeof(p));
  p.gate = c.gate; p.out = c.out; p.lse = c.lse; p.cache_row = c.cache_row; p.pages = c.pages; p.pos = c.pos; p.mpos = c.mpos;
  p.status = c.status; p.n_seq = c.n_seq; p.n_new = c.n_new; p.q_heads = c.q_heads; p.kv_heads = c.kv_heads;
  p.n_qtiles = (c.n_new + PF_BM - 1) / PF_BM;
  p.scale_log2 = c.scale * LOG2E;
  p.do_rope = c.do_rope; p.out_is_f32 = c.out_is_f32;
  p.fast_p = c.fast_p;
  p.rope = c.rope;
  CUtensorMap mq, mk, mv;
  if (encode_map(&mq, c.q, (int64_t)c.n_seq * c.n_new, c.q_heads * HEAD_DIM, PF_BM) != CUDA_SUCCESS) return 3;
  if (encode_map(&mk, c.kc, c.cache_rows, c.kv_heads * HEAD_DIM, PF_BN) != CUDA_SUCCESS) return 3;
  if (encode_map(&mv, c.vc, c.cache_rows, c.kv_heads * HEAD_DIM, 32) != CUDA_SUCCESS) return 3;
  constexpr size_t smem = 1024 + PF_QBYTES + PF_NSLOT * PF_SLOT + sizeof(SharedCtl);
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(prefill_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return 3;
    configured[dev] = true;
  }
  const long long grid = (long long)c.n_seq * p.n_qtiles * c.q_heads;
  if (grid > 0x7fffffffll) return 2;
  prefill_umma_kernel<<<(unsigned)grid, PF_THREADS, smem, st>>>(mq, mk, mv, p);
  *n_launched = 1;
  return cudaPeekAtLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace qwb
