/*
 * qwengine_attn.h -- C ABI of the B200 (sm_100a) full-attention mixer.
 *
 * The reference engine has no separately linked attention library: its forward
 * passes launch five kernels inline (paths below are relative to the reference
 * project root).  Each "per-kernel launcher" here takes the argument list of one
 * of those launch sites, in the same order, with the <<<grid, block, 0, stream>>>
 * replaced by a trailing row count and stream, so a maintainer can swap the
 * inline launch for one call.  Every function returns 0 on success or a QW_ERR_*
 * code; none allocates, frees, synchronises or reads device memory on the host,
 * so all of them are legal inside a CUDA stream capture, as the reference's
 * decode and verify graphs require (src/model.cu:318-327,378-387).
 *
 * Element types.  The reference keeps activations AND the KV cache in fp32.
 * This library keeps the cache in bf16 (same indexing: [pos][kv_head][dim], K
 * and V in separate buffers, one such block per full-attention layer) and
 * offers every launcher twice:
 *   *_bf16  activations in bf16 -- the measured path;
 *   *_f32   activations in fp32 exactly as the reference call sites hold them,
 *           converted inside the kernels; only the cache element type differs.
 * bf16 values cross this ABI as raw 16-bit patterns (uint16_t).
 *
 * Geometry supported: head_dim 256, rotary_dim 64, q_heads = 6 * kv_heads,
 * kv_heads in {1, 2, 4} (4 is the model; 1 and 2 are the per-GPU slices of a
 * KV-head-sharded layer).  Anything else returns QW_ERR_SHAPE.
 *
 * Programmatic dependent launch.  The fused calls (qw_mixer_forward*) launch their
 * first kernel with cudaLaunchAttributeProgrammaticStreamSerialization; that kernel
 * waits for everything before it on the stream before it reads or writes anything,
 * so callers need do nothing.  The split-KV attention kernels trigger their
 * dependents as soon as they start: this only matters to a caller that launches
 * its OWN next kernel with that attribute -- such a kernel must call
 * cudaGridDependencySynchronize() (griddepcontrol.wait) before it reads `out`.
 * Kernels launched the ordinary way are ordered as always.
 */
#ifndef QWENGINE_ATTN_H_
#define QWENGINE_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef uint16_t qw_bf16;  /* raw bfloat16 bits                                   */
typedef void *qw_stream;   /* a cudaStream_t                                      */

enum {
  QW_OK = 0,
  QW_ERR_ARG = 1,       /* null pointer, negative count, misaligned buffer        */
  QW_ERR_SHAPE = 2,     /* geometry outside the supported set                     */
  QW_ERR_CUDA = 3,      /* a CUDA runtime / driver call failed                    */
  QW_ERR_WORKSPACE = 4, /* scratch / workspace too small                          */
  QW_ERR_DEVICE = 5,    /* a kernel recorded an error (bounded wait ran out)      */
  QW_ERR_TOO_LARGE = 6  /* request exceeds a fixed built-in capacity              */
};

/* Human-readable text for a QW_ERR_* code. */
const char *qw_strerror(int code);
/* ABI version: bumped when a signature in this file changes. */
int qw_abi_version(void);
/* Last CUDA error string seen by this library on the calling thread ("" if none). */
const char *qw_last_cuda_error(void);

/* ------------------------------------------------------------------------------------------
 * Per-kernel launchers (drop-in for the reference's inline launches)
 * ---------------------------------------------------------------------------------------- */

/* Partial RoPE in place on v[B][heads][dim]; pairs (i, i+rot/2), angle
 * (*dpos + b) * theta^(-2i/rot), or mpos[b*3 + component(i)] when mpos != NULL.
 * Replaces rope(): src/elem.cu:255-259 (kernel k_rope, src/elem.cu:119-137);
 * called at src/model.cu:228-229, src/prefill.cu:142-143, src/mtp.cu:172-173. */
int qw_rope_bf16(qw_bf16 *v, int heads, int dim, int rot, const int *dpos, float theta,
                 qw_stream stream, int B, const int *mpos);
int qw_rope_f32(float *v, int heads, int dim, int rot, const int *dpos, float theta,
                qw_stream stream, int B, const int *mpos);

/* Store rows k[b], v[b] (kvdim elements each) at cache slot *dpos + b.
 * Replaces k_kv_append<<<dim3(ceil(kvdim/256), B), 256>>>: src/mixers.cu:416-425;
 * launched at src/model.cu:234, src/prefill.cu:148, src/mtp.cu:174. */
int qw_kv_append_bf16(const qw_bf16 *k, const qw_bf16 *v, qw_bf16 *kc, qw_bf16 *vc,
                      const int *dpos, int kvdim, int B, qw_stream stream);
int qw_kv_append_f32(const float *k, const float *v, qw_bf16 *kc, qw_bf16 *vc,
                     const int *dpos, int kvdim, int B, qw_stream stream);

/* Decode / speculative-verify attention: row b of q[B][q_heads][dim] attends to the
 * first *dpos + b + 1 cache rows (its own included).  `scratch` is the reference's
 * score workspace and MUST hold B * q_heads * ctx floats, 16-byte aligned -- what the
 * reference's own kernel needs at the same launch (src/mixers.cu:441, rt.scores at
 * src/model.cu:168, M.scores at src/mtp.cu:115).  The launcher uses exactly that many floats
 * (qw_attn_decode_scratch_floats() returns the same number) for split-KV partials and
 * arrival counters: the more there are, the more CTAs share a sequence.  If they do not hold
 * even one set of partials (ctx below about 370: the reference sizes ctx as prompt + new
 * tokens + 8, src/main.cu:38, so short runs get there) the launcher leaves `scratch` untouched
 * and keeps the partials in the library's own fixed device array, the one
 * qw_attn_decode_bf16_noalloc uses.
 * ctx is the number of rows in kc / vc.  1 <= B <= 8.  The bf16 flavour runs B >= 2 on the
 * tcgen05 split-KV kernel; the fp32 flavour keeps q exact (bf16 hi + lo on all channels)
 * on the mma.sync kernel.  These launchers serve one sequence, so they take the kernel variant
 * whose CTAs merge a KV head together (see QW_F_NO_GRID_WAIT below): run them on one stream per
 * GPU at a time, as the reference does; an engine that overlaps attention calls on one GPU uses
 * qw_mixer_forward with that flag instead.
 * Replaces k_attn_decode<<<dim3(q_heads, B), 256>>>: src/mixers.cu:436-525;
 * launched at src/model.cu:236-238, src/mtp.cu:176-178. */
int qw_attn_decode_bf16(const qw_bf16 *q, const qw_bf16 *kc, const qw_bf16 *vc, qw_bf16 *out,
                        const int *dpos, int dim, int kv_heads, int q_heads, float scale,
                        float *scratch, int ctx, int B, qw_stream stream);
int qw_attn_decode_f32(const float *q, const qw_bf16 *kc, const qw_bf16 *vc, float *out,
                       const int *dpos, int dim, int kv_heads, int q_heads, float scale,
                       float *scratch, int ctx, int B, qw_stream stream);
size_t qw_attn_decode_scratch_floats(int q_heads, int kv_heads, int ctx, int B);

/* Decode / verify attention for callers that cannot hand over scratch memory.
 * No counterpart in the reference, whose call sites always pass their own `scores` buffer.
 * Some hosts of this library may not allocate device memory at the point where they launch
 * attention: an engine that takes all of its device memory in one block at start-up and has
 * nothing left to carve a workspace from, a plugin slot that is given tensors but no allocator,
 * or a latency-critical loop where a cudaMalloc (which can synchronise the device) is banned.
 * This variant of qw_attn_decode_bf16 takes no scratch argument: the split-KV partials go to
 * a fixed array that lives inside the library image, 5.2 MB of device memory that every GPU
 * which loads the library keeps until the process exits.  Limits: B <= 8 and kv_heads <= 4;
 * anything larger returns QW_ERR_TOO_LARGE.  It calls no cudaMalloc, cudaFree or other
 * allocating routine.  The first call on each device looks the array's device address up
 * (cudaGetSymbolAddress) and remembers it; make that first call outside any stream capture.
 * All calls on a device share the one array and leave their partials in it; nothing in it has
 * to be cleared between calls, but two calls whose kernels overlap on the GPU (different
 * streams, or concurrent graph branches) race on it -- serialise them. */
int qw_attn_decode_bf16_noalloc(const qw_bf16 *q, const qw_bf16 *kc, const qw_bf16 *vc, qw_bf16 *out,
                                const int *dpos, int dim, int kv_heads, int q_heads, float scale,
                                int ctx, int B, qw_stream stream);

/* Chunked-prefill attention: row t of q[T][q_heads][dim] attends to the first
 * *dpos + t + 1 cache rows.  Chunks of T >= 64 rows run on the tcgen05 CTA-pair kernel,
 * shorter ones on the split-KV kernels.  `scratch` (reference: T * q_heads * ctx floats,
 * src/prefill.cu:75), 16-byte aligned, holds either the reference's size or
 * qw_attn_prefill_scratch_floats() floats: the launcher, which is not told which, writes
 * no further than the smaller of the two, and where that is too little (a cache of a few
 * rows) it leaves `scratch` untouched and uses the library's fixed device array.  It holds
 * split-KV partials for short chunks and, in the fp32 flavour with T >= 64, the bf16 copy
 * of q that the tensor cores read (q is rounded to bf16 there, exactly as k is when it
 * enters the bf16 cache; short chunks keep q exact).
 * Replaces k_attn_prefill<<<dim3(q_heads, ceil(T/8)), 256>>>: src/mixers.cu:546-649;
 * launched at src/prefill.cu:152-154. */
int qw_attn_prefill_bf16(const qw_bf16 *q, const qw_bf16 *kc, const qw_bf16 *vc, qw_bf16 *out,
                         const int *dpos, int dim, int kv_heads, int q_heads, float scale,
                         float *scratch, int ctx, int T, qw_stream stream);
int qw_attn_prefill_f32(const float *q, const qw_bf16 *kc, const qw_bf16 *vc, float *out,
                        const int *dpos, int dim, int kv_heads, int q_heads, float scale,
                        float *scratch, int ctx, int T, qw_stream stream);
size_t qw_attn_prefill_scratch_floats(int q_heads, int kv_heads, int ctx, int T);

/* x[i] *= sigmoid(gate[i]) for i < n.
 * Replaces k_gate_sigmoid<<<ceil(n/256), 256>>>: src/mixers.cu:653-657;
 * launched at src/model.cu:239-240, src/prefill.cu:155-156, src/mtp.cu:179. */
int qw_gate_sigmoid_bf16(qw_bf16 *x, const qw_bf16 *gate, int n, qw_stream stream);
int qw_gate_sigmoid_f32(float *x, const float *gate, int n, qw_stream stream);

/* ------------------------------------------------------------------------------------------
 * Fused, batched mixer (the measured path)
 *
 * One call = rope(q), rope(k), append, attention and the sigmoid gate for a batch of
 * independent sequences -- the five launches of src/model.cu:228-240 (decode/verify),
 * src/prefill.cu:142-156 (prefill chunk) and src/mtp.cu:172-179 (draft head) in one
 * descriptor.  The reference serves one sequence; n_seq > 1 is a batched superset.
 * ---------------------------------------------------------------------------------------- */

enum {
  QW_F_ROPE = 1,       /* rotate q and k_new (else they arrive rotated)                 */
  QW_F_APPEND = 2,     /* write k_new / v_new into the cache before attending           */
  QW_F_GATE = 4,       /* multiply the output by sigmoid(gate)                          */
  QW_F_OUT_F32 = 8,    /* `out` is float instead of bf16 (checking aid)                 */
  QW_F_NO_UMMA = 16,   /* force the split-KV kernel even for long prefill chunks        */
  QW_F_FAST_P = 32,    /* tcgen05 prefill only: feed P as one bf16 instead of a bf16 hi+lo
                          pair; 1/3 less tensor work, output rel-L2 ~1.4e-3 instead of 2e-6 */
  QW_F_NO_CAUSAL = 128, /* every row sees exactly pos[s] (>= 1) keys of its sequence: the call covers
                          a KV sub-range that does not contain the new rows (cross-GPU KV split);
                          excludes QW_F_APPEND; with QW_F_ROPE the descriptor must carry q_pos    */
  QW_F_NO_ATTENTION = 256 /* with QW_F_APPEND: rotate k_new and store k_new / v_new, nothing else (q, gate, out
                          and workspace are not touched and may be NULL).  For a rank that holds a whole
                          chunk's keys but computes only some of its query rows (query-row split of one
                          sequence over a GPU pair): it appends the chunk once, then attends per row block
                          without QW_F_APPEND                                                        */,
  QW_F_NO_GRID_WAIT = 512 /* never pick a kernel whose CTAs wait for one another.  One to four sequences decoding
                          alone are served by a variant in which all CTAs of a KV head merge its result together
                          once every part has arrived (a bounded wait on an arrival counter); that needs the whole
                          grid -- one CTA per SM -- resident at once, which it is unless ANOTHER kernel that
                          holds SMs for as long runs beside it on the same GPU (two such calls on two streams can
                          starve each other: the wait then runs out after 0.2 s and *status is set).  A caller
                          that runs attention calls concurrently on one GPU sets this flag; it costs 4 to 5 us
                          of the 21 us such a call takes                                               */
};

typedef struct qw_mixer_desc {
  /* geometry */
  int n_seq;       /* sequences in this call                                            */
  int n_new;       /* new tokens per sequence: 1 decode, 2..8 verify, up to 32768 prefill */
  int q_heads, kv_heads, head_dim, rotary_dim;
  float theta;     /* RoPE base (1e7)                                                   */
  float scale;     /* softmax scale (1/16)                                              */
  int flags;       /* QW_F_*                                                            */
  /* activations, bf16, contiguous */
  const qw_bf16 *q;     /* [n_seq][n_new][q_heads][head_dim]                            */
  const qw_bf16 *k_new; /* [n_seq][n_new][kv_heads][head_dim]   (QW_F_APPEND)           */
  const qw_bf16 *v_new; /* same shape                            (QW_F_APPEND)           */
  const qw_bf16 *gate;  /* same shape as q                       (QW_F_GATE)             */
  void *out;            /* same shape as q, bf16 (float with QW_F_OUT_F32)               */
  float *lse;           /* [n_seq][n_new][q_heads] natural-log LSE, or NULL              */
  /* cache pool: rows of kv_heads*head_dim bf16; sequence s owns rows
   * cache_row[s] .. cache_row[s] + pos[s] + n_new - 1 */
  qw_bf16 *kc, *vc;
  int64_t cache_rows;        /* rows in the pool (extent of the tensor maps)            */
  const int64_t *cache_row;  /* device, [n_seq]; NULL means all zero (one sequence)      */
  const int *pos;            /* device, [n_seq]: tokens cached before this call (*dpos)  */
  const int *mpos;           /* device, [n_seq][n_new][3] mrope positions, or NULL       */
  /* workspace, device, qw_mixer_workspace_bytes() bytes, 256-byte aligned */
  void *workspace;
  size_t workspace_bytes;
  /* device int that receives a non-zero code if a kernel gave up on a bounded wait; may
   * be NULL.  It is only ever written on error. */
  int *status;
  /* Paged cache (optional; the reference keeps one contiguous cache per layer, src/model.cu:182-184, and
   * serves one sequence, README.md:365-367 -- a block table is what a multi-sequence server puts here).
   * block_table != NULL: the pool is cut into pages of page_rows rows (a multiple of 128) and token t of
   * sequence s lives in row block_table[s * block_table_stride + t / page_rows] * page_rows + t % page_rows;
   * cache_row is then ignored.  Device memory, int32, at least ceil((pos[s] + n_new) / page_rows) entries
   * per sequence.  NULL (a zeroed descriptor) keeps the contiguous layout. */
  const int *block_table;
  int block_table_stride;
  int page_rows;
  /* Optional, device, [n_seq]: absolute position of each sequence's first new row, used for the RoPE
   * angles (row b rotates by q_pos[s] + b) instead of pos[s].  A call that covers a KV sub-range of a
   * sequence (cross-GPU KV split) counts keys from the start of its range in pos[s] while its rows sit at
   * their absolute positions; with q_pos such a call rotates q (and, with QW_F_APPEND, k) itself, in
   * fp32 like every other call.  NULL (a zeroed descriptor): angles come from pos[s].  mpos, when given,
   * wins over both.  No counterpart in the reference (one GPU, one range). */
  const int *q_pos;
} qw_mixer_desc;

size_t qw_mixer_workspace_bytes(const qw_mixer_desc *d);
int qw_mixer_forward(const qw_mixer_desc *d, qw_stream stream);

/* Number of kernels the last qw_* call on this thread launched (for launch accounting). */
int qw_last_launch_count(void);
/* Name of the attention kernel that the last attention call on this thread launched: "splitkv_kernel"
 * (mma.sync), "splitkv_umma_kernel" or "prefill_umma_pair_kernel" (tcgen05); "" if it launched none.
 * For tests and benchmarks that must know which kernel a route reaches.  No counterpart in the reference. */
const char *qw_last_attention_kernel(void);

/* Instrumentation for benchmarks.  While enabled (per host thread), every attention call
 * records a CUDA event pair around its dominant kernel (split-KV or tcgen05 prefill) on the
 * launching stream.  qw_profile_last_kernel_ms() waits for that kernel and returns its
 * duration; not for use inside a stream capture.  Enabling creates the two events once.
 * No counterpart in the reference, which times whole graphs (bench/spec_budget.cu:38-54). */
int qw_profile_enable(int on);
int qw_profile_last_kernel_ms(float *ms);

/* The fused mixer fed by the layer's fused q/k/v projection, i.e. with the launches that the reference
 * puts between that GEMM and attention folded in: unpack3 (src/model.cu:221, src/elem.cu:226-237),
 * k_split_qgate (src/model.cu:223-224, src/mixers.cu:382-390) and the two k_rmsnorm_head launches
 * (src/model.cu:225-226, src/mixers.cu:393-413; weights are used as 1 + w).  `fused` holds one row per new
 * token, [ (q[256] | gate[256]) x q_heads | k[kv_heads][256] | v[kv_heads][256] ], fp32 (the reference's GEMM
 * output, fused_is_f32 = 1) or bf16.  d->q and d->gate are OUTPUT scratch of n_seq * n_new * q_heads * 256 bf16
 * each (normalised query and gate, consumed by the attention kernel of the same call); d->k_new and d->v_new
 * are ignored.  d->flags must contain QW_F_APPEND; q_norm_w / k_norm_w are the 256 bf16 weights of q_norm /
 * k_norm, eps the reference's RMS_EPS (qwen38.h:32).  Same return codes as qw_mixer_forward. */
int qw_mixer_forward_fused(const qw_mixer_desc *d, const void *fused, int fused_is_f32, const qw_bf16 *q_norm_w,
                           const qw_bf16 *k_norm_w, float eps, qw_stream stream);

/* ------------------------------------------------------------------------------------------
 * Cross-GPU split-KV combine (used only where one sequence's KV range is split across GPUs)
 *
 * A partial is, per (row, q_head), QW_PARTIAL_FLOATS floats: o[256] un-normalised fp32,
 * m (running max of scale*log2(e)*score) and l (sum of exp2), then two pad floats.
 * qw_mixer_forward_partial() runs the mixer (any kernel but the tcgen05 prefill one: chunks of 64
 * rows or more use the split-KV kernels here) but emits partials [n_seq*n_new][q_heads][260]
 * instead of normalised output; after the ranks exchange them (NCCL, outside this library)
 * qw_combine_partials() merges n_parts of them, laid out [n_parts][rows][q_heads][260], in
 * index order (fixed order => bit-stable) and applies the gate (QW_F_GATE, QW_F_OUT_F32).
 * No counterpart in the reference (single GPU).
 * ---------------------------------------------------------------------------------------- */
#define QW_PARTIAL_FLOATS 260
int qw_mixer_forward_partial(const qw_mixer_desc *d, float *partial, qw_stream stream);
int qw_combine_partials(const float *parts, int n_parts, int64_t rows, int q_heads,
                        const qw_bf16 *gate, void *out, float *lse, int flags, qw_stream stream);

/* The same merge with the exchange done inside the kernel over NVLink peer memory instead of a collective in
 * front of it.  part_ptrs / flag_ptrs: device arrays of n_parts pointers, element k being THIS process's
 * mapping of rank k's partial buffer [rows][q_heads][260] and of rank k's flag word (symmetric memory, CUDA IPC
 * or any other peer mapping; the flag words start at zero).  Every rank calls it with the same `step`
 * (1, 2, 3, ...) after the launch that wrote its own partials on the same stream; the kernel publishes the step
 * in the rank's own flag, waits (at most two seconds, else *status = 106) until
 * every peer has published it, then reads the peers' partials in place.  The wait is per thread block: if
 * *status is 106 afterwards, blocks that saw the peers in time have written their rows and the others have
 * not, so the whole output must be treated as undefined.  Alternate two buffer / flag sets by
 * step parity.  No counterpart in the reference (single GPU). */
int qw_combine_partials_peer(const float *const *part_ptrs, int *const *flag_ptrs, int rank, int n_parts, int step,
                             int64_t rows, int q_heads, const qw_bf16 *gate, void *out, float *lse, int flags,
                             int *status, qw_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* QWENGINE_ATTN_H_ */
