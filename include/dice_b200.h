/*
 * dice_b200 — C ABI of the B200 (sm_100a) kernels behind the DiT-MoE block.
 *
 * The reference project (DICE) is pure Python on PyTorch and has no FFI of its
 * own; each entry point below states which reference lines it replaces (paths
 * relative to the reference project's root).  The Python host code in
 * dice_b200/ binds these with ctypes and mirrors the reference's module
 * interface on top of them.
 *
 * Conventions
 *  - every pointer is a DEVICE pointer owned by the caller unless stated;
 *    nothing here allocates, frees or synchronises;
 *  - work is enqueued on `stream` (a cudaStream_t passed as void*);
 *  - return value: 0 = enqueued, negative = argument error found on the host
 *    (nothing was enqueued); see dice_strerror();
 *  - kernels that wait on hardware barriers bound every wait; when a wait
 *    expires the kernel stores a non-zero code into the caller's `status`
 *    word, releases what it holds and returns.  The host reads the word when
 *    it next synchronises (dice_status_message() names the code);
 *  - row-major everywhere; "rows" are token-expert rows (one per routed
 *    (token, slot) pair) sorted by expert, "segments" are the per-expert runs
 *    of rows.
 */
#ifndef DICE_B200_H_
#define DICE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DICE_ABI_VERSION 2

#if defined(__GNUC__)
#define DICE_API __attribute__((visibility("default")))
#else
#define DICE_API
#endif

/* element types of activations and weights */
#define DICE_BF16 0
#define DICE_F32 1

/* expert activation variants */
#define DICE_ACT_SWIGLU 0    /* down(silu(gate(x)) * up(x))      models.py:271 */
#define DICE_ACT_GELU_TANH 1 /* fc2(gelu_tanh(fc1(x)))            no reference counterpart */

/* epilogue modes of dice_grouped_gemm */
#define DICE_EPI_STORE 0     /* out = A * W^T                                   */
#define DICE_EPI_GELU_TANH 1 /* out = gelu_tanh(A * W^T)                        */
#define DICE_EPI_SWIGLU 2    /* W holds 128-row gate/up blocks interleaved;
                                out[:, j] = silu(gate_j) * up_j                 */
/* (a fourth epilogue, the gate-weighted scatter-add into token rows, is reached
 *  through dice_grouped_ffn_combine only) */

/* error codes (negative) */
#define DICE_OK 0
#define DICE_ERR_ARG -1         /* null pointer, negative size                  */
#define DICE_ERR_SHAPE -2       /* unsupported shape / divisibility             */
#define DICE_ERR_DTYPE -3       /* unsupported element type                     */
#define DICE_ERR_ALIGN -4       /* pointer not 16-byte aligned                  */
#define DICE_ERR_SCRATCH -5     /* scratch buffer too small                     */
#define DICE_ERR_CUDA -6        /* a CUDA runtime/driver call failed            */
#define DICE_ERR_LIMIT -7       /* size beyond a documented maximum             */

DICE_API int dice_abi_version(void);
DICE_API const char* dice_strerror(int code);
/* text for a device status word written by a kernel (0 = "ok") */
DICE_API const char* dice_status_message(uint32_t status);
/* kernels this library has launched in this process so far (a benchmark reads
 * it before and after a region to report measured launches) */
DICE_API uint64_t dice_kernel_launches(void);

/* ---------------------------------------------------------------------------
 * Router: logits -> softmax -> top-2 (+ expert histogram), one fused kernel.
 * Replaces MoEGate.forward in eval mode (models.py:179-217: F.linear :184,
 * softmax :186, topk :191, optional renormalisation :194-196) and the
 * bincount of ep_fwd.py:70-76 / models.py:366.
 *   x        [n_tokens, hidden]   dtype
 *   w_gate   [n_experts, hidden]  dtype
 *   out_idx  [n_tokens, 2] int64  slot 0 = larger score; equal scores: lower
 *                                 expert index first
 *   out_w    [n_tokens, 2] fp32   softmax scores of the two (renormalised to
 *                                 sum 1 when renorm != 0)
 *   out_hist [n_experts]  int32   rows per expert (zeroed by the call; NULL to
 *                                 skip when out_chunk_hist is given)
 *   out_chunk_hist  optional [ceil(n_tokens / 128), n_experts] int32, bf16
 *                   only: rows per expert of every 128 tokens (every cell is
 *                   written), the input of dice_permute_plan_chunked
 *   out_logits  optional [n_tokens, n_experts] dtype (NULL to skip)
 * Logits are accumulated in fp32 and rounded to dtype before the softmax,
 * which is evaluated in fp32.  hidden*sizeof(dtype) must be a multiple of 16,
 * n_experts in [2, 64].  bf16 runs as a 128 x E tcgen05 tile per 128 tokens
 * with the selection in the epilogue, fp32 on the CUDA cores.  `status`
 * (device uint32, may be NULL) receives a code if a bounded wait expires;
 * tokens of a tile that gave up get expert -1 and weight 0 (fp32 kernel) or
 * are left unwritten (bf16 kernel).
 */
DICE_API int dice_router_top2(const void* x, const void* w_gate, int64_t n_tokens, int hidden, int n_experts,
                     int dtype, int renorm, int64_t* out_idx, float* out_w, int32_t* out_hist,
                     int32_t* out_chunk_hist, void* out_logits, uint32_t* status, void* stream);

/* The selection stage alone, on logits supplied by the caller (same outputs
 * as above).  Lets the selection be checked bit-exactly against
 * softmax+topk (models.py:186-196) on the reference's own logits. */
DICE_API int dice_top2_from_logits(const void* logits, int64_t n_tokens, int n_experts, int dtype, int renorm,
                          int64_t* out_idx, float* out_w, int32_t* out_hist, void* stream);

/* ---------------------------------------------------------------------------
 * Permutation plan: stable counting sort of rows by expert.
 * Replaces flat_expert_indices.argsort() + bincount (ep_fwd.py:70-76, :100;
 * models.py:365-366); the order inside an expert is the stable one.
 *   flat_idx        [n_rows] int64   expert of each (token, slot) row
 *   scratch         dice_permute_scratch_bytes(n_rows, n_experts) bytes
 *   out_pos         [n_rows] int32   row -> position in expert-sorted order
 *   out_order       [n_rows] int32   position -> row (NULL to skip)
 *   out_seg_offsets [n_experts+1] int32  first position of each expert's run
 * Rows whose expert is outside [0, n_experts) get position -1 and are
 * counted in no segment.
 */
DICE_API size_t dice_permute_scratch_bytes(int64_t n_rows, int n_experts);
DICE_API int dice_permute_plan(const int64_t* flat_idx, int64_t n_rows, int n_experts, void* scratch,
                      size_t scratch_bytes, int32_t* out_pos, int32_t* out_order,
                      int32_t* out_seg_offsets, void* stream);

/* The same plan in ONE launch, from the per-128-token histograms the bf16
 * router files (the two counting passes are already done), optionally with
 * the row gather of dice_permute_rows fused in (ep_fwd.py:70-76, :100,
 * :107-111; models.py:365-366, :374).
 *   chunk_hist  [ceil(n_rows / 256), n_experts] int32 as written by
 *               dice_router_top2 (a chunk = 128 tokens x 2 slots = 256 rows)
 *   world       1: rows are ordered by expert id; > 1: by (owner rank, local
 *               slot) of the round-robin placement of etrim.py:23-24, i.e. by
 *               key(e) = (e mod world) * (n_experts / world) + e / world, the
 *               order the expert-parallel exchange sends rows in;
 *               out_seg_offsets is then indexed by key
 *   x, k, hidden, dtype, out_rows   x == NULL: plan only; else also
 *               out_rows[out_pos[t*k + s]] = x[t]
 *   limit: ceil(n_rows / 256) * n_experts <= 16384 (DICE_ERR_LIMIT beyond; use
 *   dice_permute_plan + dice_permute_rows there). */
DICE_API int dice_permute_plan_chunked(const int64_t* flat_idx, const int32_t* chunk_hist, int64_t n_rows,
                              int n_experts, int world, int32_t* out_pos, int32_t* out_order,
                              int32_t* out_seg_offsets, const void* x, int k, int hidden, int dtype,
                              void* out_rows, void* stream);

/* Allocation-free variant of dice_permute_plan; it has no counterpart in the
 * reference.  It is for hosts that must not allocate device memory while they
 * run: a serving loop whose memory pool was sized and frozen at start-up, a
 * plug-in that is handed its caller's buffers and nothing else, or an
 * embedding application that enforces a fixed memory budget and treats any
 * cudaMalloc on the request path as an error.  Such a caller still passes the
 * input and the three outputs, but no scratch: the per-chunk histograms live
 * in a fixed 256 KB array inside the library (present on every GPU that loads
 * it, until the process exits).
 *   limit: ceil(n_rows / 256) * n_experts <= DICE_PLAN_STATIC_MAX_INTS
 *          (2 M rows at 8 experts, 262144 rows at 64); larger requests return
 *          DICE_ERR_LIMIT and enqueue nothing.
 *   The first call on a device looks up the array's address (once per device,
 *   with that device current); that first call should come before any stream
 *   capture.  The call never calls cudaMalloc, cudaFree or an allocating
 *   library routine.
 *   All calls share the one array, which keeps the previous call's contents;
 *   every cell that is read is rewritten first by the same call, so nothing
 *   needs clearing, but two calls that overlap on the GPU (different streams,
 *   or host threads without ordering between them) race on it: serialise them.
 *   The address is remembered per device for the life of the process: do not
 *   use the entry point across a cudaDeviceReset.
 * Outputs are identical to dice_permute_plan's. */
#define DICE_PLAN_STATIC_MAX_INTS 65536
DICE_API int dice_permute_plan_static(const int64_t* flat_idx, int64_t n_rows, int n_experts,
                             int32_t* out_pos, int32_t* out_order, int32_t* out_seg_offsets,
                             void* stream);

/* Row gather into expert-sorted order (ep_fwd.py:107-111, :344-347;
 * models.py:374): out_rows[pos[t*k + s]] = x[t] for s < k.  Negative
 * positions are skipped. */
DICE_API int dice_permute_rows(const void* x, const int32_t* pos, int64_t n_tokens, int k, int hidden,
                      int dtype, void* out_rows, void* stream);

/* ---------------------------------------------------------------------------
 * Un-permute + gate-weighted sum of a token's two rows (+ optional addend).
 * Replaces _local_combine (ep_fwd.py:349-354), the conditional-communication
 * merge (ep_fwd.py:177-187), mul_ by the gate weights (:190-193) and the
 * pair sum (:195); on one device the mul_/scatter_reduce_ of
 * models.py:377-381 and the shared-expert add of models.py:357.
 *   y[t]   = w0[t*w_stride] * src0[i0] + w1[t*w_stride] * src1[i1] + addend[t]
 *   out[t] = resid[t] + gate[t / tokens_per_sample] * y[t]
 * with i0 = idx0 ? idx0[t*idx0_stride] : t (same for i1).  src1 == NULL drops
 * the second term, w0/w1 == NULL mean weight 1, addend == NULL means 0.
 * A negative index contributes 0.  Sums are formed in fp32.
 * resid [n_tokens, hidden] and gate [n_samples, hidden] (either may be NULL:
 * no residual / gate 1) fold the DiT block's gated residual around the MoE
 * block, x + gate_mlp.unsqueeze(1) * moe(...) (models.py:519), into the same
 * pass.
 */
DICE_API int dice_unpermute_combine(const void* src0, const int32_t* idx0, int idx0_stride, const void* src1,
                           const int32_t* idx1, int idx1_stride, const float* w0, const float* w1,
                           int w_stride, const void* addend, const void* resid, const void* gate,
                           int tokens_per_sample, int64_t n_tokens, int hidden, int dtype, void* out,
                           void* stream);

/* ---------------------------------------------------------------------------
 * The DiT block's input glue in one pass (models.py:75-76, :494, :519):
 *   out[t] = LayerNorm(x[t]) * (1 + scale[b]) + shift[b],  b = t / tokens_per_sample
 * LayerNorm over `hidden` without affine parameters, statistics in fp32 (two
 * passes over the row, which stays in registers); x, shift [n_samples, hidden]
 * and scale have element type `dtype`, out has `out_dtype` (bf16 -> bf16,
 * fp32 -> fp32 or fp32 -> bf16).  hidden <= 2048.
 */
DICE_API int dice_ln_modulate(const void* x, const void* shift, const void* scale, int64_t n_tokens, int hidden,
                     int tokens_per_sample, float eps, int dtype, int out_dtype, void* out, void* stream);

/* ---------------------------------------------------------------------------
 * Expert weights.  SwiGLU experts (models.py:246-247) are packed once at load
 * time so that one 256-wide output tile of the first GEMM holds 128 gate and
 * the matching 128 up columns:
 *   out_w13 [dice_w13_rows(ffn), hidden]; block j = gate[128j:128j+128] then
 *   up[128j:128j+128]; rows beyond ffn are zero.
 */
DICE_API int64_t dice_w13_rows(int ffn);
DICE_API int dice_pack_w13(const void* gate_proj, const void* up_proj, int hidden, int ffn, int dtype,
                  void* out_w13, void* stream);

/* ---------------------------------------------------------------------------
 * Grouped (per-segment) GEMM on the 5th-generation tensor cores:
 *   out[r, :] = epilogue( a[r, :] * w[slab(seg(r))]^T )
 * Replaces the per-expert nn.Linear calls driven from Python loops
 * (ep_fwd.py:199-211, models.py:368-376, MoeMLP.forward models.py:252-273).
 *   a            [n_rows, k_dim]            bf16, 16-byte aligned
 *   w            [n_slabs, w_rows, k_dim]   bf16 (nn.Linear layout: out x in)
 *   seg_offsets  [n_seg+1] int32 (device)   rows of segment s are
 *                                           [seg_offsets[s], seg_offsets[s+1])
 *   seg_slab     [n_seg] int32 (device) weight slab of each segment, or NULL
 *                                           for slab = segment index
 *   out          [n_rows, ld_out]           bf16; columns [0, n_out)
 *   n_out        logical output width: w_rows for STORE/GELU_TANH, ffn for
 *                SWIGLU (where w_rows = dice_w13_rows(ffn))
 *   reserve_sms  SMs the persistent kernel leaves free for kernels of other
 *                streams (0 = use the whole GPU).  The asynchronous exchange
 *                runs its pushes on those SMs next to the expert FFN
 *                (diep.py:219-259, :284-310 overlap the all-to-all with compute).
 *   status       device uint32, non-zero after a bounded wait expired
 * k_dim, ld_out, n_out multiples of 8; n_seg <= 256.  The tile list is derived
 * on the device from seg_offsets, so no host synchronisation is needed.
 */
DICE_API int dice_grouped_gemm(const void* a, int64_t n_rows, int k_dim, const void* w, int n_slabs,
                      int64_t w_rows, const int32_t* seg_offsets, const int32_t* seg_slab, int n_seg,
                      int epilogue, void* out, int64_t ld_out, int n_out, int reserve_sms,
                      uint32_t* status, void* stream);

/* The expert FFN over expert-sorted rows: two dice_grouped_gemm launches
 * (ep_fwd.py:199-211 proc_experts; models.py:368-376).
 *   act = DICE_ACT_SWIGLU   : w1 = packed gate/up [n_slabs, dice_w13_rows(ffn), hidden]
 *   act = DICE_ACT_GELU_TANH: w1 = fc1 [n_slabs, ffn, hidden]
 *   w2  [n_slabs, hidden, ffn];  inter = caller's scratch [n_rows, ffn] bf16.
 * The block's always-on shared expert (models.py:292-296, :355-357: one more
 * expert of width shared_ffn applied to EVERY token) can ride in the same two
 * launches as an extra problem at the end of the tile list, where its tiles
 * fill the routed experts' partly empty last wave:
 *   shared_in  [n_shared, hidden] the tokens (NULL: no shared expert),
 *   shared_w1 / shared_w2 as w1 / w2 for one slab of width shared_ffn,
 *   shared_inter [n_shared, shared_ffn] scratch, shared_out [n_shared, hidden].
 *   rows_done  NULL, or device counters (zero on entry), one per 256-row block
 *              of the second GEMM's tile list (block b of segment g: rows
 *              [256 b, 256 b + 256) of the segment; segments in order, those
 *              without rows or without weights take no block; at most
 *              n_rows / 256 + n_seg blocks).  Every finished tile adds 16 to its
 *              block's counter after its stores are visible device-wide, so a
 *              block is complete at 16 * ceil(hidden / 256).  A kernel on another
 *              stream (dice_ep_return_rows_following) can then send rows on
 *              while later blocks are still being computed.
 *   first_gemm_done  NULL, or (with rows_done) a cudaEvent_t that is recorded on
 *              `stream` between the two GEMMs; then only the second GEMM leaves
 *              reserve_sms SMs free.  The stream of the following push waits
 *              for this event, so that the push takes its SMs when the first
 *              GEMM has left them, not before.
 */
DICE_API int dice_grouped_ffn(const void* rows_in, int64_t n_rows, int hidden, int ffn, int act, const void* w1,
                     const void* w2, int n_slabs, const int32_t* seg_offsets, const int32_t* seg_slab,
                     int n_seg, void* inter, void* rows_out, const void* shared_in, int64_t n_shared,
                     int shared_ffn, const void* shared_w1, const void* shared_w2, void* shared_inter,
                     void* shared_out, int reserve_sms, uint32_t* rows_done, void* first_gemm_done,
                     uint32_t* status, void* stream);

/* The expert FFN whose second GEMM also does the weighted combine
 * (models.py:377-381: mul_ by the gate weights, scatter_reduce_ into the token
 * rows): every output row is scaled by its gate weight in the epilogue and
 * added to its token's row of out_tokens with 16-byte bf16 reductions, so the
 * expert outputs are never stored in sorted order and no combine kernel runs.
 *   order        [n_rows] int32   sorted position -> flat (token, slot) row, as
 *                                 written by the plan entry points
 *   row_weights  [n_rows] fp32    gate weight of every flat row (topk_weight
 *                                 viewed flat)
 *   out_tokens   [n_rows / k, hidden] bf16; zeroed by the call
 * k must be 2: a token's row then receives exactly two addends on top of zero,
 * and since that sum does not depend on which arrives first the result is the
 * same bits in every run (each addend is rounded to bf16 before the add).  With
 * a third addend (the shared expert, a residual) it would not be; those blocks
 * keep dice_unpermute_combine.  bf16 only, on one GPU (the expert-parallel
 * path returns rows to other ranks instead). */
DICE_API int dice_grouped_ffn_combine(const void* rows_in, int64_t n_rows, int hidden, int ffn, int act,
                             const void* w1, const void* w2, int n_slabs, const int32_t* seg_offsets,
                             const int32_t* seg_slab, int n_seg, void* inter, const int32_t* order,
                             const float* row_weights, int k, void* out_tokens, int reserve_sms,
                             uint32_t* status, void* stream);

/* fp32 variant of the expert FFN on the CUDA cores (no tensor-core rounding;
 * used where fp32 parity at 1e-5 is asked for).  Same arguments as
 * dice_grouped_ffn with fp32 tensors; SwiGLU takes the packed layout too. */
DICE_API int dice_grouped_ffn_f32(const void* rows_in, int64_t n_rows, int hidden, int ffn, int act,
                         const void* w1, const void* w2, int n_slabs, const int32_t* seg_offsets,
                         const int32_t* seg_slab, int n_seg, void* inter, void* rows_out,
                         void* stream);

/* ---------------------------------------------------------------------------
 * Expert-parallel exchange over NVLink peer memory (one process per GPU, one
 * box).  Replaces, for the synchronous exchange, exchange_token_counts
 * (ep_fwd.py:214-245), global_dispatch (:247-293) and global_combine (:295-342)
 * together with the host synchronisations they need for split sizes.
 * Peers' buffers are mapped with dice_ipc_export / dice_ipc_import at set-up;
 * `peer_*` arguments are HOST arrays of `world` device pointers (entry `rank`
 * is this rank's own buffer).  A rank only writes into peer memory and raises
 * flags there; waits are bounded and report through `status`.
 *   keys are (owner rank, local slot) = owner * (n_experts / world) + slot, so
 *   seg_offsets [n_experts+1] (from dice_permute_plan on those keys) lists this
 *   rank's rows per destination;
 *   flag arrays: every entry of a `peer_flags` table points at 64 uint32 words
 *   of that peer: [0, world) the flags, [32, 32 + world) failure marks (a push
 *   that could not complete writes its sequence number there before raising the
 *   flag; the waiting peer then records "a peer rank reported ...");
 *   meta: int32 [dice_ep_meta_ints(world, n_experts/world)]: total rows
 *   received | state (0 ok, 1 a receive buffer is too small, 2 the peers'
 *   counts never arrived) | send_base[W] | back_base[W] | src_off[W+1] |
 *   src_cnt[W] | seg_off[...] (segments of the receive buffer, ready for
 *   dice_grouped_ffn).
 *   Two layouts of a receive buffer:
 *   - packed (region_rows == 0): the sources' blocks follow one another; a
 *     source learns where its block starts from everyone's counts, so
 *     dice_ep_exchange_counts (a rendezvous of all ranks) runs first and writes
 *     meta; W*El segments in (source, slot) order, seg_slab[s*El+i] = i.  Every
 *     rank holds the whole count matrix, so a receive buffer that is too small
 *     ANYWHERE is found by every rank: all of them record the overflow status
 *     and the exchange then moves no rows;
 *   - regions (region_rows > 0, capacity_rows >= world * region_rows,
 *     region_rows >= the rows any rank ever sends): source s owns rows
 *     [s*region_rows, (s+1)*region_rows) of every receive buffer.  No count
 *     exchange: dice_ep_dispatch_rows publishes this rank's counts with its
 *     rows, dice_ep_wait_dispatch waits for the sources and derives meta;
 *     W*(El+1) segments, seg_slab[s*(El+1)+i] = i for i < El and -1 for the
 *     unused rest of a region (the GEMM skips it).  Like the reference's
 *     all_to_all, it cannot drop a row;
 *   seq: a number that grows with every use of the same buffers;
 *   done_counter: device uint32, zero before first use, one per call site;
 *   max_ctas selects the form of a push: 0 = the push has the GPU to itself:
 *   rows move through shared memory with the copy unit (cp.async.bulk), one
 *   warp per SM; > 0 = the same with at most that many CTAs (rounded up to an
 *   even number, four warps each), for a push that runs on another stream next
 *   to an expert FFN which was given reserve_sms = max_ctas; -1 = SIMT push (no
 *   shared memory) sized by the rows, < -1 = SIMT push of at most -max_ctas CTAs.
 */
DICE_API int dice_ep_meta_ints(int world, int n_local_experts);
DICE_API int dice_ep_exchange_counts(const int32_t* seg_offsets, const void* const* peer_matrices,
                            const void* const* peer_flags, int32_t* meta, int rank, int world,
                            int n_experts, int capacity_rows, uint32_t seq, uint32_t* status,
                            void* stream);
/* permutation gather fused with the dispatch: row (t, s) goes straight into its
 * expert owner's receive buffer (ep_fwd.py:107-111 + :277-291) */
DICE_API int dice_ep_dispatch_rows(const void* x, const int32_t* pos, const int32_t* seg_offsets,
                          const int32_t* meta, const void* const* peer_recv,
                          const void* const* peer_flags, uint32_t* done_counter, int64_t n_tokens,
                          int k, int hidden, int dtype, int rank, int world, int n_experts,
                          int capacity_rows, uint32_t seq, int max_ctas, int region_rows,
                          const void* const* peer_matrices, uint32_t* status, void* stream);
/* region layout: wait (bounded) for every source's rows and failure marks, then
 * derive `meta` from the count matrix the sources published (my_matrix: this
 * rank's own [world][n_experts] matrix) */
DICE_API int dice_ep_wait_dispatch(const uint32_t* my_flags, const int32_t* my_matrix, int32_t* meta, int rank,
                          int world, int n_experts, int region_rows, uint32_t seq, uint32_t* status,
                          void* stream);
/* How long the exchange kernels of the CURRENT device wait for another rank (or,
 * in dice_ep_return_rows_following, for the GEMM) before they record the
 * expired wait and return: 2000 ms by default, 100 ms .. 1 h accepted.  The
 * reference's collectives wait for as long as the process group's timeout
 * (ep_fwd.py:277-291 via torch.distributed); raise the limit where ranks may
 * stall for seconds between two exchanges. */
DICE_API int dice_ep_set_wait_limit_ms(int milliseconds);
/* wait (bounded) until every source raised flag >= seq, then look at the
 * sources' failure marks; what: 0 dispatch, 1 combine; + 2: the kernel is
 * launched in plain stream order (it, and what follows it in the stream, does
 * not become resident while the kernel before it runs: needed behind an FFN
 * that leaves SMs free for dice_ep_return_rows_following) */
DICE_API int dice_ep_wait_flags(const uint32_t* my_flags, int world, uint32_t seq, int what,
                       uint32_t* status, void* stream);
/* expert outputs back to the token owners, in the order the rows were sent
 * (ep_fwd.py:326-340); max_rows = rows the buffer `rows` holds (nothing beyond
 * it is read) */
DICE_API int dice_ep_return_rows(const void* rows, const int32_t* meta, const void* const* peer_back,
                        const void* const* peer_flags, uint32_t* done_counter, int hidden, int dtype,
                        int rank, int world, int back_capacity_rows, int max_rows, uint32_t seq,
                        int max_ctas, uint32_t* status, void* stream);
/* The same return (bf16 rows, bulk-copy form on max_ctas > 0 CTAs), launched on a
 * second stream right AFTER dice_grouped_ffn(..., rows_done, first_gemm_done)
 * was launched with reserve_sms >= max_ctas, the second stream waiting for
 * first_gemm_done (after its producer, so that the push never depends on a
 * launch the host has yet to make: the first launch of a kernel may load its
 * module, which can wait for running kernels).  A chunk of rows leaves as
 * soon as the blocks of the
 * second GEMM's output that it lies in are complete, so that the transfer of the
 * synchronous all-to-all (ep_fwd.py:326-340) hides under the GEMM that produces
 * its rows.  seg_slab / n_seg: the segment table the GEMM runs with (n_seg a
 * multiple of world, at most 288; segments of one source are consecutive).  The
 * last CTA clears rows_done[0, rows_done_ints) before it raises the flags.  A
 * block that does not complete within the wait limit raises status 11. */
DICE_API int dice_ep_return_rows_following(const void* rows, const int32_t* meta, const void* const* peer_back,
                        const void* const* peer_flags, uint32_t* done_counter, int hidden, int rank,
                        int world, int back_capacity_rows, int max_rows, uint32_t seq, int max_ctas,
                        uint32_t* rows_done, int rows_done_ints, const int32_t* seg_slab, int n_seg,
                        uint32_t* status, void* stream);
/* The expert FFN fused with the return: same as dice_grouped_ffn over the
 * receive buffer, but the second GEMM's epilogue stores every output row
 * straight into the combine buffer of the rank that owns the token (NVLink
 * peer stores) and the last CTA raises the peers' flags: proc_experts
 * (ep_fwd.py:199-211) + global_combine (:295-342) in one launch pair.  `meta`,
 * `peer_back`, `peer_flags`, `done_counter`, `seq` as for dice_ep_return_rows. */
DICE_API int dice_grouped_ffn_return(const void* rows_in, int64_t n_rows, int hidden, int ffn, int act,
                            const void* w1, const void* w2, int n_slabs, const int32_t* seg_offsets,
                            const int32_t* seg_slab, int n_seg, void* inter, const int32_t* meta,
                            const void* const* peer_back, const void* const* peer_flags,
                            uint32_t* done_counter, int rank, int world, int back_capacity_rows,
                            uint32_t seq, int reserve_sms, uint32_t* status, void* stream);
/* CUDA IPC plumbing for the above (set-up time): export the allocation that
 * holds `ptr` (64-byte handle + offset of ptr inside it); import maps a peer's
 * allocation into this process and enables peer access. */
DICE_API int dice_ipc_export(const void* ptr, uint8_t* out_handle64, uint64_t* out_offset);
DICE_API int dice_ipc_import(const uint8_t* handle64, uint64_t offset, void** out_ptr);
DICE_API int dice_ipc_close(void* imported_ptr, uint64_t offset);

#ifdef __cplusplus
}
#endif
#endif /* DICE_B200_H_ */
