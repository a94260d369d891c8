/*
 * C ABI of the B200 (sm_100a) triangle-multiplicative-update forward path.
 *
 * What it replaces in the reference project (CSSB-SNU/MiniWorld): the engine operator behind
 * `TriangleMultiplication.forward(pair, mask)`, whose functional entry is
 * `b200_infer.inference(leaves[11], flat_mask, flat_scale, direction)`
 * (benchmarks/engine_ops/trimul_batch.py:24-39,66; direction 1 = outgoing, 2 = incoming), called by
 * src/miniworld/blocks/msa_module.py:116-117, src/miniworld/blocks/template.py:84-85 and the
 * FoldForge Pairformer block (benchmarks/protenix_finetune/patch_engine.py:89-90).
 *
 * Conventions
 *  - All pointers are device pointers unless the name says `host`. Activations are bf16, LayerNorm
 *    affine vectors fp32, linear weights bf16 or fp32 (`weight_dtype`), masks uint8 (non-zero = valid).
 *  - Widths: d_pair = d_hidden = 128 (every direction), and through b200_trimul_forward / _forward_ex / _forward_static
 *    also d_pair = 64 with 128 contracted channels in total: d_hidden = 128 for one direction (the template blocks,
 *    benchmarks/protenix_finetune/patch_engine.py:283-295) or d_hidden = 64 per direction for the bidirectional
 *    module. Anything else is B200_TRIMUL_E_UNSUPPORTED. The staged entry points (pack, prologue, epilogue) are
 *    128-wide.
 *    N must be a multiple of 8 (16-byte rows for the bulk copies); callers pad with masked tokens.
 *  - The caller owns every buffer, including the workspace; the library never allocates or frees
 *    device memory. Its only process-wide state is a set of caches that are filled on first use and
 *    never change afterwards (a driver entry point, the SM count of each device, which kernels have had
 *    their shared-memory size enabled on which device) plus, for b200_trimul_forward_static alone, one
 *    fixed scratch array per GPU and its cached device address. Calls are asynchronous on `cuda_stream`
 *    and may be issued from any host thread.
 *  - Magnitudes: left / right and the normalised input are rounded to fp16 with saturation (a value past
 *    +-65504 becomes +-65504, never infinity), tri likewise after its 2^-4 scaling, so the output stays
 *    finite for any finite input; results match the fp32 module to the stated bounds while
 *    |sigmoid(g) * p| < 65504 and |t| < 2^20, which holds with a wide margin for LayerNorm-ed activations.
 *    Linear weights are held as fp16(0.5 W): entries below about 1.2e-7 in magnitude flush to zero and
 *    entries below 1.2e-4 lose precision gradually (fp16 subnormals).
 *  - Return value: 0 on success, a negative B200_TRIMUL_E_* code otherwise. Device-side waits are
 *    bounded; if one runs out the kernels finish, and `b200_trimul_read_status` reports a positive
 *    device code (101 producer, 102 MMA issuer, 103 epilogue, 104 statistics, 105 drain, 106 barrier between GPUs).
 *  - Intermediate layout ("row-plane"): left / right / tri are [B, rows, 128, N] fp16, i.e. for every
 *    pair row a [channel, column] slab. fp16 (same tensor-core rate as bf16, three more mantissa bits)
 *    is what keeps the bf16 module output inside its max-abs bound; tri holds t * 2^-4, saturated to
 *    the fp16 range.
 */
#ifndef B200_TRIMUL_H_
#define B200_TRIMUL_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_TRIMUL_BIDIRECTIONAL 0 /* both of the above in one module: see b200_trimul_forward_ex */
#define B200_TRIMUL_OUTGOING 1 /* t_ij = sum_k a_ik b_jk  (einsum bikd,bjkd->bijd) */
#define B200_TRIMUL_INCOMING 2 /* t_ij = sum_k a_ki b_kj  (einsum bkid,bkjd->bijd) */

#define B200_TRIMUL_DTYPE_BF16 0
#define B200_TRIMUL_DTYPE_F32 1

#define B200_TRIMUL_OK 0
#define B200_TRIMUL_E_NULL (-1)        /* a required pointer is null */
#define B200_TRIMUL_E_SHAPE (-2)       /* bad B / N / rows / direction */
#define B200_TRIMUL_E_UNSUPPORTED (-3) /* a width outside the list above, N not a multiple of 8 */
#define B200_TRIMUL_E_ALIGN (-4)       /* a pointer is not 16-byte aligned (workspace: 1024) */
#define B200_TRIMUL_E_WORKSPACE (-5)   /* workspace too small */
#define B200_TRIMUL_E_CUDA (-6)        /* a CUDA runtime / driver call failed; see b200_trimul_last_cuda_error */
#define B200_TRIMUL_E_DEVICE (-7)      /* not an sm_100 device */
#define B200_TRIMUL_E_TOO_LARGE (-8)   /* b200_trimul_forward_static: B * N * N above its fixed limit */

/* Library version (major * 100 + minor). */
int b200_trimul_version(void);

/* Human-readable text for a status code (host or device). Never null. */
const char* b200_trimul_strerror(int code);

/* Last cudaError_t seen by this thread inside the library (0 if none). */
int b200_trimul_last_cuda_error(void);

/* Bytes of workspace needed by b200_trimul_forward for a full (unsharded) call. */
int b200_trimul_workspace_bytes(int B, int N, int d_pair, int d_hidden, int direction, size_t* out_bytes);

/* Offsets (bytes) of the regions inside a workspace: [0] status words, [1] packed weights,
 * [2] left, [3] right, [4] tri. For tests and profilers that want to look at the stages. */
int b200_trimul_workspace_layout(int B, int N, size_t out_offsets[5]);

/* Bytes of the packed-weight block written by b200_trimul_pack_weights. */
size_t b200_trimul_packed_bytes(void);

/*
 * Fold the LayerNorm affines into the six linears and write the packed block the kernels read.
 * Replaces the engine's per-call `weight.to(pair.dtype)` casts and `prepack_lr_operand`
 * (docs/archive/trimul-fusion/training-audit/harness/benchmarks/runners/bench.py:646-651).
 * `bias_opt` is null or an array of six device pointers (left, left_gate, right, right_gate, gate, out),
 * each null or fp32[128]; null everywhere is the reference layout (bias-free linears).
 */
int b200_trimul_pack_weights(const void* w_left, const void* w_left_gate, const void* w_right,
                             const void* w_right_gate, const void* w_gate, const void* w_out, int weight_dtype,
                             const float* ln_in_w, const float* ln_in_b, const float* ln_out_w,
                             const float* ln_out_b, const void* const* bias_opt, void* packed, void* cuda_stream);

/*
 * Stage 1: LayerNorm + gated left/right projections + mask, for `rows` pair rows of each sample.
 * z: [B, rows, N, 128] bf16 (rows row_begin .. row_begin+rows-1 of the full pair tensor);
 * token_mask: [B, N] uint8 or null; pair_mask: [B, rows, N] uint8 (the same rows as z) or null;
 * left / right: [B, rows, 128, N] fp16. `has_bias`: non-zero iff `packed` was built with a bias on any of the
 * four left/right linears. `status` is a device int (e.g. the workspace start).
 */
int b200_trimul_prologue(const void* z, const void* packed, const uint8_t* token_mask, const uint8_t* pair_mask,
                         void* left, void* right, int B, int N, int row_begin, int rows, float eps_in,
                         int has_bias, int* status, void* cuda_stream);

/*
 * Stage 2: per-channel contraction for output rows row_begin .. row_begin+rows-1.
 * outgoing: left is [B, rows, 128, N] (the local rows), right is [B, N, 128, N] (all rows).
 * incoming: left and right are both [B, N, 128, N] (all rows k).
 * tri: [B, rows, 128, N] fp16 (t * 2^-4). Replaces the `torch.bmm` every reference backend uses for this step
 * (docs/archive/trimul-fusion/inference.md:17).
 */
int b200_trimul_contract(const void* left, const void* right, void* tri, int B, int N, int row_begin, int rows,
                         int direction, int* status, void* cuda_stream);

/*
 * Gradients of stage 2 with respect to its operands (the reference's backward runs these four products as cuBLAS
 * calls, "B5-B6" in docs/kernels/trimul/TRIMUL_STATUS.md:47): given dtri = d loss / d tri in the layout of `tri`
 * ([B, N, 128, N] fp16, in any scale the caller chose so that it fits fp16),
 *   outgoing:  dleft[b,i,h,k] = sum_j dtri[b,i,h,j] right[b,j,h,k],   dright[b,j,h,k] = sum_i dtri[b,i,h,j] left[b,i,h,k]
 *   incoming:  dleft[b,k,h,i] = sum_j dtri[b,i,h,j] right[b,k,h,j],   dright[b,k,h,j] = sum_i dtri[b,i,h,j] left[b,k,h,i]
 * written like every contraction output of this library: times 2^-4, saturated to the fp16 range. Whole tensors only
 * (all N rows). Two launches of the stage-2 kernels; one of the four products has a K-major and an MN-major operand.
 */
int b200_trimul_contract_backward(const void* dtri, const void* left, const void* right, void* dleft, void* dright,
                                  int B, int N, int direction, int* status, void* cuda_stream);

/*
 * Stage 2, partial form for the incoming direction when the pair rows k are spread over several GPUs:
 * left / right: [B, k_rows, 128, N] fp16, the k_rows pair rows this GPU holds (any contiguous slab of k);
 * tri_partial: [B, N, 128, N] fp16 = 2^-4 * sum over those k of left[k, :, i] * right[k, :, j] for ALL (i, j).
 * Summing the partials of all slabs (a reduce-scatter over GPUs) gives the `tri` of b200_trimul_contract.
 * No reference counterpart: the reference runs this module on one GPU only
 * (docs/archive/trimul-fusion/inference.md:17 is the single-GPU bmm this replaces).
 */
int b200_trimul_contract_partial(const void* left, const void* right, void* tri_partial, int B, int N, int k_rows,
                                 int* status, void* cuda_stream);

/*
 * Multi-GPU forms (pair rows spread over the GPUs of one node, B = 1). No reference counterpart: the reference
 * runs this module on one GPU only; these replace the NCCL all-gather / reduce-scatter a row-sharded run would
 * otherwise place between the stages.
 *
 * b200_trimul_prologue_push: stage 1 for this GPU's rows, with `right` written straight into the gathered copies
 * [N, 128, N] fp16 of every GPU: `right_all` is this GPU's copy, right_all_peers[0 .. n_peers-1] (n_peers <= 7)
 * are the other GPUs' copies mapped into this process (peer memory). Local row r lands at row row_begin + r.
 * `left` stays local, [rows, 128, N]. The peers may read their copy once this call's kernel has completed on this
 * GPU and they have been told so (a stream-ordered collective, an event): the caller provides that ordering.
 *
 * b200_trimul_reduce_partials: tri[rows, 128, N] = sum over s of partials[s][row_begin .. row_begin+rows-1], where
 * partials[s] (s < n_src <= 8) is the [N, 128, N] fp16 output of b200_trimul_contract_partial on GPU s (local or
 * peer memory). fp32 sums in the order given, one saturating fp16 rounding.
 */
int b200_trimul_prologue_push(const void* z, const void* packed, const uint8_t* token_mask, const uint8_t* pair_mask,
                              void* left, void* right_all, void* const* right_all_peers, int n_peers, int N,
                              int row_begin, int rows, float eps_in, int has_bias, int* status, void* cuda_stream);
int b200_trimul_reduce_partials(void* tri, const void* const* partials, int n_src, int N, int row_begin, int rows,
                                void* cuda_stream);

/*
 * Channel-sharded multi-GPU form (B = 1, P GPUs, P divides 128, N/P a multiple of 32, N >= 256): GPU g contracts
 * the 128/P channels of group g for ALL rows, so each GPU sends 1/P of its operands and receives 1/P of the result
 * instead of (P-1)/P of an operand. No reference counterpart (single-GPU module). The three stages store directly
 * into the destination GPUs' buffers (plain TMA stores; peer memory mapped into the calling process for the other
 * GPUs); the caller orders stage s on all GPUs before stage s+1 on any (stream-ordered collective or events).
 *
 * b200_trimul_prologue_channels: stage 1 for this GPU's rows row_begin .. row_begin+rows-1. left_groups[g] /
 *   right_groups[g] (g < groups = P): GPU g's operand buffers [N, 128/P, N] fp16; this call fills rows row_begin.. .
 * b200_trimul_contract_channels: stage 2 on GPU `group`: left_group / right_group are its [N, 128/P, N] buffers,
 *   complete once every GPU's stage 1 has finished. tri_owners[s] (s < groups): GPU s's buffer
 *   [P, N/P, 128/P, N] fp16; rows s*N/P .. of the result go to slab `group` of tri_owners[s].
 * b200_trimul_epilogue_groups: stage 3 for this GPU's rows; tri_groups is its [P, rows, 128/P, N] buffer, complete
 *   once every GPU's stage 2 has finished; z / y: [rows, N, 128] bf16.
 */
/*
 * Barrier between the GPUs of a multi-GPU run, on the stream: everything this GPU enqueued before the call has
 * completed, and every other GPU has reached its call with the same `epoch`, before anything enqueued after it
 * starts. flags[r] (r < world <= 8) is GPU r's flag array (int32[8], zeroed once before the first barrier) as
 * mapped into this process (flags[rank] is this GPU's own). `epoch` grows by one per barrier. One tiny kernel: it
 * writes `epoch` into slot `rank` of every peer's array and polls its own array until every peer's slot has reached
 * `epoch`; after `timeout_ms` of waiting it gives up, records device code 106 in `status` and returns, so the
 * context stays usable. No reference counterpart; replaces a one-element NCCL all-reduce (about 20 us) where the
 * data itself already moves through peer memory.
 */
int b200_trimul_peer_barrier(int* const* flags, int rank, int world, int epoch, int timeout_ms, int* status,
                             void* cuda_stream);

int b200_trimul_prologue_channels(const void* z, const void* packed, const uint8_t* token_mask, void* const* left_groups,
                                  void* const* right_groups, int groups, int N, int row_begin, int rows, float eps_in,
                                  int has_bias, int* status, void* cuda_stream);
int b200_trimul_contract_channels(const void* left_group, const void* right_group, void* const* tri_owners, int groups,
                                  int group, int N, int direction, int* status, void* cuda_stream);
int b200_trimul_epilogue_groups(const void* tri_groups, const void* z, const void* packed, void* y, int N, int rows,
                                int groups, float eps_in, float eps_out, int residual, int* status, void* cuda_stream);

/*
 * Stage 3: output LayerNorm + output projection + sigmoid output gate (+ residual) for `rows` rows.
 * tri: [B, rows, 128, N] fp16 as written by stage 2; z, y: [B, rows, N, 128] bf16. y may alias z.
 */
int b200_trimul_epilogue(const void* tri, const void* z, const void* packed, void* y, int B, int N, int rows,
                         float eps_in, float eps_out, int residual, int* status, void* cuda_stream);

/*
 * Whole forward on one device: pack -> prologue -> contract -> epilogue, all on `cuda_stream`.
 * y = z + update when `residual` is non-zero (the reference module owns its residual,
 * src/miniworld/blocks/msa_module.py:116-117), else the update alone.
 * Mirrors `inference(leaves, flat_mask, flat_scale, direction)` of the reference engine
 * (benchmarks/engine_ops/trimul_batch.py:66).
 */
int b200_trimul_forward(const void* z, const void* w_left, const void* w_left_gate, const void* w_right,
                        const void* w_right_gate, const void* w_gate, const void* w_out, int weight_dtype,
                        const float* ln_in_w, const float* ln_in_b, const float* ln_out_w, const float* ln_out_b,
                        const void* const* bias_opt, const uint8_t* token_mask, const uint8_t* pair_mask, void* y,
                        void* workspace, size_t workspace_bytes, int B, int N, int d_pair, int d_hidden,
                        int direction, float eps_in, float eps_out, int residual, void* cuda_stream);

/*
 * General forward. Everything of b200_trimul_forward, plus:
 *  - direction B200_TRIMUL_BIDIRECTIONAL (0, the engine's numbering: benchmarks/engine_ops/trimul_batch.py:10,66):
 *    the BidirectionalTriangleMultiplication MiniWorld's trunk builds (src/miniworld/modules/mini_pairformer.py:76-80,
 *    algorithm docs/paper/supplement.tex:125-136). Same eleven leaves with wider shapes: w_left, w_left_gate, w_right,
 *    w_right_gate are [256, 128] (rows 0-127 -> outgoing contraction, rows 128-255 -> incoming), ln_out_w / ln_out_b
 *    have 256 entries, w_out is [128, 256], w_gate stays [128, 128]; the first four entries of bias_opt, if given,
 *    are fp32[256]. d_hidden is the width of one direction (128). Workspace: b200_trimul_workspace_bytes with
 *    direction 0.
 *  - drop_scale: null, or [B, N, 128] bf16 - the row-shared dropout scale [B, 1, N, C] of the training path
 *    (keep-mask / (1 - p), scripts/check_trimul_module_reference.py:43 in the reference project): y = z + scale * update.
 *    A zero scale returns z exactly. This is `flat_scale` of the engine's entry point. 128-wide pairs only.
 *  - d_pair = 64: z, y are [B, N, N, 64]; w_left, w_left_gate, w_right, w_right_gate are [128, 64], ln_in 64 entries,
 *    ln_out 128 entries, w_out [64, 128], w_gate [64, 64]; bias_opt entries 0-3 fp32[128], 4-5 fp32[64]. With one
 *    direction (d_hidden = 128) all 128 channels are contracted that way; with direction 0 (d_hidden = 64) channels
 *    0-63 are contracted outgoing and 64-127 incoming, as in the reference's 64-wide validation case
 *    (docs/archive/engine2-validation-20260923/validate_bidir_reference.py:11). drop_scale must be null.
 */
int b200_trimul_forward_ex(const void* z, const void* w_left, const void* w_left_gate, const void* w_right,
                           const void* w_right_gate, const void* w_gate, const void* w_out, int weight_dtype,
                           const float* ln_in_w, const float* ln_in_b, const float* ln_out_w, const float* ln_out_b,
                           const void* const* bias_opt, const uint8_t* token_mask, const uint8_t* pair_mask,
                           const void* drop_scale, void* y, void* workspace, size_t workspace_bytes, int B, int N,
                           int d_pair, int d_hidden, int direction, float eps_in, float eps_out, int residual,
                           void* cuda_stream);

/*
 * Weight packing of the bidirectional module (shapes as in b200_trimul_forward_ex): two blocks of
 * b200_trimul_packed_bytes() each. `packed_out` feeds stage 1 of the outgoing half and stage 3, `packed_in` stage 1
 * of the incoming half; stage 3 also reads the second half of w_out from `packed_in`.
 */
int b200_trimul_pack_weights_bidir(const void* w_left, const void* w_left_gate, const void* w_right,
                                   const void* w_right_gate, const void* w_gate, const void* w_out, int weight_dtype,
                                   const float* ln_in_w, const float* ln_in_b, const float* ln_out_w,
                                   const float* ln_out_b, const void* const* bias_opt, void* packed_out,
                                   void* packed_in, void* cuda_stream);

/*
 * Stage 3, general form: output LayerNorm over 128 (tri_in null) or 256 (tri_in given: [tri, tri_in]) contracted
 * channels, output projection, sigmoid gate, optional row-shared dropout scale, residual. tri / tri_in:
 * [B, rows, 128, N] fp16 as written by stage 2; packed / packed_in: the blocks of b200_trimul_pack_weights(_bidir);
 * drop_scale: null or [B, N, 128] bf16; z, y: [B, rows, N, 128] bf16.
 */
int b200_trimul_epilogue_wide(const void* tri, const void* tri_in, const void* z, const void* packed,
                              const void* packed_in, const void* drop_scale, void* y, int B, int N, int rows,
                              float eps_in, float eps_out, int residual, int* status, void* cuda_stream);

/*
 * The same forward for callers that cannot give the library a workspace because they cannot allocate device
 * memory at all: a server whose pool already owns the whole GPU (a late cudaMalloc fails, or stalls a
 * latency-critical loop by synchronising the device), or a plug-in whose host forbids allocation after start-up.
 * It has no counterpart in the reference, whose engine allocates its intermediates through PyTorch.
 *
 * The scratch is a fixed 12.2 MiB device array that belongs to the library's module: it takes no space in the
 * file, and every GPU on which the library's kernels are loaded reserves it until the process exits. Limit: B * N * N <= 16384 pair cells (one 128-token sample, four 64-token samples, ...);
 * anything larger returns B200_TRIMUL_E_TOO_LARGE before any device work is issued. The function itself calls
 * no allocator of any kind. Its first call on a device looks up the array's device address, so make that
 * call before starting a stream capture. Every call on a device uses the same array, which keeps the previous
 * call's contents: the status words are cleared on entry and all other regions are overwritten before they are
 * read, but two calls that overlap on the GPU race on it - issue them on one stream, or serialise them.
 * `device_status_out` (may be null) receives the device address of the status word for b200_trimul_read_status.
 * The looked-up address is cached per device for the life of the process: after cudaDeviceReset (or any other
 * teardown of the device's primary context) it is stale and this entry point must not be used again.
 */
int b200_trimul_forward_static(const void* z, const void* w_left, const void* w_left_gate, const void* w_right,
                               const void* w_right_gate, const void* w_gate, const void* w_out, int weight_dtype,
                               const float* ln_in_w, const float* ln_in_b, const float* ln_out_w,
                               const float* ln_out_b, const void* const* bias_opt, const uint8_t* token_mask,
                               const uint8_t* pair_mask, void* y, int B, int N, int d_pair, int d_hidden,
                               int direction, float eps_in, float eps_out, int residual, int** device_status_out,
                               void* cuda_stream);

/*
 * Backward, for every width the forward takes (d_pair = d_hidden = 128; d_pair = 64 with d_hidden = 128 for one direction
 * or 64 per direction for direction 0, where dz is [B, N, N, 64], the gradients have the parameters' shapes of the
 * forward's d_pair = 64 note, and drop_scale must be null): the reference's training path, stages B1-B12 of
 * docs/kernels/trimul/TRIMUL_STATUS.md:43-52 (its B5-B6, the contraction gradients, are cuBLAS calls there). Given
 * dy = d loss / d y ([B, N, N, 128] bf16), the inputs of the forward call and the workspace that
 * b200_trimul_forward / _forward_ex left behind for these inputs (it holds the stage tensors), it writes
 *   dz  [B, N, N, 128] bf16          d loss / d z, the residual path included when `residual` is non-zero
 *   dw[6] fp32, the parameters' shapes: gradients of w_left, w_left_gate, w_right, w_right_gate, w_gate, w_out (that
 *                                    order): [128, 128] each, or [256, 128] x 4, [128, 128], [128, 256] for direction 0
 *   d_ln_in_w / _b fp32 [128],  d_ln_out_w / _b fp32 [128] (direction 0: [256])
 * Every output is overwritten, not accumulated into. Biases are constants (no gradient). drop_scale as in the forward.
 * Launches, one direction: weight packing, max |dy| and the power-of-two scale the fp16 gradient tiles carry, the
 * epilogue's backward (one kernel: both LayerNorm-folded GEMMs recomputed, four gradient GEMMs on the tensor cores), the
 * two contraction gradient launches, the prologue's backward once per side, partial-sum reductions, the parameter
 * gradients. Direction 0 (the bidirectional module): the statistics of the 256-channel output LayerNorm, the epilogue's
 * backward once per 128-channel tensor plus a kernel that finishes the first tensor's LayerNorm backward, the forward's
 * prologue once more (left / right of the first half, which the forward overwrote), four contraction gradient launches,
 * the prologue's backward four times (side x half).
 * The result is deterministic (fixed summation order). Workspace: b200_trimul_backward_workspace_bytes, 1024-byte
 * aligned; _layout gives its 17 region offsets + the total (status, packed weights, scale, reduced sums M and S, per-CTA
 * partials of M and S, dtri, dleft, dright, d x_hat, then the bidirectional module's extra regions) for tests.
 */
int b200_trimul_backward_workspace_bytes(int B, int N, int direction, size_t* out_bytes);
int b200_trimul_backward_workspace_layout(int B, int N, int direction, size_t* offsets18);
int b200_trimul_backward(const void* dy, const void* z, const void* w_left, const void* w_left_gate, const void* w_right,
                         const void* w_right_gate, const void* w_gate, const void* w_out, int weight_dtype,
                         const float* ln_in_w, const float* ln_in_b, const float* ln_out_w, const float* ln_out_b,
                         const void* const* bias_opt, const uint8_t* token_mask, const uint8_t* pair_mask,
                         const void* drop_scale, const void* forward_workspace, void* dz, void* const* dw,
                         float* d_ln_in_w, float* d_ln_in_b, float* d_ln_out_w, float* d_ln_out_b, void* workspace,
                         size_t workspace_bytes, int B, int N, int d_pair, int d_hidden, int direction, float eps_in,
                         float eps_out, int residual, void* cuda_stream);

/*
 * Pair Transition, the operator on the other side of the triangle update in every block
 * (src/miniworld/modules/mini_pairformer.py:81-84,108 in the reference project; the engine's fused kernel is
 * `transition_fused_fwd_sm100a`, docs/phase2-b200-training-speed.md:165):
 *   y = x + squeeze( SiLU(expand_a(LN(x))) * expand_b(LN(x)) ),  expand_a / expand_b: [4 d, d], squeeze: [d, 4 d], no biases
 * (parameter names and the OpenFold mapping: benchmarks/protenix_finetune/patch_engine.py:35-37). d = 128, n = 4 only.
 * x, y: [positions, 128] bf16 (any leading shape flattened; y may alias x); `packed`: b200_transition_packed_bytes()
 * bytes, 1024-aligned, written by b200_transition_pack_weights (weights bf16 or fp32, LayerNorm affine fp32);
 * `status`: a device int, zero before the call, receives a positive device code if a bounded wait runs out.
 */
size_t b200_transition_packed_bytes(void);
int b200_transition_pack_weights(const void* w_expand_a, const void* w_expand_b, const void* w_squeeze, int weight_dtype,
                                 const float* ln_w, const float* ln_b, void* packed, void* cuda_stream);
int b200_transition_forward(const void* x, const void* packed, void* y, long long positions, int d, int n, float eps,
                            int residual, int* status, void* cuda_stream);

/* Zero the status words at the start of a workspace (asynchronous). */
int b200_trimul_clear_status(int* status, void* cuda_stream);

/* Synchronise `cuda_stream` and copy the device status word to *host_status. */
int b200_trimul_read_status(const int* status, void* cuda_stream, int* host_status);

/*
 * Backward of the pair Transition (the operator has no training kernel of its own in the reference tree; its forward is
 * `transition_fused_fwd_sm100a`, docs/phase2-b200-training-speed.md:165). Given dy = d loss / d y ([positions, 128]
 * bf16) and the forward's inputs, writes dx ([positions, 128] bf16, the residual path included when `residual` is
 * non-zero) and, in fp32 and the parameters' shapes, d_expand_a / d_expand_b [512, 128], d_squeeze [128, 512],
 * d_ln_w / d_ln_b [128]. Every output is overwritten. One launch per block of 128 hidden units (four), whose three
 * weight-gradient accumulators stay in tensor memory over all positions; the running d x_hat is carried between the
 * launches in the workspace. Deterministic. Workspace: b200_transition_backward_workspace_bytes, 1024-byte aligned.
 */
int b200_transition_backward_workspace_bytes(long long positions, size_t* out_bytes);
int b200_transition_backward(const void* dy, const void* x, const void* w_expand_a, const void* w_expand_b,
                             const void* w_squeeze, int weight_dtype, const float* ln_w, const float* ln_b, void* dx,
                             float* d_expand_a, float* d_expand_b, float* d_squeeze, float* d_ln_w, float* d_ln_b,
                             void* workspace, size_t workspace_bytes, long long positions, int d, int n, float eps,
                             int residual, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_TRIMUL_H_ */
