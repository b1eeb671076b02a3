/*
 * b200ta — C ABI of the sm_100a triangle-attention / pair-transition kernels.
 *
 * Every entry point takes plain device pointers, sizes, element strides and a
 * CUDA stream (passed as void*; NULL = the legacy default stream).  Calls only
 * enqueue work on that stream: they never synchronise, never allocate device
 * memory (the caller passes workspaces) and return 0 or a negative status code.
 * b200ta_last_error() gives the reason for the calling thread's last failure.
 *
 * Tensors are bf16 unless stated; "positions" are the B*R*S cells of a pair
 * tensor z[B, R, S, 128] addressed through element strides, so the ending node
 * (which works on the transposed pair tensor) passes the same buffers with the
 * R and S strides swapped instead of materialising a transpose.
 *
 * The first call on a device creates a small per-device state (the address of a status
 * word); make it outside any stream capture.
 *
 * Each declaration cites the interface of the reference runtime it replaces
 * (paths are relative to the reference project root).
 */
#ifndef B200TA_H_
#define B200TA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200TA_OK 0
#define B200TA_ERR_INVALID (-1)     /* bad argument: shape, alignment, stride, null pointer */
#define B200TA_ERR_CUDA (-2)        /* a CUDA runtime call failed */
#define B200TA_ERR_DRIVER (-3)      /* tensor-map encoding failed / driver entry point missing */
#define B200TA_ERR_DEVICE_WAIT (-4) /* a kernel gave up on a bounded wait (status word) */
#define B200TA_ERR_UNSUPPORTED (-5) /* valid request outside what the kernels cover */

/* Fixed model dimensions the kernels are specialised for (Boltz-2 / AF3 pair track). */
#define B200TA_C 128       /* pair channels c_z */
#define B200TA_HEADS 4     /* attention heads */
#define B200TA_HEAD_DIM 32 /* head width */
#define B200TA_HIDDEN 512  /* transition hidden width (4 x c_z) */

#define B200TA_DTYPE_BF16 0
#define B200TA_DTYPE_F32 1

#define B200TA_EMPTY_ROW_ZEROS 0   /* rows with no valid key produce 0 (fused reference kernels) */
#define B200TA_EMPTY_ROW_UNIFORM 1 /* rows with no valid key average V over all keys (eager reference) */

/* Library ABI version (major*100 + minor). */
int b200ta_version(void);

/* Message describing the calling thread's most recent non-zero return. */
const char* b200ta_last_error(void);

/*
 * Reads (*status) the current device's status word: 0, or B200TA_ERR_DEVICE_WAIT
 * if any kernel since the last reset abandoned a bounded wait.  Synchronise the
 * stream first if the answer must cover work still in flight.
 * Replaces: error propagation of cubin launches, cpp/kernels/cubin_runtime.h
 * (the reference has no device-side status; its kernels have unbounded waits).
 */
int b200ta_device_status(int* status);
int b200ta_reset_device_status(void);

/* ---- weight packing --------------------------------------------------------
 *
 * Folds LayerNorm(gamma, beta) into the projection that follows it, so the
 * kernels can feed raw bf16 rows of z to the tensor cores and apply mean / rstd
 * in the GEMM epilogue.  Packed buffers are opaque, device-resident and must be
 * rebuilt when any source weight changes.
 * Replaces: pack_weights, bionemo_ir/_torch/custom_ops/transition_mlp_w_norm/ops.py:198-302
 * (same idea, applied here to the attention in-projection as well).
 */

/* Bytes of a packed node / transition weight buffer (256-byte aligned pointer required). */
size_t b200ta_node_pack_bytes(void);
size_t b200ta_transition_pack_bytes(void);

/*
 * ln_w, ln_b: [128].  w_in: [512,128], rows ordered q,k,v,g (head-major inside
 * each, as Linear.load_weights builds it, bionemo_ir/_torch/layers/linear.py:184-198).
 * b_in: [512] or NULL.  w_bias: [4,128] (pair_bias_proj).  w_out: [128,128]
 * (o_proj), b_out: [128] or NULL.  weight_dtype: B200TA_DTYPE_* of all six.
 */
int b200ta_pack_node_weights(const void* ln_w, const void* ln_b, const void* w_in,
                             const void* b_in, const void* w_bias, const void* w_out,
                             const void* b_out, int weight_dtype, void* packed, void* stream);

/*
 * ln_w, ln_b: [128].  w1: [1024,128] (fused_fc2_fc1: value rows first, gate rows
 * second).  w2: [128,512] (fc3).  The LayerNorm vectors are kept beside the bf16 weights (the kernel normalises
 * the rows of x and rounds them to bf16 before the first GEMM, as the eager module does).
 */
int b200ta_pack_transition_weights(const void* ln_w, const void* ln_b, const void* w1,
                                   const void* w2, int weight_dtype, void* packed, void* stream);

/*
 * The ReLU pair transition's weights into a buffer of b200ta_transition_pack_bytes() bytes (for
 * b200ta_transition_relu).  ln_w, ln_b: [128] or both NULL.  w1: [512,128], b1: [512] or NULL (linear_1).
 * w2: [128,512], b2: [128] or NULL (linear_2).
 * Replaces: pack_weights(..., activation="relu"), bionemo_ir/_torch/custom_ops/transition_mlp_w_norm/ops.py:198-302.
 */
int b200ta_pack_relu_transition_weights(const void* ln_w, const void* ln_b, const void* w1, const void* b1,
                                        const void* w2, const void* b2, int weight_dtype, void* packed,
                                        void* stream);

/* ---- triangle-attention node ------------------------------------------------- */

/*
 * Prologue: LayerNorm over channels, the q/k/v/gate projection and the 4-head
 * triangle-bias projection of every position, one tcgen05 GEMM per 128-position tile.
 *
 *   z          [B,R,S,128] via element strides (zs_b, zs_r, zs_s); channel stride 1.
 *   qkvg       output, four planes (q,k,v,g) of [B*R, 4 heads, S, 32]:
 *              element (which, br, h, s, d) at which*qs_which + br*qs_br + h*qs_h + s*qs_s + d.
 *              The g plane holds sigmoid(gate logit), rounded to bf16 from the bf16-rounded logit as
 *              the eager module's gate.sigmoid_() does (bionemo_ir/_torch/layers/attention.py:288);
 *              it is the `gate` operand of b200ta_attention.
 *   bias       output, bias[b,h,q=r,k=s] * sqrt(32) (i.e. divided by the softmax scale, the form
 *              b200ta_attention consumes) at b*bs_b + h*bs_h + r*bs_q + s*bs_k;
 *              entries S <= s < S_pad are written as zero.  May be NULL (no bias written).
 *   want_qkvg  0 = bias only (used to finish the bias of all rows before a
 *              row-chunked pass), 1 = both.
 *
 * Replaces: LNPairBias (bionemo_ir/dsl_kernels/triton/ln_pair_bias.py:261-322) plus the
 * in_proj GEMM (bionemo_ir/_torch/layers/attention.py:257-258).
 */
int b200ta_prologue(const void* z, int64_t zs_b, int64_t zs_r, int64_t zs_s, const void* packed,
                    float eps, void* qkvg, int64_t qs_which, int64_t qs_br, int64_t qs_h,
                    int64_t qs_s, int want_qkvg, void* bias, int64_t bs_b, int64_t bs_h,
                    int64_t bs_q, int64_t bs_k, int B, int R, int S, int S_pad, void* stream);

/*
 * Pair bias of the single-track attention: bias[b,h,q,k] = bias_scale * ( LayerNorm(z[b,q,k,:]) · W_z[h,:] ) for up
 * to 16 heads, written head-major with the key axis padded: the projection, the moveaxis and the padding in one pass
 * over z (a streaming kernel of its own: six-stage TMA ring, one N=16 tcgen05 GEMM per 128-position tile).
 *
 *   b200ta_pack_pair_bias_weights: ln_w, ln_b [128] (both NULL: z is used as it is), w_z [num_heads,128] in
 *       weight_dtype; bias_scale multiplies the result (pass 1/softmax_scale for b200ta_attention);
 *       packed: b200ta_node_pack_bytes() bytes, 256-byte aligned.
 *   b200ta_pair_bias: z [B,Q,K,128] bf16 via element strides; bias at b*bs_b + h*bs_h + q*bs_q + k*bs_k;
 *       entries K <= k < K_pad are written as zero; num_heads even, at most 16.
 *
 * Replaces: LNProjMoveaxisPad.forward (bionemo_ir/_torch/custom_ops/fused_ln_proj_moveaxis_pad.py:90-154), as
 * AttentionPairBias.project_pair_bias calls it (bionemo_ir/_torch/layers/attention.py:835-852).
 */
int b200ta_pack_pair_bias_weights(const void* ln_w, const void* ln_b, const void* w_z, int num_heads,
                                  float bias_scale, int weight_dtype, void* packed, void* stream);
int b200ta_pair_bias(const void* z, int64_t zs_b, int64_t zs_q, int64_t zs_k, const void* packed, float eps,
                     void* bias, int64_t bs_b, int64_t bs_h, int64_t bs_q, int64_t bs_k, int num_heads,
                     int B, int Q, int K, int K_pad, void* stream);

/*
 * Attention core.  For every (b, r, h) and query s:
 *   o[s,:] = softmax_t( scale * (q[s]·k[t] + bias[b,h,s,t]) ; t < len[b,r] ) · v[t,:]
 * optionally multiplied by gate[s,:], the gate factors in [0,1] (sigmoid already applied, as
 * b200ta_prologue writes them).
 *
 *   q,k,v,gate [B*R, 4, S, 32] via element strides (br, h, s); d stride 1; gate may be NULL.
 *   bias       [B, 4, S, S_pad]: the additive triangle bias DIVIDED by softmax_scale (the tensor core adds
 *              it to q·k before the scale is applied; b200ta_prologue writes it in this form);
 *              element strides (b, h, q); key stride 1; S_pad % 8 == 0.
 *   lengths    int32, len[b,r] at b*ls_b + r*ls_r (ls_r = 0 broadcasts one length per item).
 *              NULL = every key valid.
 *   out        [B*R, S, 4, 32] via element strides (br, s, h); d stride 1.
 *   lse        optional fp32 natural-log-sum-exp, [B*R, S, 4] contiguous, or NULL.
 *   empty_row_mode  B200TA_EMPTY_ROW_*.
 *
 * Replaces: triangle_attention.launch(config, LaunchParams)
 * (cpp/kernels/cutedsl_triangle_attention/launcher.h:515-532, launcher.cpp:548-627) and the
 * gate multiply of bionemo_ir/_torch/layers/attention.py:285-288.
 */
int b200ta_attention(const void* q, const void* k, const void* v, const void* gate, int64_t s_br,
                     int64_t s_h, int64_t s_s, const void* bias, int64_t bs_b, int64_t bs_h,
                     int64_t bs_q, const int32_t* lengths, int64_t ls_b, int64_t ls_r, void* out,
                     int64_t os_br, int64_t os_s, int64_t os_h, float* lse, float softmax_scale,
                     int empty_row_mode, int B, int R, int S, int S_pad, void* stream);

/*
 * The same attention core with keys that may be switched off anywhere in a row (pair masks that are not
 * 1…1 0…0).  key_mask holds one bit per key: bit (t % 32) of the 32-bit word at b*km_b + r*km_r + t/32 is 1 when
 * key t of pair row (b, r) takes part; ceil(S / 32) words per row, bits at and past the row's length 0.
 * lengths (required here) is the position of the row's last valid key + 1 (0 = no valid key: empty_row_mode
 * applies).  All queries of a pair row share its bits.  Otherwise as b200ta_attention.
 * Replaces: the additive-mask backends the reference uses when a node is built with
 * pair_mask_left_aligned=False (bionemo_ir/_torch/layers/triangle_nodes.py:230-246,
 * bionemo_ir/_torch/attention_backend/utils.py:305-317).
 */
int b200ta_attention_masked(const void* q, const void* k, const void* v, const void* gate, int64_t s_br,
                            int64_t s_h, int64_t s_s, const void* bias, int64_t bs_b, int64_t bs_h,
                            int64_t bs_q, const int32_t* lengths, int64_t ls_b, int64_t ls_r,
                            const uint32_t* key_mask, int64_t km_b, int64_t km_r, void* out, int64_t os_br,
                            int64_t os_s, int64_t os_h, float* lse, float softmax_scale, int empty_row_mode,
                            int B, int R, int S, int S_pad, void* stream);

/*
 * Epilogue: out = residual + og · W_oᵀ + b_o, with og = o ⊙ sigmoid(g) as written by
 * b200ta_attention.
 *
 *   og        [B,R,S,128] via element strides (b, r, s).
 *   residual  [B,R,S,128] via element strides, or NULL (out = update only).
 *   out       [B,R,S,128] via element strides; may alias residual.
 *
 * Replaces: AttnEpilogue.__call__ (bionemo_ir/_torch/custom_ops/attn_epilogue/ops.py:195-254).
 */
int b200ta_epilogue(const void* og, int64_t gs_b, int64_t gs_r, int64_t gs_s, const void* packed,
                    const void* residual, int64_t rs_b, int64_t rs_r, int64_t rs_s, void* out,
                    int64_t os_b, int64_t os_r, int64_t os_s, int B, int R, int S, void* stream);

/*
 * The same epilogue with its result written transposed into the column shards of the GPUs of one box: the
 * calling GPU holds the pair rows [rank*R, rank*R + R) of a [B, S, S, 128] pair tensor (R = S / num_peers); the
 * row (b, rank*R + r) position s goes to GPU s / R, whose column shard is a contiguous [B][S][R][128] bf16
 * tensor, at (b, rank*R + r, s % R).  peer_out[g] is that shard's address on GPU g as mapped into this process
 * (peer access over NVLink, e.g. a symmetric-memory allocation); the kernel stores straight into it, so the
 * all-to-all between the starting and the ending node needs no separate pass.  The caller orders this call
 * after every GPU has finished reading its shard and orders the readers after it (one barrier on each side).
 * The reference has no counterpart (its multi-GPU mode is whole-model replicas).
 */
int b200ta_epilogue_scatter(const void* og, int64_t gs_b, int64_t gs_r, int64_t gs_s, const void* packed,
                            const void* residual, int64_t rs_b, int64_t rs_r, int64_t rs_s,
                            void* const* peer_out, int num_peers, int rank, int B, int R, int S, void* stream);

/*
 * Whole node in one call: prologue -> attention -> epilogue on `stream`, intermediates in `workspace`
 * (b200ta_node_workspace_bytes(B, N) bytes, 256-byte aligned, caller-owned; contents are scratch).
 *
 *   z, out     square pair tensors [B,N,N,128] via element strides in kernel order (b, row, sequence): the
 *              starting node passes (stride_b, stride_i, stride_j), the ending node (stride_b, stride_j, stride_i).
 *   lengths    int32 valid-key count per (b, row) at b*ls_b + row*ls_r, or NULL (all keys valid).
 *   add_residual  1: out = z + update (out may alias z), 0: out = update.
 *
 * Replaces: TriangleAttentionNode.forward (bionemo_ir/_torch/layers/triangle_nodes.py:195-250) below the
 * Python layer, i.e. what a single native call per node would bind.
 */
size_t b200ta_node_workspace_bytes(int B, int N);
int b200ta_node_forward(const void* z, int64_t zs_b, int64_t zs_r, int64_t zs_s, const void* packed, float eps,
                        const int32_t* lengths, int64_t ls_b, int64_t ls_r, int empty_row_mode,
                        int add_residual, void* out, int64_t os_b, int64_t os_r, int64_t os_s,
                        void* workspace, size_t workspace_bytes, int B, int N, void* stream);

/*
 * The same node without any workspace argument, for callers that are not allowed to allocate device memory:
 * code running while a stream is being captured into a CUDA graph (a capture forbids cudaMalloc), request
 * handlers of a serving process whose own pool already owns all device memory, or a host that pre-sizes
 * everything at start-up and treats a later allocation as a bug.  The intermediates live in a fixed array that
 * is part of the library image: about 5.25 MiB of device memory on every GPU that loads the library, held
 * until the process exits.  This entry point has no counterpart in the reference runtime.
 *
 * Limit: B*N*N <= b200ta_node_static_max_positions() (4096 pair positions, e.g. one 64 x 64 pair tensor);
 * larger problems are refused with B200TA_ERR_UNSUPPORTED and a message, and belong to b200ta_node_forward.
 * The call makes no cudaMalloc/cudaFree and calls no allocating routine.  Its first call on a device looks up
 * the array's device address (with that device current); make that first call before starting a stream capture.
 * The looked-up address is kept per device for the life of the process: it does not survive a cudaDeviceReset
 * or any other teardown of the device's context, after which this entry point must not be called again.
 * Every call uses the one array and leaves its last intermediates there, so two calls that can overlap on the
 * GPU (different streams, or different host threads without ordering) race on it: order them on one stream
 * or with events.  Nothing in the array needs clearing between calls: each call writes all it later reads.
 * Arguments are those of b200ta_node_forward minus the workspace.
 */
int b200ta_node_static_max_positions(void);
int b200ta_node_forward_static(const void* z, int64_t zs_b, int64_t zs_r, int64_t zs_s, const void* packed,
                               float eps, const int32_t* lengths, int64_t ls_b, int64_t ls_r,
                               int empty_row_mode, int add_residual, void* out, int64_t os_b, int64_t os_r,
                               int64_t os_s, int B, int N, void* stream);

/* ---- pair transition ---------------------------------------------------------------
 *
 * out = [x +] mask * ( (silu(gate) * value) · W2ᵀ ),  [value|gate] = LayerNorm(x) · W1ᵀ,
 * one kernel, hidden activation kept on chip.
 *
 *   x     [rows,128] bf16, row stride xs (elements).   out likewise (may alias x).
 *   mask  one bf16 value per row (contiguous) or NULL.
 *   add_residual  1: out = x + ..., 0: out = update.
 *
 * Replaces: transition_mlp_w_norm launch
 * (bionemo_ir/_torch/custom_ops/transition_mlp_w_norm/ops.py:349-518).
 */
int b200ta_transition(const void* x, int64_t xs, const void* mask, const void* packed, float eps,
                      void* out, int64_t os, int64_t rows, int add_residual, void* stream);

/*
 * The ReLU pair transition  out = [x +] mask * ( relu(LayerNorm(x) · W1ᵀ + b1) · W2ᵀ + b2 )  (hidden 512, both
 * linears with biases), on the same kernel pipeline; arguments as for b200ta_transition, `packed` from
 * b200ta_pack_relu_transition_weights.
 * Replaces: PairTransition / _ReluTransition (bionemo_ir/_torch/layers/transition.py:540-656) and its fused form
 * transition_mlp_w_norm(..., activation="relu") (bionemo_ir/_torch/custom_ops/transition_mlp_w_norm/ops.py:198-338).
 */
int b200ta_transition_relu(const void* x, int64_t xs, const void* mask, const void* packed, float eps, void* out,
                           int64_t os, int64_t rows, int add_residual, void* stream);

/*
 * The transition of a column shard x = [B][tokens][cols][128] (contiguous bf16, cols = tokens / num_peers, a
 * multiple of 32; this GPU holds the pair columns [rank*cols, rank*cols + cols)) with its result written into the
 * row shards of the GPUs of one box: position (b, i, j) goes to GPU i / cols, whose row shard is a contiguous
 * [B][cols][tokens][128] bf16 tensor, at (b, i % cols, rank*cols + j).  peer_out[g] is that shard's address on
 * GPU g as mapped into this process; the kernel's TMA stores go straight to it, so the all-to-all that returns a
 * row-sharded pair tensor to row order needs no separate pass.  mask: one bf16 value per position of x, or NULL.
 * The caller orders this call after every GPU has finished reading its row shard and orders the readers after it.
 * The reference has no counterpart (its multi-GPU mode is whole-model replicas).
 */
int b200ta_transition_scatter(const void* x, const void* mask, const void* packed, float eps,
                              void* const* peer_out, int num_peers, int rank, int B, int tokens, int cols,
                              int add_residual, void* stream);

/* ---- dense layers of the single track ---------------------------------------------------
 *
 * The single representation s[B, tokens, 384] has one row per token; its layers are small GEMMs.
 *
 * b200ta_row_stats: {rstd, -mean*rstd} (two floats) of every row of x[rows, K] (bf16, row stride in elements):
 *     the LayerNorm statistics b200ta_linear applies to a GEMM whose weights have the LayerNorm folded in.
 *
 * b200ta_linear: out = finish(A · Wᵀ) on the tensor cores, one 128x128 tile per CTA.
 *     A      bf16, element (b, row, k) at b*as_b + row*as_row + (k / 128)*as_chunk + k % 128 (a row-major matrix
 *            has as_chunk = 128; the attention output [B, 4, rows, 128] is read in place with as_chunk = rows*128).
 *     w      bf16 [N, K] row-major; K, N multiples of 128.
 *     sc     float [N][2] {rowsum, const}: value[n] = rstd*acc[n] + nmr*rowsum[n] + const[n] with {rstd, nmr} the
 *            row's entry of `stats` ([B*rows][2]) or {1, 0} when stats is NULL.
 *     mode   B200TA_LINEAR_PLANES: N = 2048 columns ordered (which, head, 32) are written head-major as
 *                [which][B][16][rows][32] (plane_stride elements between planes), plane 3 as sigmoid(value): the
 *                q, k, v and gate operands of b200ta_attention;
 *            B200TA_LINEAR_ROWS: out[(b*rows + row)*os_row + n] = value[n] (+ residual, same indexing with rs_row);
 *            B200TA_LINEAR_SWIGLU: every 32 columns are 16 values followed by their 16 gates;
 *                out[(b*rows + row)*os_row + n/2 + j] = silu(gate_j) * value_j.
 *
 * Replaces: the eager projections of AttentionPairBias (in_proj, proj_o; bionemo_ir/_torch/layers/attention.py:
 * 764-805 and 1099-1132) and of the single-track Transition (bionemo_ir/_torch/layers/transformers/
 * pairformer.py:153-160), which the reference runs through cuBLAS and Triton element-wise kernels.
 */
#define B200TA_LINEAR_PLANES 0
#define B200TA_LINEAR_ROWS 1
#define B200TA_LINEAR_SWIGLU 2
int b200ta_row_stats(const void* x, int64_t row_stride, int64_t rows, int K, float eps, void* stats, void* stream);
int b200ta_linear(const void* a, int64_t as_b, int64_t as_row, int64_t as_chunk, const void* w, const void* sc,
                  const void* stats, const void* residual, int64_t rs_row, void* out, int64_t os_row,
                  int64_t plane_stride, int mode, int B, int rows, int K, int N, void* stream);

/* ---- triangle multiplication ---------------------------------------------------------
 *
 * update = sigmoid(LN_in(z)·W_goᵀ) ⊙ ( LN_out(t)·W_poᵀ ),   t[b,i,j,d] = Σ_k a[b,i,k,d]·b[b,j,k,d]  (outgoing)
 *                                                                       Σ_k a[b,k,i,d]·b[b,k,j,d]  (incoming)
 * [a|b] = sigmoid(LN_in(z)·W_giᵀ) ⊙ (LN_in(z)·W_piᵀ) ⊙ mask;  dim 128, hidden 128, bf16.
 * Three kernels with two channel-major intermediates the caller provides:
 *   ab [B][256][N][pitch]  bf16   a planes (0..127) then b planes; contraction index contiguous
 *   x  [B][128][N][pitch]  bf16   x[b][d][i][j]
 * pitch % 16 == 0, pitch >= N; both 32-byte aligned.
 *
 * Replaces: TriangleMultiplicationNode._forward_impl (bionemo_ir/_torch/layers/triangle_nodes.py:646-727), i.e.
 * layer_norm_transpose + dual_gemm_x_x (custom_ops/dual_gemm_x_x/ops.py:34-58) -> project,
 * _contract_projection (triangle_nodes.py:596-612) -> contract,
 * layer_norm_transpose + dual_gemm_x0_x1 (custom_ops/dual_gemm_x0_x1/ops.py:29-52) -> output;
 * the same split as the reference's own fused chain trimul_kf_k1/k2/k3 (triangle_nodes.py:551-594).
 */
size_t b200ta_trimul_pack_bytes(void);

/*
 * Folds norm_in into p_in/g_in (rows a then b, as torch.chunk splits them) and into g_out, norm_out into p_out.
 * All tensors share weight_dtype; biases may be NULL.  p_in/g_in: [256,128]; p_out, g_out: [128,128].
 * Source of the parameters: triangle_nodes.py:378-417.
 */
int b200ta_pack_trimul_weights(const void* ln_in_w, const void* ln_in_b, const void* w_p_in, const void* b_p_in,
                               const void* w_g_in, const void* b_g_in, const void* ln_out_w, const void* ln_out_b,
                               const void* w_p_out, const void* b_p_out, const void* w_g_out, const void* b_g_out,
                               int weight_dtype, void* packed, void* stream);

/*
 * ab = gated, masked input projection of z[B,R,S,128] (element strides zs_*), written channel-major with S
 * contiguous.  The outgoing node passes z as it is (R = i, S = k); the incoming node passes the two pair strides
 * swapped (R = i read along the second pair axis, S = k along the first), and the mask likewise.
 *   mask     fp32, element (b,r,s) at b*ms_b + r*ms_r + s*ms_s, or NULL (all ones).
 *   b_scale  fp32 [B] multiplying the b channels (mean normalisation: 1 / (n_valid + 1e-3)), or NULL.
 */
int b200ta_trimul_project(const void* z, int64_t zs_b, int64_t zs_r, int64_t zs_s, const float* mask, int64_t ms_b,
                          int64_t ms_r, int64_t ms_s, const float* b_scale, const void* packed, float eps, void* ab,
                          int64_t pitch, int B, int R, int S, void* stream);

/* x[b][d][i][j] = Σ_k ab[b][d][i][k] * ab[b][128+d][j][k]  (fp32 accumulation, bf16 result). */
int b200ta_trimul_contract(const void* ab, void* x, int B, int N, int64_t pitch, void* stream);

/*
 * out[b,i,j,:] = sigmoid(LN_in(z)·W_goᵀ + b_go) ⊙ (LN_out(x[b,:,i,j])·W_poᵀ + b_po)  [+ z]  [then * mask]
 * z and out in the caller's orientation [B,N,N,128] via element strides (multiples of 16, 32-byte aligned bases);
 * out may alias z.  mask (fp32, strides ms_*) multiplies the result as the reference's fused residual kernel does
 * (tests/_torch/test_triangle_nodes.py:272-311); NULL leaves it unmasked like the unfused path.
 */
int b200ta_trimul_output(const void* z, int64_t zs_b, int64_t zs_i, int64_t zs_j, const void* x, int64_t pitch,
                         const float* mask, int64_t ms_b, int64_t ms_i, int64_t ms_j, const void* packed, float eps,
                         int add_residual, void* out, int64_t os_b, int64_t os_i, int64_t os_j, int B, int N,
                         void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200TA_H_ */
