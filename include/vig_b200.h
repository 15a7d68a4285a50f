/*
 * vig_b200 -- C ABI of the B200 (sm_100a) bi-directional gated-linear-attention operator and the
 * bandwidth-bound kernels of the ViG block around it.
 *
 * Conventions (all entry points):
 *   - plain C: pointers are DEVICE pointers unless stated otherwise, sizes are ints, no C++ types;
 *   - nothing is allocated and nothing synchronises: the caller owns every buffer (workspace
 *     included) and every launch goes to the `stream` argument (a cudaStream_t passed as void*);
 *   - return value: 0 = ok, < 0 = rejected argument (VIG_ERR_*), > 0 = a cudaError_t value;
 *   - dtype codes: 0 = fp32, 1 = bf16, 2 = fp16.  Accumulation, cumulative gates and scan states
 *     are always fp32;
 *   - one thread per device at a time per entry point (the reference has the same rule: one Python
 *     thread per process, one process per GPU).
 *
 * Paths cited below are those of the reference repository (hustvl/ViG).
 */
#ifndef VIG_B200_H
#define VIG_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define VIG_API __attribute__((visibility("default")))
#else
#define VIG_API
#endif

#define VIG_DTYPE_F32 0
#define VIG_DTYPE_BF16 1
#define VIG_DTYPE_F16 2

#define VIG_OK 0
#define VIG_ERR_NULL (-1)       /* a required pointer is NULL */
#define VIG_ERR_SHAPE (-2)      /* unsupported size (dk, dv, C, N, ...) */
#define VIG_ERR_DTYPE (-3)      /* unknown dtype code */
#define VIG_ERR_ALIGN (-4)      /* pointer or stride not aligned as the kernel needs */
#define VIG_ERR_WORKSPACE (-5)  /* workspace missing or too small */
#define VIG_ERR_ARG (-6)        /* any other rejected argument */
#define VIG_ERR_DEVICE (-7)     /* not an sm_100 device / driver entry point missing */
#define VIG_ERR_SCRATCH_LIMIT (-8) /* the call needs more scratch than vig_bigla_fwd_noalloc's fixed array holds */

/* Which implementation of the scan runs.  AUTO picks the tcgen05 kernel for bf16/fp16 inputs whose
 * layout it supports and the SIMT kernel otherwise (fp32 inputs always take the SIMT kernel: the
 * 5th-generation tensor cores have no fp32 MMA and tf32 would miss the 1e-4 bar). */
#define VIG_IMPL_AUTO 0
#define VIG_IMPL_SIMT 1
#define VIG_IMPL_TC 2
#define VIG_IMPL_TC_SINGLE 3 /* tensor-core path as ONE persistent launch for multi-segment sequences: half the DRAM
                               traffic, ~20 MB more workspace, needs as many co-resident CTAs as a sequence has
                               256-token segments (falls back to three launches when either is missing).  AUTO and TC
                               pick it for sequences of 2048..8192 tokens, where it is the faster form. */
#define VIG_IMPL_TC_SPLIT 4  /* tensor-core path as three launches (segment states, scan, outputs) at every length */
#define VIG_IMPL_TC_WAVE 5   /* warp-specialised wavefront form (dk = 64 or 32, dv = 64, 16-bit types; with or without an output): one persistent
                              CTA per SM, states handed from segment to segment; built for batches with at least as
                              many (sequence, direction) chains as the GPU has SMs */

VIG_API int vig_version(void);
VIG_API const char* vig_strerror(int status);

/*
 * Bi-directional gated linear attention, forward.
 *
 *   S^f_t = diag(exp(gf_t)) S^f_{t-1} + k_t^T v_t      (t = 0 .. L-1,  S^f_{-1} = init_state_fwd or 0)
 *   S^b_t = diag(exp(gb_t)) S^b_{t+1} + k_t^T v_t      (t = L-1 .. 0,  S^b_{L}  = init_state_bwd or 0)
 *   o_t   = out_scale * scale * q_t (S^f_t + S^b_t)
 *
 * Replaces, in one call and one pass over q/k/v/g:
 *   - `bid_fused_recurrent_gla` (flash-linear-attention/fla/ops/gla/recurrent_fuse.py:659-685, kernel
 *     :18-148) -- the eval path of classification/models/vig.py:442 (gk[:B] forward gates, gk[B:]
 *     backward gates, both indexed by original token position; that wrapper returns (o_f+o_b)/2, i.e.
 *     out_scale = 0.5);
 *   - `fused_chunk_gla` on batch-doubled, sequence-flipped inputs followed by (o_f + flip(o_b))/2
 *     (fla/ops/gla/chunk_fuse.py:554-572 and vig.py:407-426), with the flips done by indexing;
 *   - with dir_mask = 1 or 2, the one-direction `fused_chunk_gla` / `fused_recurrent_gla`
 *     (chunk_fuse.py:554-572, recurrent_fuse.py:631-657) including initial_state / final_state.
 *
 * q, k, g_fwd, g_bwd: [B,H,L,dk]; v, o: [B,H,L,dv]; the last dimension is contiguous and the element
 * strides of (b, h, l) are given per tensor in strides_*[3] (NULL = contiguous [B,H,L,d]), so views of
 * a packed [B,L,(h d)] projection need no copy.  scale < 0 means dk^-0.5 (the reference's scale=-1).
 * gate_logit_normalizer > 0: g_* hold RAW gate logits and the kernel applies
 * logsigmoid(x) / gate_logit_normalizer (vig.py:439); = 0: g_* are log-space gates (<= 0).
 * clamp_min: lower clamp of the log-gates (vig.py:440-441); pass a NaN to disable.
 * init_state_*: fp32 [B,H,dk,dv] or NULL.  final_state_*: fp32 [B,H,dk,dv] out or NULL (state after the
 * last token in scan order).  total_logdecay_*: fp32 [B,H,dk] out or NULL (sum of the log-gates over L;
 * with the final state of a zero-initialised scan it is what a sequence split across GPUs exchanges).
 * o may be NULL when only states are wanted.  dir_mask: 1 forward, 2 backward, 3 both.
 * status_dev: optional device int32; kernels OR error bits into it (bit 0: a bounded wait ran out,
 * bit 1: a chunk's cumulative log-gate left the range the tensor-core factorisation covers) -- never a trap.
 * Supported: dk in {16,32,64,128}, dv in {32,64,128} (SIMT); dk in {32,64}, dv = 64, bf16/fp16 (tensor core).
 */
VIG_API size_t vig_bigla_workspace_bytes(int B, int H, int L, int dk, int dv, int dtype, int impl);

VIG_API int vig_bigla_fwd(const void* q, const void* k, const void* v, const void* g_fwd, const void* g_bwd, void* o,
                  int B, int H, int L, int dk, int dv, int dtype,
                  const int64_t* strides_q, const int64_t* strides_k, const int64_t* strides_v,
                  const int64_t* strides_gf, const int64_t* strides_gb, const int64_t* strides_o,
                  float scale, float out_scale, float gate_logit_normalizer, float clamp_min,
                  const float* init_state_fwd, const float* init_state_bwd,
                  float* final_state_fwd, float* final_state_bwd,
                  float* total_logdecay_fwd, float* total_logdecay_bwd,
                  int dir_mask, int impl,
                  void* workspace, size_t workspace_bytes, int32_t* status_dev, void* stream);

/*
 * Backward of vig_bigla_fwd with log-space gates, no initial states: gradients of q, k, v and, per direction,
 * e = dq*q - dk*k, from which the gate gradients follow by a cumulative sum over the tokens
 * (dg_fwd[t] = sum_{s >= t} e_fwd[s], dg_bwd[t] = sum_{s <= t} e_bwd[s]; the reference takes the same sum in
 * PyTorch, flash-linear-attention/fla/ops/gla/chunk_fuse.py:506-516).  Replaces FusedChunkGLAFunction.backward
 * (chunk_fuse.py:413-518) for the merged bidirectional operator, i.e. the training path of
 * classification/models/vig.py:407-426 without the flipped copies.  fp32 arithmetic for every dtype.
 * q, k, g_*: [B,H,L,dk], v, d_out: [B,H,L,dv] with (b,h,l) element strides (NULL = contiguous); dq, dk, dv
 * (input dtype) and e_fwd, e_bwd (fp32) are contiguous [B,H,L,d].  dk in {16,32,64}, dv in {32,64,128}
 * (dk = 64 with dv = 128 included, dk = 16 only with dv = 32).
 */
VIG_API size_t vig_bigla_bwd_workspace_bytes(int B, int H, int L, int dk, int dv);
VIG_API int vig_bigla_bwd(const void* q, const void* k, const void* v, const void* g_fwd, const void* g_bwd, const void* d_out,
                  void* dq, void* dk_out, void* dv_out, float* e_fwd, float* e_bwd,
                  int B, int H, int L, int dk, int dv, int dtype,
                  const int64_t* strides_q, const int64_t* strides_k, const int64_t* strides_v,
                  const int64_t* strides_gf, const int64_t* strides_gb, const int64_t* strides_do,
                  float scale, float out_scale, int dir_mask,
                  void* workspace, size_t workspace_bytes, void* stream);

/*
 * Bi-GLA forward for callers that cannot allocate device memory (no counterpart in the reference: its
 * operators allocate their temporaries through PyTorch on every call).
 *
 * Who needs it: a host that is given only input and output buffers and may not call cudaMalloc when it
 * runs the operator -- an inference plugin inside someone else's runtime, a server whose memory pool is
 * fixed after start-up, any caller without a workspace to lend.  Same arithmetic and same kernels as
 * vig_bigla_fwd with both directions, no initial / final states; the scratch that call takes as
 * `workspace` lives here in a fixed device array of VIG_NOALLOC_SCRATCH_BYTES inside the library, which
 * every GPU that loads the library holds until the process exits.
 *
 * Limit: what the call really uses must fit VIG_NOALLOC_SCRATCH_BYTES, else VIG_ERR_SCRATCH_LIMIT is returned
 * and nothing is launched.  Used: B*H*ceil(L/256)*2*(dk*dv+dk)*4 bytes on the tensor-core path (16-bit types,
 * dk in {32,64}, dv = 64) when L > 256 and nothing for a single segment; B*H*ceil(L/64)*2*(dk*dv+dk)*4 bytes
 * on the SIMT path (fp32, other head sizes, impl = VIG_IMPL_SIMT) when L > 64 and nothing up to 64 tokens.
 * At dk = dv = 64 that is B*H*ceil(L/256) <= 504 (tensor core) or B*H*ceil(L/64) <= 504 (SIMT).
 * The call allocates nothing: no cudaMalloc / cudaFree, no allocating library routine.
 * The first call on each device looks up the array's device address (with that device current); with CUDA's
 * lazy module loading that is also the moment the runtime places this library's device image -- the array
 * included -- in device memory, so cudaMemGetInfo drops by the array's size across that one call.  Make that
 * first call at start-up (any tiny problem will do), outside any stream capture; later calls change nothing.  All calls on a device share the one array: calls that may overlap
 * on the GPU (different streams without ordering between them) race on it -- keep them on one stream or
 * order them with events.  Nothing in the array has to start at zero; each call overwrites what it uses.
 */
#define VIG_NOALLOC_SCRATCH_BYTES (16u << 20)
VIG_API size_t vig_bigla_noalloc_scratch_bytes(void);
VIG_API int vig_bigla_fwd_noalloc(const void* q, const void* k, const void* v, const void* g_fwd, const void* g_bwd, void* o,
                          int B, int H, int L, int dk, int dv, int dtype,
                          const int64_t* strides_q, const int64_t* strides_k, const int64_t* strides_v,
                          const int64_t* strides_gf, const int64_t* strides_gb, const int64_t* strides_o,
                          float scale, float out_scale, float gate_logit_normalizer, float clamp_min,
                          int impl, int32_t* status_dev, void* stream);

/*
 * Depthwise 3x3 convolution (zero padding 1) over tokens laid out [B, L = h*w, C] with C contiguous,
 * optional bias, optional SiLU.  Replaces `in_proj` = nn.Conv2d(C, C, 3, padding=1, groups=C) [+ SiLU]
 * and the two NCHW<->NLC copies around it (classification/models/vig.py:291-294, 428-430).
 * weight_tap_major: [9][C] (tap = 3*ky + kx), i.e. the reference's [C,1,3,3] parameter transposed;
 * same dtype as x.  C must be a multiple of 16 bytes / element size.  status_dev: optional int32 on the device,
 * bit 0 = a bounded wait ran out (large 16-bit inputs run a TMA-fed kernel with a shared-memory pipeline).
 */
VIG_API int vig_dwconv3x3_fwd(const void* x, const void* weight_tap_major, const void* bias, void* y,
                      int B, int h, int w, int C, int act_silu, int dtype, int32_t* status_dev, void* stream);

/*
 * The same convolution on a horizontal band of a taller image (rows [r0, r0 + h) of the token grid): `top` and `bottom`
 * are the image rows just above and below the band, [B, w, C] each, or NULL where the band touches the image border
 * (zero padding there, as in vig_dwconv3x3_fwd).  It is what a sequence split across GPUs by rows of the patch grid
 * needs from `in_proj` (classification/models/vig.py:291-294, 428-430): the two halo rows arrive from the neighbouring
 * ranks and are read in place, no padded copy of the band is made.  bf16 / fp16, C % 4 == 0.
 */
VIG_API int vig_dwconv3x3_halo_fwd(const void* x, const void* top, const void* bottom, const void* weight_tap_major,
                           const void* bias, void* y, int B, int h, int w, int C, int act_silu, int dtype, void* stream);

/*
 * out[M, N] = x W^T + bias as one tensor-core GEMM with the bias added in fp32 before the rounding: the stacked input
 * projection of the block -- qkv_proj, g_proj and gk_proj of GatedLinearAttention read the same conv output
 * (classification/models/vig.py:283-290, 431-439), so their weights are stacked into one [N, K] matrix.
 * x: [M, K] rows ldx elements apart, w: [N, K] contiguous, bias: [N] or NULL, out: [M, N] rows ldo apart; bf16 / fp16.
 * vig_linear_bias_supported: K % 64 == 0, K <= 192, N % 8 == 0 and at least 256 rows per SM of the current device
 * (smaller problems are left to a library GEMM).  status_dev: optional int32 on the device, bit 0 = a bounded wait ran out.
 */
VIG_API int vig_linear_bias_supported(int64_t M, int K, int N, int dtype);
VIG_API int vig_linear_bias_fwd(const void* x, int64_t ldx, const void* w, const void* bias, void* out, int64_t ldo,
                        int64_t M, int K, int N, int dtype, int32_t* status_dev, void* stream);

/*
 * 2-D gating locality injection: y = RMSNorm_g(o) * sigmoid(gate_logits) + RMSNorm_l(local) * (1 - sigmoid),
 * head-wise norms over dv, optional swish on y.  Replaces l_norm, g_norm, sigmoid, the blend, out_act and
 * the `b h l d -> b l h d` transposes of classification/models/vig.py:444-457 (norm:
 * fla/modules/rmsnorm.py:491-512).  o: [B,H,L,dv] addressed by strides_o[3] (elements; NULL = contiguous
 * [B,H,L,dv]); local, gate_logits, y: [B*L, H*dv] row-major with row strides ld_local, ld_gate, ld_y in
 * elements (H*dv for a contiguous tensor; larger when the operand is a column slice of a wider projection).
 */
VIG_API int vig_gate_inject_fwd(const void* o, const int64_t* strides_o, const void* local, const void* gate_logits,
                        const void* w_gnorm, const void* w_lnorm, void* y,
                        int64_t ld_local, int64_t ld_gate, int64_t ld_y,
                        int B, int H, int L, int dv, float eps, int out_act_swish, int dtype, void* stream);

/*
 * Optional residual add, then RMSNorm: s = x (+ residual); y = s * rsqrt(mean(s^2) + eps) * w;
 * residual_out (optional) receives s.  Replaces RMSNorm.forward(x, residual, prenorm)
 * (fla/modules/rmsnorm.py:491-512; reference semantics rms_norm_ref :38-52).  x, residual, y,
 * residual_out: [rows, N] contiguous; N * element size must be a multiple of 16 and N <= 8192.
 */
VIG_API int vig_add_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* residual_out,
                        int64_t rows, int N, float eps, int dtype, void* stream);

/*
 * LayerNorm over the last dimension with weight and bias, optional swish on the result:
 * y = swish?((x' - mean) * rsqrt(var + eps) * w + b) with x' = x + pre_bias (pre_bias: optional [N] vector, the
 * bias of the convolution that produced x, rounded to the tensor dtype like the convolution would).  Replaces `LayerNorm2d` (+ the swish that follows the
 * first one) of the patch-embedding stem (classification/models/vig.py:619-624, 650-656) on channels-last
 * activations viewed as [rows = B*h*w, N = channels].  x, y contiguous; N * element size a multiple of 16.
 */
VIG_API int vig_layernorm_act_fwd(const void* x, const void* pre_bias, const void* w, const void* bias, void* y,
                          int64_t rows, int N, float eps, int act_swish, int dtype, void* stream);
/* The same, followed by `+ post_add[row % post_period]` (post_add: [post_period, N], added to the rounded result like a
 * separate add): the last LayerNorm2d of the stem with the position-embedding add of `ViG.forward_features`
 * (classification/models/vig.py:860-866) folded in. */
VIG_API int vig_layernorm_act_add_fwd(const void* x, const void* pre_bias, const void* w, const void* bias, const void* post_add,
                                      int64_t post_period, void* y, int64_t rows, int N, float eps, int act_swish, int dtype, void* stream);
/* The same (post_add optional here), with the RMSNorm that follows as a second output: h = y * rsqrt(mean(y^2) + rms_eps) * rms_w
 * from the rounded y, like vig_add_rmsnorm_fwd on y -- the stem's last LayerNorm2d, the position-embedding add and the first
 * block's `attn_norm` (classification/models/vig.py:596-600) in one pass over the tokens. */
VIG_API int vig_layernorm_act_add_rmsnorm_fwd(const void* x, const void* pre_bias, const void* w, const void* bias, const void* post_add,
                                              int64_t post_period, void* y, const void* rms_w, float rms_eps, void* h, int64_t rows, int N,
                                              float eps, int act_swish, int dtype, void* stream);

/*
 * Space-to-depth of the input image for the stem's first convolution (`V2PatchEmbed`, classification/models/vig.py:
 * 650-651: kernel s+1, stride s, padding 1), which is then a 2x2 convolution over s x s pixel blocks:
 * cells[b, cy, cx, (dy*s + dx)*Cin + ic] = x[b, ic, s*cy + dy - 1, s*cx + dx - 1], zero outside the image.
 * x: [B, Cin, H, W] contiguous, cells: [B, H/s + 1, W/s + 1, s*s*Cin] contiguous; H, W multiples of s; s*Cin = 24.
 */
VIG_API int vig_stem_unfold_fwd(const void* x, void* cells, int B, int Cin, int H, int W, int s, int dtype, void* stream);

/*
 * Fold of the input image into cells of 8 x 8 pixels on 8-pixel boundaries (bf16 / fp16, 3 channels):
 * cells[b, cy, cx, (dy*3 + ic)*8 + dx] = x[b, ic, 8cy + dy, 8cx + dx].  x: [B, 3, H, W] contiguous, cells: [B, H/8, W/8, 192]
 * contiguous; H, W multiples of 8.  Input of vig_stem_conv_ln_fwd.
 */
VIG_API int vig_stem_fold_fwd(const void* x, void* cells, int B, int Cin, int H, int W, int dtype, void* stream);

/*
 * The stem's first convolution with its bias, the LayerNorm2d after it and the swish after that, as one tensor-core
 * kernel (bf16 / fp16; `V2PatchEmbed.proj[0..2]`, classification/models/vig.py:650-656, for kernel 9, stride 8, padding 1,
 * 3 input channels and 96 output channels: ViG-T).  cells: [B, CH, CW, 192] from `vig_stem_fold_fwd`.  w2: [96, 512], the
 * convolution's weight in the cell layout: columns 0..191 multiply cell (oy, ox), 192..383 cell (oy, ox-1), 384..447 the
 * last 64 values of cell (oy-1, ox), 448..511 the last 64 values of cell (oy-1, ox-1), each in the cell's value order
 * (dy*3 + ic)*8 + dx (the window of output pixel (oy, ox) starts at image pixel (8oy - 1, 8ox - 1); the taps a 9 x 9 kernel
 * has in the neighbouring cells are among those values; cells outside the image count as zeros).  conv_bias (optional),
 * ln_w, ln_b: [96].  y: [B, CH, CW, 96] contiguous (channels last).  Same roundings as convolution -> bias add -> LayerNorm
 * run separately.  status_dev as in vig_bigla_fwd.
 */
VIG_API int vig_stem_conv_ln_supported(int B, int CH, int CW, int cell, int N, int dtype);
VIG_API int vig_stem_conv_ln_fwd(const void* cells, const void* w2, const void* conv_bias, const void* ln_w, const void* ln_b, void* y,
                                 int B, int CH, int CW, int cell, int N, float eps, int act_swish, int dtype,
                                 int32_t* status_dev, void* stream);

/*
 * Projection with the residual add and the next RMSNorm as its epilogue (bf16 / fp16): r = x W^T + residual (r = x W^T
 * when residual is NULL), h = RMSNorm(r) * norm_weight -- `o_proj` followed by `mlp_norm(h, residual, prenorm=True)`,
 * and `down_proj` followed by the next block's `attn_norm` / the model's final norm (classification/models/vig.py:463,
 * 497, 596-606; fla/modules/rmsnorm.py:491-512).  One tcgen05 GEMM kernel; the projection output is not written.
 * Same roundings as the unfused sequence (projection rounded to the tensor dtype, sum rounded to the tensor dtype).
 * x: [M, K] with row stride ldx; w: [N, K] contiguous; residual, out_r, out_h: [M, N] contiguous; K % 64 == 0,
 * N one of 64, 128, 192, 256, 384.  status_dev: optional int32 on the device, bit 0 = a bounded wait ran out.
 */
VIG_API int vig_linear_add_rmsnorm_supported(int64_t M, int K, int N, int dtype);
VIG_API int vig_linear_add_rmsnorm_fwd(const void* x, int64_t ldx, const void* w, const void* residual, const void* norm_weight,
                                       void* out_r, void* out_h, int64_t M, int K, int N, float eps, int dtype,
                                       int32_t* status_dev, void* stream);

/*
 * SwiGLU: out = gate * sigmoid(gate) * y (fla/modules/activations.py:109-113, the `swiglu` half of
 * `swiglu_linear`).  gate, y: [rows, I] with row stride ld_in elements (gate and y are the two halves of
 * one [rows, 2I] projection in the reference, vig.py:494-497); out: [rows, I] with row stride ld_out.
 */
VIG_API int vig_swiglu_fwd(const void* gate, const void* y, void* out, int64_t rows, int I,
                   int64_t ld_in, int64_t ld_out, int dtype, void* stream);

/*
 * Gate projection of the SwiGLU MLP fused with its activation (tcgen05 GEMM, bf16 / fp16):
 *   out[M, I] = silu(x Wg^T) * (x Wy^T),   W = [Wg ; Wy] of shape [2I, K] (row-major, rows contiguous)
 * Replaces `gate_proj` -> chunk(2) -> `swiglu` of GLAMLP.forward (classification/models/vig.py:494-497,
 * flash-linear-attention/fla/modules/activations.py:109-113) so that the [M, 2I] intermediate is never written.
 * x: [M, K] with row stride ldx, out: [M, I] with row stride ldo (elements).  K % 64 == 0, I % 64 == 0,
 * K <= 384 (one 128-row tile of x stays resident in shared memory); vig_linear_swiglu_supported tells.
 */
VIG_API int vig_linear_swiglu_supported(int64_t M, int K, int I, int dtype);
VIG_API int vig_linear_swiglu_preferred(int64_t M, int K, int I, int dtype);   /* supported AND faster than GEMM + SwiGLU */
VIG_API int vig_linear_swiglu_fwd(const void* x, int64_t ldx, const void* w, void* out, int64_t ldo,
                          int64_t M, int K, int I, int dtype, int32_t* status_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VIG_B200_H */
