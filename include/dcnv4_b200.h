/*
 * dcnv4_b200 -- C ABI of the B200 (sm_100a) DCNv4 / FlashDeformAttn operator library.
 *
 * This is the drop-in boundary: plain pointers and sizes, no framework types.  Each entry
 * point names the reference interface it replaces (paths relative to the reference
 * project root).  The reference exposes these four operations as the pybind module
 * `DCNv4.ext` (DCNv4_op/src/vision.cpp:14-21, dispatch in DCNv4_op/src/dcnv4.h:19-107).
 *
 * Conventions
 *  - Every pointer is DEVICE memory owned by the caller, 16-byte aligned, contiguous in the
 *    layouts stated below.  The library never allocates, frees or synchronises; all work is
 *    enqueued on `stream` (a cudaStream_t passed as void*; NULL = the legacy default stream).
 *  - Return value: 0 on success, a negative DCNV4B200_ERR_* for a rejected argument (nothing
 *    was launched), or a positive cudaError_t reported by a launch.
 *  - dtype: DCNV4B200_F32 / _F16 / _BF16 selects the storage type of all floating tensors of
 *    a call; arithmetic is always fp32.
 *  - The launch-tuning arguments of the reference (`d_stride`, `block_thread`) and its
 *    `im2col_step` batch chunking have no counterpart: the kernels derive their own geometry
 *    and take the whole batch in one launch.
 */
#ifndef DCNV4_B200_H_
#define DCNV4_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DCNV4B200_ABI_VERSION 1

enum { DCNV4B200_F32 = 0, DCNV4B200_F16 = 1, DCNV4B200_BF16 = 2 };

enum {
  DCNV4B200_OK = 0,
  DCNV4B200_ERR_NULL = -1,        /* a required pointer is NULL */
  DCNV4B200_ERR_DTYPE = -2,       /* unknown dtype code */
  DCNV4B200_ERR_SHAPE = -3,       /* non-positive or inconsistent dimension */
  DCNV4B200_ERR_ALIGN = -4,       /* pointer not 16-byte aligned */
  DCNV4B200_ERR_WORKSPACE = -5,   /* workspace missing or too small */
  DCNV4B200_ERR_UNSUPPORTED = -6, /* outside the supported parameter space (see strerror) */
  DCNV4B200_ERR_PADDED_DIM = -7,  /* padded_offset_dim not a multiple of 8 or < 3*K*G */
  DCNV4B200_ERR_CHANNELS = -8,    /* group_channels not a multiple of 16 bytes worth of elements */
  DCNV4B200_ERR_TOO_LARGE = -9,   /* an index would overflow 31 bits */
  DCNV4B200_ERR_SCRATCH_LIMIT = -10 /* tensor larger than the built-in scratch of *_static_scratch */
};

/* Activation codes of the fused kernels around the operator. */
#define DCNV4B200_ACT_NONE 0
#define DCNV4B200_ACT_GELU 1

/* Version of this ABI (DCNV4B200_ABI_VERSION of the build). */
int dcnv4b200_abi_version(void);

/* Text for a return code of this library (negative codes) or of the CUDA runtime (positive). */
const char* dcnv4b200_strerror(int code);

/* Output extent along one axis: (in + 2*pad - (dil*(k-1)+1))/stride + 1.
 * Replaces the size rule of DCNv4_op/src/cuda/dcnv4_cuda.cu:48-52. */
int dcnv4b200_out_size(int in, int pad, int dil, int k, int stride);

/*
 * DCNv4 forward.  Replaces `dcnv4_forward` / `dcnv4_cuda_forward`
 * (DCNv4_op/src/dcnv4.h:64-83, DCNv4_op/src/cuda/dcnv4_cuda.cu:26-90) and the kernel
 * forward_kernel_dcn_reg (DCNv4_op/src/cuda/dcnv4_im2col_cuda.cuh:142-325).
 *   value       (N,H,W,G*D)          channels-last
 *   offset_mask (N,Ho,Wo,padded_offset_dim); per group g the 3K values at g*3K are
 *               [x0,y0,...,x(K-1),y(K-1), m0..m(K-1)], K = kh*kw - remove_center, point order
 *               k = i*kh + j with i over kernel_w (outer) and j over kernel_h (inner)
 *   out         (N,Ho,Wo,G*D)        fully overwritten (no pre-zeroing needed)
 * softmax != 0 normalises the K mask values per (query, group) before use.
 */
int dcnv4b200_fwd(const void* value, const void* offset_mask, void* out, int dtype,
                  int N, int H, int W, int G, int D,
                  int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                  float offset_scale, int remove_center, int padded_offset_dim, int softmax,
                  void* stream);

/* Bytes of caller-provided scratch `dcnv4b200_bwd` needs: 0 for fp32 (gradients accumulate
 * in grad_value itself), N*H*W*G*D*4 for fp16/bf16 (the fp32 accumulation buffer that the
 * reference allocates inside dcnv4_cuda_backward, DCNv4_op/src/cuda/dcnv4_cuda.cu:133-139). */
size_t dcnv4b200_bwd_workspace_bytes(int dtype, int N, int H, int W, int G, int D);

/*
 * DCNv4 backward.  Replaces `dcnv4_backward` / `dcnv4_cuda_backward`
 * (DCNv4_op/src/dcnv4.h:85-107, DCNv4_op/src/cuda/dcnv4_cuda.cu:92-175) and the kernels of
 * DCNv4_op/src/cuda/dcnv4_col2im_cuda.cuh:20-472.
 *   grad_out         (N,Ho,Wo,G*D)
 *   grad_value       like value        fully overwritten
 *   grad_offset_mask like offset_mask  fully overwritten, pad columns are zero
 *   workspace        >= dcnv4b200_bwd_workspace_bytes(...) bytes (may be NULL when that is 0)
 * grad_value is accumulated with floating-point atomics, so its low-order bits depend on
 * the execution order; everything else is deterministic.
 */
int dcnv4b200_bwd(const void* value, const void* offset_mask, const void* grad_out,
                  void* grad_value, void* grad_offset_mask, void* workspace, size_t workspace_bytes,
                  int dtype, int N, int H, int W, int G, int D,
                  int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                  float offset_scale, int remove_center, int padded_offset_dim, int softmax,
                  void* stream);

/*
 * FlashDeformAttn forward.  Replaces `flash_deform_attn_forward` /
 * `flash_deform_attn_cuda_forward` (DCNv4_op/src/dcnv4.h:19-38,
 * DCNv4_op/src/cuda/flash_deform_attn_cuda.cu:26-84) and forward_kernel_reg
 * (DCNv4_op/src/cuda/flash_deform_im2col_cuda.cuh:129-451).
 *   value             (B,Len_in,G,D)
 *   spatial_shapes    (L,2) int64 on the device: (H_l, W_l); the caller guarantees
 *                     level_start[l] + H_l*W_l <= Len_in (the library cannot check device data)
 *   level_start_index (L)   int64 on the device
 *   sampling_loc_attn (B,Len_q,G,3*L*K): [x,y] for each of the L*K points (level-major,
 *                     normalised to [0,1]) followed by the L*K attention logits
 *   out               (B,Len_q,G*D)   fully overwritten
 */
int fdab200_fwd(const void* value, const int64_t* spatial_shapes, const int64_t* level_start_index,
                const void* sampling_loc_attn, void* out, int dtype,
                int B, int Len_in, int G, int D, int L, int Len_q, int K, void* stream);

/* Scratch bytes for fdab200_bwd: 0 for fp32, B*Len_in*G*D*4 for fp16/bf16
 * (DCNv4_op/src/cuda/flash_deform_attn_cuda.cu:125-131). */
size_t fdab200_bwd_workspace_bytes(int dtype, int B, int Len_in, int G, int D);

/*
 * FlashDeformAttn backward.  Replaces `flash_deform_attn_backward` /
 * `flash_deform_attn_cuda_backward` (DCNv4_op/src/dcnv4.h:40-62,
 * DCNv4_op/src/cuda/flash_deform_attn_cuda.cu:86-163) and the kernels of
 * DCNv4_op/src/cuda/flash_deform_col2im_cuda.cuh:20-580.
 *   grad_out (B,Len_q,G*D); grad_value like value; grad_sampling_loc_attn like
 *   sampling_loc_attn; both fully overwritten.
 */
int fdab200_bwd(const void* value, const int64_t* spatial_shapes, const int64_t* level_start_index,
                const void* sampling_loc_attn, const void* grad_out,
                void* grad_value, void* grad_sampling_loc_attn, void* workspace, size_t workspace_bytes,
                int dtype, int B, int Len_in, int G, int D, int L, int Len_q, int K, void* stream);

/*
 * Corner-index probes: for every sampling point write (h_low, w_low) = floor of the fp32
 * sampling coordinate the kernels use, or INT32_MIN twice for a point that fails the range
 * test.  corners: (N,Ho,Wo,G,K,2) resp. (B,Len_q,G,L*K,2) int32.  They restate the
 * coordinate arithmetic of DCNv4_op/src/cuda/dcnv4_im2col_cuda.cuh:203-227 and
 * DCNv4_op/src/cuda/flash_deform_im2col_cuda.cuh:185-190 with DCNv4_op/src/cuda/common.h:47-48
 * and exist so parity tests can check corner selection bit for bit.
 */
int dcnv4b200_fwd_corners(const void* offset_mask, int32_t* corners, int dtype,
                          int N, int H, int W, int G,
                          int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                          float offset_scale, int remove_center, int padded_offset_dim, void* stream);
int fdab200_fwd_corners(const int64_t* spatial_shapes, const void* sampling_loc_attn, int32_t* corners,
                        int dtype, int B, int G, int L, int Len_q, int K, void* stream);

/*
 * LayerNorm forward over the last (contiguous) dimension of a channels-last tensor:
 * y[r,:] = (x[r,:] - mean_r) * rsqrt(var_r + eps) * gamma + beta, statistics in fp32.
 * The FlashInternImage blocks around the operator normalise millions of short rows
 * (C = 64..1280); the reference uses torch.nn.LayerNorm for them
 * (classification/models/flash_intern_image.py:34-56) and has no kernel of its own.
 *   x, y   (rows, C) in `dtype`; gamma, beta (C) in `param_dtype` (fp32 or the same as dtype)
 * C*elem must be a multiple of 16 bytes and at most 1024 (fp32) / 2048 (fp16, bf16) channels;
 * larger or odd sizes return DCNV4B200_ERR_UNSUPPORTED / _ERR_CHANNELS and launch nothing.
 */
int dcnv4b200_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, int dtype,
                            int param_dtype, long long rows, int C, float eps, void* stream);

/*
 * LayerNorm followed by an activation in the same pass: y = act(LayerNorm(x)), with the normalised
 * value rounded to `dtype` before the activation, as a separate LayerNorm and GELU pair would.
 * FlashInternImage's stem is conv -> LayerNorm -> GELU -> conv -> LayerNorm over the largest
 * activations of the network (classification/models/flash_intern_image.py:235-272, built with
 * norm_layer='LN' at :615-618); the reference runs the norm and the activation as two kernels.
 * `activation` is DCNV4B200_ACT_NONE or DCNV4B200_ACT_GELU (erf form); other arguments and limits
 * as dcnv4b200_layernorm_fwd.
 */
int dcnv4b200_layernorm_act_fwd(const void* x, const void* gamma, const void* beta, void* y, int dtype,
                                int param_dtype, long long rows, int C, float eps, int activation, void* stream);

/*
 * Centre-feature-scale blend of the DCNv4 module, forward, in one pass:
 *     s[r, g]   = sigmoid(sum_c x[r, c] * weight[g, c] + bias[g])
 *     out[r, c] = x[r, c] * (1 - s[r, c / D]) + x_proj[r, c] * s[r, c / D]
 * Replaces the Linear + sigmoid + repeat + blend of DCNv4_op/DCNv4/modules/dcnv4.py:18-26,142-147
 * (five PyTorch kernels in the reference; none of its CUDA sources covers them).
 *   x, x_proj, out (rows, G*D) in `dtype`; weight (G, G*D) and bias (G) in `param_dtype`
 *   (fp32 or the same as dtype).  D*elem must be a multiple of 16 bytes; G*D at most 1024 (fp32) /
 *   2048 (fp16, bf16) channels and G at most 128, else DCNV4B200_ERR_UNSUPPORTED.
 */
int dcnv4b200_center_scale_blend_fwd(const void* x, const void* x_proj, const void* weight, const void* bias,
                                     void* out, int dtype, int param_dtype, long long rows, int G, int D,
                                     void* stream);

/*
 * Linear layer with a fused epilogue, inference only, on the tcgen05 tensor cores:
 *     t = x . weight^T + bias            rounded to `dtype` (what nn.Linear would store)
 *     t = GELU(t)                        if activation == DCNV4B200_ACT_GELU (erf form)
 *     y = t + residual                   if residual != NULL
 * The reference runs these steps as separate kernels around every DCNv4 operator: nn.Linear,
 * nn.GELU and the residual additions of MLPLayer / InternImageLayer
 * (classification/models/flash_intern_image.py:308-341, :414-432); it has no fused kernel.
 *   x (M,K), weight (N,K) as nn.Linear stores it, bias (N) or NULL, residual (M,N) or NULL,
 *   y (M,N); all row-major and contiguous in `dtype`, which must be fp16 or bf16
 *   (DCNV4B200_ERR_DTYPE otherwise).  N and K must be multiples of 8 (_ERR_CHANNELS), every
 *   pointer 16-byte aligned.  y may alias residual; it must not alias x.
 */
int dcnv4b200_linear_fwd(const void* x, const void* weight, const void* bias, const void* residual, void* y,
                         int dtype, long long M, int N, int K, int activation, void* stream);

/*
 * dcnv4b200_linear_fwd (no activation) that also returns the LayerNorm of its result:
 *     y = x . weight^T + bias [+ residual]               as above, rounded to `dtype`
 *     z = LayerNorm(y) * gamma + beta                    over the N columns of each row, fp32 statistics
 * In a pre-norm FlashInternImage layer every residual sum is followed by a LayerNorm
 * (classification/models/flash_intern_image.py:424-425: x + dcn(norm1(x)), x + mlp(norm2(x))),
 * which the reference runs as a separate torch.nn.LayerNorm kernel.  Here the row is
 * normalised while it is still on chip.
 *   gamma, beta (N) in `dtype`; y and z (M,N).  N must be at most 256 (a row has to lie inside
 *   one tile) and a multiple of 32, of 64 above 128 (DCNV4B200_ERR_UNSUPPORTED / _ERR_CHANNELS
 *   otherwise).
 */
int dcnv4b200_linear_ln_fwd(const void* x, const void* weight, const void* bias, const void* residual, void* y,
                            const void* gamma, const void* beta, float eps, void* z, int dtype, long long M,
                            int N, int K, void* stream);

/*
 * Two Linear layers over the same input in one product (inference): with weight = [W1; W2]
 * stacked along the output dimension ((N1 + N2, K) row-major) and bias likewise ((N1 + N2) or NULL),
 *     y1 = x . W1^T + b1   (M, N1)        y2 = x . W2^T + b2   (M, N2)
 * are written as two separate contiguous tensors while x is read once.  In the reference's
 * DCNv4 module both the value projection and the offset/mask projection consume the layer input
 * (DCNv4_op/DCNv4/modules/dcnv4.py:116-124) as two separate nn.Linear calls.
 *   fp16 / bf16; N1 a multiple of 64, N2 and K multiples of 8; every pointer 16-byte aligned.
 */
int dcnv4b200_linear_pair_fwd(const void* x, const void* weight, const void* bias, void* y1, int N1, void* y2,
                              int N2, int dtype, long long M, int K, void* stream);

/*
 * DCNv4 forward that computes the offset/mask rows itself (inference):
 *     offset_mask = x . weight^T + bias,    out = dcnv4b200_fwd(value, offset_mask, 3x3, stride 1, pad 1,
 *                                                  dilation 1, no softmax, remove_center 0)
 * in one kernel.  The rows of 128 consecutive positions are produced on the tensor cores by the CTA
 * that samples for them, rounded to `dtype` as the Linear would have stored them, and never go to
 * memory.  In the reference this is `self.offset_mask(input)` followed by `DCNv4Function.apply`
 * (DCNv4_op/DCNv4/modules/dcnv4.py:121-140) with the (N, H, W, padded 27 G) tensor between them.
 *   value, out (N, H, W, G*D), 32-byte aligned; x (N*H*W, K) and weight (weight_rows, K) row-major,
 *   16-byte aligned; bias (weight_rows) or NULL; all fp16 or all bf16.
 *   D must be 16 and G at most 128 (DCNV4B200_ERR_UNSUPPORTED otherwise: the caller
 *   then runs the two steps separately); K a multiple of 8; weight_rows >= 27 G
 *   (_ERR_PADDED_DIM), rows beyond 27 G -- the Linear's padding -- are ignored.
 */
int dcnv4b200_fwd_fused_offset(const void* value, const void* x, const void* weight, const void* bias, void* out,
                               int dtype, int N, int H, int W, int G, int D, int K, int weight_rows,
                               float offset_scale, void* stream);

/*
 * y = act(x + bias) over the last dimension of a channels-last tensor, in one pass:
 *   x, y (rows, C) contiguous in `dtype` (fp16 or bf16; y may alias x), bias (C) in `dtype`,
 *   C a multiple of 8, activation DCNV4B200_ACT_NONE or DCNV4B200_ACT_GELU (erf form, on the
 *   sum rounded to `dtype`).
 * FlashInternImage's stem is conv -> BatchNorm -> GELU -> conv -> BatchNorm
 * (classification/models/flash_intern_image.py:235-272); once the BatchNorms are folded into
 * the convolutions for inference, their shift remains as a convolution bias, which PyTorch applies
 * as a separate broadcast addition followed by a separate GELU kernel.  The reference has no
 * kernel for this.
 */
int dcnv4b200_bias_act_fwd(const void* x, const void* bias, void* y, int dtype, long long rows, int C,
                           int activation, void* stream);

/*
 * Read and clear the current device's kernel status word: 0 = nothing to report; 1 = a kernel
 * gave up on a bounded wait for its staged tile; 2 = a FlashDeformAttn call was given a level
 * (spatial_shapes / level_start_index) that does not lie inside the flattened value tensor --
 * that level was treated as empty, its samples contributing nothing, instead of being read or
 * written out of bounds (the reference trusts these device tensors unchecked).  Synchronises the
 * device; meant for tests and post-mortems, not for the hot path.  No counterpart in the reference.
 */
int dcnv4b200_device_status(int* status_out);

/*
 * DCNv4 backward without any device allocation -- not even a caller-provided workspace.
 * (This entry point has no counterpart in the reference, whose backward allocates its
 * buffers with ATen on every call.)
 *
 * Who needs it: code that runs the operator from inside another runtime's execution hook
 * (an inference server's or plugin framework's enqueue callback, a latency-critical loop).
 * There cudaMalloc is forbidden -- it stalls the whole device and may fail outright once the
 * host application has claimed the remaining memory for its own pools -- so the caller can
 * pass inputs and outputs but cannot produce the fp32 accumulation buffer that
 * dcnv4b200_bwd wants for fp16/bf16 tensors.  Here that buffer is a fixed array inside the
 * library image instead.
 *
 * Same arguments and results as dcnv4b200_bwd minus workspace/workspace_bytes.  Limits and
 * rules:
 *  - fp16/bf16: N*H*W*G*D must not exceed dcnv4b200_bwd_static_scratch_max_elements()
 *    (4 Mi elements = 16 MiB of fp32, held by every GPU that loads the library until the
 *    process exits); larger tensors return DCNV4B200_ERR_SCRATCH_LIMIT and launch nothing.
 *    fp32 tensors accumulate in grad_value itself and have no size limit.
 *  - The first call on a device looks up the array's device address; make that first call
 *    outside any stream capture.  The 16 MiB themselves are reserved by the CUDA runtime when
 *    this library's device code is first loaded on a device, which with lazy module loading
 *    (the default) happens at the first call of ANY entry point that touches the device.  A
 *    host that later hands all remaining device memory to its own arena should therefore make
 *    one call per device at start-up -- dcnv4b200_device_status() is enough -- BEFORE it claims
 *    the memory; after that no call of this entry point changes the amount of free memory.
 *  - All calls on a device share the one array.  Each call clears the part it uses before
 *    summing into it, so calls issued one after another on a stream are fine; calls that may
 *    overlap on the GPU (different streams, different host threads) race on it and must be
 *    serialised by the caller.
 *  - Calls no cudaMalloc / cudaFree / allocating library routine.
 */
size_t dcnv4b200_bwd_static_scratch_max_elements(void);
int dcnv4b200_bwd_static_scratch(const void* value, const void* offset_mask, const void* grad_out,
                                 void* grad_value, void* grad_offset_mask,
                                 int dtype, int N, int H, int W, int G, int D,
                                 int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                                 float offset_scale, int remove_center, int padded_offset_dim, int softmax,
                                 void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DCNV4_B200_H_ */
