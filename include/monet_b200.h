/*
 * monet_b200.h — C ABI of libmonet_b200.so, the sm_100a replacement for the
 * native extensions underneath MONeT's low-memory operator library
 * (monet/lm_ops/*.cpp, *.cu in utsaslab/MONeT).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless the parameter name ends in
 *     `_host`.  All activations are fp32.  Nothing here allocates device
 *     memory: outputs and workspaces are supplied by the caller (the Python
 *     operators obtain them from PyTorch's caching allocator so that MONeT's
 *     memory profiler, monet/meminfo.py:231-243, keeps measuring the truth).
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default
 *     stream).  Every kernel is enqueued on it; no call synchronises.
 *   - Return value: MB_OK or an MB_ERR_* code; mb_last_error() gives the
 *     message of the calling thread's last failure.
 *   - `layout` selects the physical order of a logical N x C x H x W
 *     activation: MB_NCHW (the reference's only layout) or MB_NHWC
 *     (torch.channels_last; the layout the tensor-core convolutions use).
 *   - Packed intermediates (1-bit ReLU masks, 4-bit max-pool indices) are
 *     indexed by the PHYSICAL element offset, so for MB_NCHW they are
 *     byte-identical with the reference's pack.cu output.
 */
#ifndef MONET_B200_H
#define MONET_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  MB_OK = 0,
  MB_ERR_INVALID_ARGUMENT = 1,   /* bad pointer / size / alignment            */
  MB_ERR_UNSUPPORTED = 2,        /* variant or shape this build cannot run    */
  MB_ERR_WORKSPACE = 3,          /* workspace missing or too small            */
  MB_ERR_LAUNCH = 4,             /* CUDA reported an error at launch          */
  MB_ERR_DEVICE = 5              /* kernel-side status word reported a fault  */
};

enum { MB_NCHW = 0, MB_NHWC = 1 };

/* ---- library ---------------------------------------------------------- */

/* Message of the calling thread's most recent failing call ("" if none).    */
const char* mb_last_error(void);
/* ABI version, bumped when a signature changes.                             */
int mb_abi_version(void);

/* ---- ReLU (replaces lrrelu.cpp:11-20, lrrelu.cu:4-15; relu.py:9-118) ---- */

/* y = max(x, 0) (NaN propagates).  y may alias x (in-place, relu.py:17-18). */
int mb_relu_fwd(const float* x, float* y, size_t n, void* stream);
/* y = max(x, 0) and mask = packbits(x > 0), MSB first, ceil(n/8) bytes, tail
 * bits zero: BinaryActReLU.forward (relu.py:100-104) + pack_kernel
 * (pack.cu:22-31) in one pass.  y may alias x.                              */
int mb_relu_fwd_mask(const float* x, float* y, uint8_t* mask, size_t n, void* stream);
/* dx = bit ? dy : 0: BinaryActReLU.backward (relu.py:109-118) without the
 * n-byte bool temporary of unpack_kernel (pack.cu:32-40).  dx may alias dy. */
int mb_relu_bwd_mask(const float* dy, const uint8_t* mask, float* dx, size_t n, void* stream);
/* dx = act > threshold ? dy : 0, `act` being the saved input or output:
 * threshold_kernel (lrrelu.cu:4-9).  dx may alias dy (the reference always
 * works in place on dy, lrrelu.cpp:14-15).                                  */
int mb_relu_bwd_act(const float* dy, const float* act, float threshold, float* dx, size_t n,
                    void* stream);
/* dx = act > threshold ? dy1 + dy2 : 0.  A tensor read by two consumers (a
 * residual block's input) receives two gradients; the reference's executor sums
 * them with a separate add (schedule.py:296-301) before relu.py's backward.
 * dx may alias dy1 or dy2.                                                  */
int mb_relu_bwd_act2(const float* dy1, const float* dy2, const float* act, float threshold,
                     float* dx, size_t n, void* stream);

/* ---- bit / nibble packing (replaces pack.cpp:38-131, pack.cu:3-50) ------ */

/* out[j] bit (7-k) = (in[8j+k] != 0); ceil(n/8) bytes.                      */
int mb_pack_bits(const uint8_t* in, uint8_t* out, size_t n, void* stream);
/* out[i] = bit i of the packed stream, as 0/1 bytes.                        */
int mb_unpack_bits(const uint8_t* in, uint8_t* out, size_t n, void* stream);
/* out[i] = bit i ? v[i] : 0 (unpack_multiply_kernel, pack.cu:41-50).        */
int mb_unpack_multiply(const uint8_t* in, const float* v, float* out, size_t n, void* stream);
/* out[j] = in[2j] << 4 | in[2j+1]; ceil(n/2) bytes, odd tail low nibble 0.  */
int mb_pack_nibbles(const uint8_t* in, uint8_t* out, size_t n, void* stream);
int mb_unpack_nibbles(const uint8_t* in, uint8_t* out, size_t n, void* stream);

/* ---- hardtanh / ReLU6 (replaces lrhardtanh.cpp:9-16; hardtanh.py:9-93) -- */

int mb_hardtanh_fwd(const float* x, float* y, float lo, float hi, size_t n, void* stream);
/* dx = (lo < act < hi) ? dy : 0, act = saved input or output.               */
int mb_hardtanh_bwd(const float* dy, const float* act, float lo, float hi, float* dx, size_t n,
                    void* stream);

/* ---- residual add (replaces the ATen calls of funcs.py:23-59) ----------- */

/* y = a + alpha * b.  y may alias a (AddIP with op.inplace).                */
int mb_add_fwd(const float* a, const float* b, float alpha, float* y, size_t n, void* stream);
/* y = relu(a + alpha * b): funcs.py add followed by relu.py forward in one pass. */
int mb_add_relu_fwd(const float* a, const float* b, float alpha, float* y, size_t n, void* stream);
/* y = alpha * x  (the `grad_output * s` of Add.backward when s != 1).       */
int mb_scale(const float* x, float alpha, float* y, size_t n, void* stream);

/* ---- max-pool with 4-bit window-local indices --------------------------- */
/* (replaces maxpool.cpp:369-435, maxpool.cu:26-131 and the nibble kernels
 *  pack.cu:3-21; pool.py:38-69)                                             */

typedef struct {
  int N, C, H, W;        /* input extent                                     */
  int P, Q;              /* output extent                                    */
  int kh, kw, sh, sw, ph, pw, dh, dw;
  int layout;            /* MB_NCHW or MB_NHWC, same for input and output    */
} mb_pool_desc;

/* Output extent for one spatial dim (PyTorch's pooling_output_shape).       */
int mb_pool_out_size(int in, int k, int s, int p, int d, int ceil_mode);
/* y = maxpool(x); nibbles = packed window-local argmax, kh*kw <= 16.  Local
 * index of tap (i,j) is i*kw+j counted from the UNCLIPPED window origin
 * (maxpool.cu:42-61); first maximum wins, NaN wins.  Element e (physical
 * offset in y) goes to byte e/2, even e in the high nibble (pack.cu:3-12).
 * `nibbles` may be NULL (values only: SimpleMaxPool2D, pool.py:8-24).       */
int mb_maxpool2d_fwd(const float* x, float* y, uint8_t* nibbles, const mb_pool_desc* d,
                     void* stream);
/* dx[n,c,h,w] = sum of dy over the windows whose stored index points at
 * (h,w); every element of dx is written (no memset needed, unlike
 * pool.py:64).                                                              */
int mb_maxpool2d_bwd(const float* dy, const uint8_t* nibbles, float* dx, const mb_pool_desc* d,
                     void* stream);

/* ---- batch norm (replaces lrbn.cpp:21-172, lrbn.cu:138-235; bn.py) ------ */

typedef struct {
  int N, C, HW;          /* logical extent, HW = H*W                         */
  int layout;
  float eps;
  float momentum;
} mb_bn_desc;

/* Bytes of scratch the statistics kernels need for this shape.              */
size_t mb_bn_workspace_bytes(const mb_bn_desc* d);
/* Training forward (lrbn.cpp:21-41): batch statistics over (N,H,W), then
 * y = gamma*(x-mean)*invstd + beta.  Writes save_mean[C], save_invstd[C]
 * (= 1/sqrt(biased var + eps), cuDNN semantics) and, when non-NULL, updates
 * running_mean / running_var (unbiased) with `momentum`.  y may alias x.    */
int mb_bn_fwd_train(const float* x, const float* gamma, const float* beta, float* running_mean,
                    float* running_var, float* y, float* save_mean, float* save_invstd,
                    const mb_bn_desc* d, void* workspace, size_t workspace_bytes, void* stream);
/* No counterpart in the reference.  mb_bn_fwd_train for callers that must not allocate
 * at run time (a schedule executing inside a solved memory budget, a host whose pool owns
 * the whole device): the statistics scratch is an 8 MiB array built into the library
 * instead of a workspace argument, and the call performs no cudaMalloc / cudaFree.  Shapes
 * needing more scratch than that return MB_ERR_WORKSPACE.  The first call on a device
 * resolves the array's address (do it before any stream capture); all calls on a device
 * share the array, so calls that overlap on the GPU race.                                  */
int mb_bn_fwd_train_noalloc(const float* x, const float* gamma, const float* beta,
                            float* running_mean, float* running_var, float* y, float* save_mean,
                            float* save_invstd, const mb_bn_desc* d, void* stream);
/* y = gamma*(x-mean)*invstd + beta with given statistics: the recompute
 * forward of bn.py:33-34 (with the exact saved invstd, i.e. without that
 * path's second +eps).  y may alias x.                                      */
int mb_bn_fwd_apply(const float* x, const float* gamma, const float* beta, const float* mean,
                    const float* invstd, float* y, const mb_bn_desc* d, void* stream);
/* Backward from the stored OUTPUT y (output_activated_bn_backward,
 * lrbn.cpp:154-172, lrbn.cu:138-209): xhat = (y-beta)/gamma.  gamma == 0 is
 * undefined, as in the reference.  dx may alias dy.                          */
int mb_bn_bwd_from_output(const float* dy, const float* y, const float* gamma, const float* beta,
                          const float* save_invstd, float* dx, float* dgamma, float* dbeta,
                          const mb_bn_desc* d, void* workspace, size_t workspace_bytes,
                          void* stream);
/* Backward from the stored INPUT x (cudnn_backward, lrbn.cpp:43-70).         */
int mb_bn_bwd_from_input(const float* dy, const float* x, const float* gamma,
                         const float* save_mean, const float* save_invstd, float* dx,
                         float* dgamma, float* dbeta, const mb_bn_desc* d, void* workspace,
                         size_t workspace_bytes, void* stream);

/* Fused forms.  The reference runs batch norm, the residual add and ReLU as
 * three operators (bn.py, funcs.py add, relu.py), i.e. three passes over the
 * activation; these do the same arithmetic in the batch-norm sweep.
 *   y = act(bn(x) + residual),  residual may be null; `relu` is the activation
 *   code: 0 none, 1 ReLU, 2 ReLU6 (hardtanh.py's clamp to [0, 6]).
 * Same statistics, workspace and aliasing rules as mb_bn_fwd_train / _apply
 * (y may alias x or residual).                                                */
int mb_bn_act_fwd_train(const float* x, const float* residual, int relu, const float* gamma,
                        const float* beta, float* running_mean, float* running_var, float* y,
                        float* save_mean, float* save_invstd, const mb_bn_desc* d, void* workspace,
                        size_t workspace_bytes, void* stream);
int mb_bn_act_fwd_apply(const float* x, const float* residual, int relu, const float* gamma,
                        const float* beta, const float* mean, const float* invstd, float* y,
                        const mb_bn_desc* d, void* stream);
/* The same forward when the producer of x already summed it per channel
 * (mb_conv2d_fprop_bnstats): `partials` is [2][partial_rows][C] with
 * sum(x - shift) and sum((x - shift)^2) per row and channel, `shift` [C] or null
 * for zero.  Skips the statistics pass over x (4 of the 12 bytes per element);
 * needs no workspace.                                                          */
int mb_bn_act_fwd_train_partials(const float* x, const float* residual, int relu, const float* gamma,
                                 const float* beta, float* running_mean, float* running_var,
                                 float* y, float* save_mean, float* save_invstd,
                                 const mb_bn_desc* d, const float* partials, int partial_rows,
                                 const float* shift, void* stream);
/* Backward through y = relu(bn(x)) from the stored INPUT x: relu.py's backward
 * (dy gated by y > 0) followed by cudnn_backward (lrbn.cpp:43-70) in one reduce
 * and one sweep.  The gate is re-evaluated from x with the forward's own
 * expression, so neither y nor a mask has to be kept.  dx may alias dy.       */
/* The same with the activation code of the forward (1 ReLU, 2 ReLU6: the gate
 * is 0 < z < 6, hardtanh.py's backward).                                       */
int mb_bn_act_bwd_from_input(const float* dy, const float* x, const float* gamma, const float* beta,
                             const float* save_mean, const float* save_invstd, int act, float* dx,
                             float* dgamma, float* dbeta, const mb_bn_desc* d, void* workspace,
                             size_t workspace_bytes, void* stream);
int mb_bn_relu_bwd_from_input(const float* dy, const float* x, const float* gamma,
                              const float* beta, const float* save_mean, const float* save_invstd,
                              float* dx, float* dgamma, float* dbeta, const mb_bn_desc* d,
                              void* workspace, size_t workspace_bytes, void* stream);

/* Backward through y = relu(bn(x) + r): the gated gradient
 * d = (dy1 + dy2) * (y > 0) (dy2 may be NULL) is formed, written to `d` - it is
 * the gradient of r - and summed per channel in ONE pass, then dx follows from
 * d and x as in mb_bn_bwd_from_input.  Replaces relu.py's backward (plus the
 * executor's gradient add, schedule.py:296-301) followed by cudnn_backward
 * (lrbn.cpp:43-70): 32 instead of 36 bytes per element.  d may alias dy1.     */
int mb_bn_add_relu_bwd(const float* dy1, const float* dy2, const float* y, const float* x,
                       const float* gamma, const float* save_mean, const float* save_invstd,
                       float* d, float* dx, float* dgamma, float* dbeta, const mb_bn_desc* desc,
                       void* workspace, size_t workspace_bytes, void* stream);

/* ---- softmax / cross-entropy (replaces softmax.cpp:11-33, softmax.cu) --- */

/* Softmax over `classes` for a [outer, classes, inner] contiguous tensor.   */
int mb_softmax_fwd(const float* x, float* y, size_t outer, int classes, size_t inner,
                   int log_softmax, void* stream);
/* dx = y*(dy - sum(dy*y)) (softmax) or dy - exp(y)*sum(dy) (log-softmax),
 * one kernel instead of the reference's product + reduce pair
 * (softmax.cpp:31).                                                          */
int mb_softmax_bwd(const float* dy, const float* y, float* dx, size_t outer, int classes,
                   size_t inner, int log_softmax, void* stream);
/* Fused log-softmax + NLL forward AND backward in one pass over the logits
 * ([outer, classes, inner], int64 labels [outer, inner]):
 *   loss_rows[r] = logsumexp(x_r) - x_r[label_r]
 *   dlogits      = (softmax(x_r) - onehot(label_r)) * grad_scale
 * The reference has no such operator (its loss sits outside the graph,
 * examples/imagenet.py:327); it stands for nn.CrossEntropyLoss fwd+bwd.     */
int mb_softmax_ce_fwd_bwd(const float* logits, const int64_t* labels, float* loss_rows,
                          float* dlogits, size_t outer, int classes, size_t inner,
                          float grad_scale, void* stream);

/* ---- layout / pooling glue --------------------------------------------- */

/* Physical NCHW -> NHWC (and back) of an N x C x H x W fp32 tensor.         */
int mb_nchw_to_nhwc(const float* x, float* y, int N, int C, int H, int W, void* stream);
int mb_nhwc_to_nchw(const float* x, float* y, int N, int C, int H, int W, void* stream);
/* NCHW -> NHWC with the channels zero-padded to Cp (multiple of 4): prepares a
 * few-channel network input (C = 3) for the tensor-core convolution.         */
int mb_nchw_to_nhwc_pad(const float* x, float* y, int N, int C, int H, int W, int Cp,
                        void* stream);
/* Concatenation and its backward (cat.py:5-29: torch.cat forward, torch.split +
 * one .contiguous() copy per piece backward) as ONE row-copy launch for all
 * pieces.  With the extents before the concatenation axis folded into `rows`
 * and the axis and everything after it into a row, piece i is `widths[i]`
 * consecutive floats of every row of `whole`.  to_pieces = 0: pieces -> whole
 * (forward); 1: whole -> pieces (the split of the gradient).  `pieces` and
 * `widths` are HOST arrays of n_pieces (<= MB_CAT_MAX_PIECES) device pointers /
 * widths in floats.  128-bit accesses when every width is a multiple of 4 and
 * every pointer 16-byte aligned.                                              */
#define MB_CAT_MAX_PIECES 8
int mb_cat_rows(float* whole, float* const* pieces, const int* widths, int n_pieces, size_t rows,
                int to_pieces, void* stream);
/* Global average pool (adaptive_avg_pool2d to 1x1; funcs.py:7-21):
 * y[N,C] = mean over H*W; backward dx = dy / HW broadcast, written fully
 * (no zeros tensor as in funcs.py:20).                                       */
int mb_global_avgpool_fwd(const float* x, float* y, int N, int C, int HW, int layout,
                          void* stream);
int mb_global_avgpool_bwd(const float* dy, float* dx, int N, int C, int HW, int layout,
                          void* stream);

/* ---- convolution on the tensor cores ------------------------------------ */
/* (replaces conv.cpp:299-731: cudnn_convolution, cudnn_convolution_backward_input,
 *  cudnn_convolution_backward_weight and the n_*_algos counters; conv.py:260-341)
 *
 * Layout: activations NHWC fp32 (torch.channels_last), filters [K][R][S][C]
 * fp32 (a channels_last weight tensor), gradients alike.  Arithmetic: TF32
 * operands, fp32 accumulation (tcgen05.mma kind::tf32).  C and K must be
 * multiples of 4, groups == 1, stride <= 2.
 *
 * "Variants" take the place of the reference's cuDNN algorithm index: each
 * pass has mb_conv_num_variants(pass) of them, numbered from 0, that trade
 * workspace for speed or determinism; mb_conv_workspace_bytes() says how much
 * scratch a variant needs so the MONeT solver can budget for it.  A variant
 * that cannot run a shape returns MB_ERR_UNSUPPORTED (the profiler records it
 * as infeasible, meminfo.py:52-55).                                          */

typedef struct {
  int N, C, H, W;        /* input  N x C x H x W                             */
  int K, R, S;           /* filter K x C x R x S                             */
  int P, Q;              /* output N x K x P x Q                             */
  int stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int groups;
} mb_conv_desc;

enum { MB_CONV_FPROP = 0, MB_CONV_DGRAD = 1, MB_CONV_WGRAD = 2 };

/* conv.cpp:729-731 (n_fwd_algos / n_bwd_ip_algos / n_bwd_wt_algos).         */
int mb_conv_num_variants(int pass);
size_t mb_conv_workspace_bytes(int pass, int variant, const mb_conv_desc* d);
/* y = conv(x, w) (+ bias[K] when non-NULL, fused; conv.py:284-285 adds it in
 * a second kernel).  Variant 0: implicit GEMM, no workspace.                 */
int mb_conv2d_fprop(const float* x, const float* w, const float* bias, float* y,
                    const mb_conv_desc* d, int variant, void* workspace, size_t workspace_bytes,
                    void* stream);
/* The same convolution, also leaving the per-channel sums of its output that a
 * following batch norm needs (the reference's batch norm re-reads the whole
 * activation for them, lrbn.cpp:32-40): four extra warps per CTA walk every
 * staged output chunk and add partials[0][cta][k] = sum(y - shift[k]),
 * partials[1][cta][k] = sum((y - shift[k])^2); *partial_rows returns the number
 * of CTA rows written.  `partials` must hold mb_conv_bnstats_bytes(d); `shift` is
 * [K] or NULL (zero) - a value near the channel mean (the running mean) keeps the
 * variance from cancelling.  K must be a multiple of 32; stride-1 multi-tap
 * filters return MB_ERR_UNSUPPORTED (run the plain pair).  Hand the result to
 * mb_bn_act_fwd_train_partials.                                               */
size_t mb_conv_bnstats_bytes(const mb_conv_desc* d);
int mb_conv2d_fprop_bnstats(const float* x, const float* w, const float* bias, float* y,
                            const mb_conv_desc* d, int variant, void* workspace,
                            size_t workspace_bytes, const float* shift, float* partials,
                            size_t partials_bytes, int* partial_rows, void* stream);
/* dx = backward-data.  Variant 0: implicit GEMM over dy.  When C is a multiple of
 * 32 the filter is read in place (MN-major tiles of w) and no workspace is needed;
 * otherwise it is first transposed to [C][R][S][K] in the workspace
 * (mb_conv_workspace_bytes = K*R*S*C*4 bytes).                                  */
int mb_conv2d_dgrad(const float* dy, const float* w, float* dx, const mb_conv_desc* d, int variant,
                    void* workspace, size_t workspace_bytes, void* stream);
/* dw = backward-filter, dbias[K] = sum of dy when non-NULL (conv.py:313-314).
 * Variant 0: split reduction combined with red.global.add (no workspace,
 * summation order not fixed).  Variant 1: per-split partials in the
 * workspace and a deterministic reduction.                                   */
int mb_conv2d_wgrad(const float* x, const float* dy, float* dw, float* dbias,
                    const mb_conv_desc* d, int variant, void* workspace, size_t workspace_bytes,
                    void* stream);
/* Depthwise convolution (groups == C == K; replaces convolution_main / backward_depthwise,
 * conv.cpp:704-726, which defer to ATen's depthwise kernels).  NHWC activations; the filter
 * and its gradient are [R*S][C] (channel innermost).  fp32 FMA, HBM-bound.  C % 4 == 0;
 * backward-filter is built for 1x1, 3x3 and 5x5 windows and zeroes dw / dbias itself.     */
int mb_depthwise_fprop(const float* x, const float* w_tc, const float* bias, float* y,
                       const mb_conv_desc* d, void* stream);
int mb_depthwise_dgrad(const float* dy, const float* w_tc, float* dx, const mb_conv_desc* d,
                       void* stream);
int mb_depthwise_wgrad(const float* x, const float* dy, float* dw_tc, float* dbias,
                       const mb_conv_desc* d, void* stream);
/* Few-channel convolutions (C <= 4, filter width <= 8, stride <= 2: the network's first
 * layer).  The input is copied once into a zero-padded 4-channel NHWC buffer
 * xp[N][Hp][Wp][4] (Hp, Wp from mb_conv_smallc_geometry; N*Hp*Wp*16 bytes, the caller's
 * workspace), the filter is given / returned as [K][R][8][4] (s, c; zero beyond S and C),
 * and the GEMM K dimension becomes R x 32 instead of R*S x 32-with-28-zeros.
 * `d` describes the logical convolution (C = real channel count).  They replace the
 * same cuDNN calls as mb_conv2d_fprop / mb_conv2d_wgrad for that layer.             */
int mb_conv_smallc_geometry(const mb_conv_desc* d, int* Hp, int* Wp);
int mb_conv_smallc_pack_input(const float* x_nchw, float* xp, const mb_conv_desc* d, void* stream);
int mb_conv2d_fprop_smallc(const float* xp, const float* wp, const float* bias, float* y,
                           const mb_conv_desc* d, void* stream);
/* The same first layer when its stride is 2 (3 <= R <= 8): both row phases of the padded input
 * in one buffer xp2[N][Hp2][Wp][2][4] (N*Hp2*Wp*32 bytes, the caller's; extents from
 * mb_conv_smallc2_geometry) and the filter as wp2[K][ceil(R/2)][64] with
 * wp2[k][dh][(s/4)*32 + (s%4)*8 + (r%2)*4 + c] = w[k][c][r = 2*dh + r%2][s], zero elsewhere.
 * The forward then runs on the many-tap kernel with ceil(R/2) row taps, which fetches every
 * input window once per tile instead of once per filter row.                                  */
int mb_conv_smallc2_geometry(const mb_conv_desc* d, int* Hp2, int* Wp);
int mb_conv_smallc2_pack_input(const float* x_nchw, float* xp2, const mb_conv_desc* d, void* stream);
int mb_conv2d_fprop_smallc2(const float* xp2, const float* wp2, const float* bias, float* y,
                            const mb_conv_desc* d, void* stream);
size_t mb_conv_smallc_wgrad_workspace_bytes(const mb_conv_desc* d, int variant);
int mb_conv2d_wgrad_smallc(const float* xp, const float* dy, float* dwp, float* dbias,
                           const mb_conv_desc* d, int variant, void* workspace,
                           size_t workspace_bytes, void* stream);
/* Status word of the tensor-core kernels: 0 = healthy, otherwise the code of
 * the first pipeline wait that timed out (the kernel then gave up cleanly).
 * Synchronises the device.  reset != 0 clears it.                            */
int mb_conv_device_status(int reset);

/* ---- diagnostics (NOT part of the drop-in boundary: nothing in the operator library calls
 * them; they exist for the bench harness and for kernel work and may change freely) -------- */

/* Number of kernels this library has launched in this process (all threads).
 * bench.py reads it to report `gpu_launches`.                               */
unsigned long long mb_launch_count(void);
/* When `device_buffer` (16 x int64, device memory) is non-NULL the stride-1 multi-tap
 * forward / backward-data kernel's first CTA records how many SM cycles each of its roles
 * spent waiting ([0] total, [1] input tile, [2] filter tile, [3] accumulator free, [4]/[5]
 * producer on free slots, [6] epilogue on results, [7] epilogue busy, [8] work items).
 * NULL switches it off (the default).                                                   */
int mb_conv_debug_counters(long long* device_buffer);

#ifdef __cplusplus
}
#endif
#endif /* MONET_B200_H */
