/*
 * winograd2x2_b200 — C ABI of the B200 (sm_100a) Winograd-ReLU F(2x2,3x3) convolution path.
 *
 * Every entry point takes plain device pointers and sizes, enqueues its work on the
 * caller's CUDA stream (a cudaStream_t passed as void*; NULL = the default stream),
 * allocates nothing, never synchronises the device and never aborts: the return value
 * is a wg2x2_status.  The caller owns every buffer, scratch included.  Inputs are never
 * written.
 *
 * Tensor layouts
 *   image-like tensors X, Y, dX, dY : `layout` = WG2X2_NHWC (B,H,W,C) — the reference's —
 *                                     or WG2X2_NCHW (B,C,H,W)
 *   V, dV : (16, B, nH, nW, C), nH=(H+1)/2, nW=(W+1)/2, Winograd position t=4*row+col
 *   W, dW, mask : (16, C, K)
 * all fp32, dense, contiguous.  Padding is 1 and the tile stride is 2, as the reference
 * hard-wires them at every call site (e.g. winograd2x2_imTrans_op.cc:55).
 */
#ifndef WINOGRAD2X2_B200_H
#define WINOGRAD2X2_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    WG2X2_OK = 0,
    WG2X2_ERR_BAD_ARG = -1,     /* null pointer, non-positive size, unknown enum, misaligned buffer */
    WG2X2_ERR_WORKSPACE = -2,   /* workspace missing or smaller than the *_workspace_bytes query */
    WG2X2_ERR_LAUNCH = -3,      /* the CUDA runtime refused a launch (cudaGetLastError != success) */
    WG2X2_ERR_TIMEOUT = -4,     /* a bounded device-side wait gave up (reported by wg2x2_last_device_status) */
    WG2X2_ERR_UNSUPPORTED = -5  /* shape outside what the selected math mode supports */
} wg2x2_status;

enum { WG2X2_NHWC = 0, WG2X2_NCHW = 1 };

/* WG2X2_MATH_FP32: FFMA on the CUDA cores, fp32 accumulate (max rel err <= 1e-5 vs float64).
 * WG2X2_MATH_TF32: tcgen05 kind::tf32 tensor-core MMAs accumulating in TMEM (<= 5e-3). */
enum { WG2X2_MATH_FP32 = 0, WG2X2_MATH_TF32 = 1 };

const char *wg2x2_status_string(int status);

/* Version of this ABI (bumped when a signature changes). */
int wg2x2_abi_version(void);

/*
 * Input transform V = B^T d B over 4x4 tiles at stride 2, pad 1, optionally followed by
 * the Winograd-domain ReLU (relu != 0).
 * Replaces Winograd2x2ImTransComputeLauncher (winograd2x2_imTrans_op.cc:30,
 * winograd2x2_imTrans_cuda.cu.cc:151-157) and, with relu, the tf.nn.relu the layer wrapper
 * applies to its result (ResNet-18-var/winograd_imtrans.py:16-17).
 */
int wg2x2_imtrans_fwd(const float *X, float *V, int B, int H, int W, int C, int layout, int relu,
                      void *stream);

/*
 * The same with a per-channel affine map applied to the pixels first, V = [relu](B^T (x*in_scale[c]+in_shift[c]) B),
 * the zero padding staying zero.  It folds the inference-form BatchNorm that the reference graph places in front
 * of every WinogradImTrans (ResNet-18-var/imagenet-resnet-transWino-prune.py:117-118) into the transform's load.
 */
int wg2x2_imtrans_fwd_affine(const float *X, const float *in_scale, const float *in_shift, float *V, int B, int H,
                             int W, int C, int layout, int relu, void *stream);

/*
 * Gradient of the input transform: dX = overlap-add of B g B^T over the tiles covering each
 * pixel.  dV is read, never written (the reference transforms it in place).  V_relu, when
 * not NULL, is the saved forward output of wg2x2_imtrans_fwd(relu=1): the gradient is taken
 * as zero where V_relu <= 0 (the ReluGrad step).  H, W are the true image sizes.
 * Replaces Winograd2x2ImTransGradComputeLauncher (winograd2x2_imTrans_grad_op.cc:29,
 * winograd2x2_imTrans_grad_cuda.cu.cc:118-129).
 */
int wg2x2_imtrans_bwd(const float *dV, const float *V_relu, float *dX, int B, int H, int W, int C,
                      int layout, void *stream);

/*
 * Winograd-domain product and output transform: Y = A^T (V_t . W_t) A, cropped to
 * out_h x out_w (2nH-1 <= out_h <= 2nH, same for w).
 * Replaces Winograd2x2ConvComputeLauncher (winograd2x2_conv_op.cc:31,
 * winograd2x2_conv_cuda.cu.cc:65-93): the 16 cublasSgemmBatched products and the
 * Output_transform kernel become one kernel that stores no product tensor -- except for
 * WG2X2_MATH_TF32 with C, K >= 256 and a workspace that has room for it, where the products
 * go through scratch memory (see wg2x2_conv_fwd_prepared_ws).
 * workspace: see wg2x2_conv_fwd_workspace_bytes (0 bytes for WG2X2_MATH_FP32).
 */
int wg2x2_conv_fwd(const float *V, const float *Wt, float *Y, int B, int nH, int nW, int C, int K,
                   int out_h, int out_w, int layout, int math, void *workspace, size_t workspace_bytes,
                   void *stream);
size_t wg2x2_conv_fwd_workspace_bytes(int B, int nH, int nW, int C, int K, int math);

/*
 * Weights prepared once for the tensor-core path, for callers whose weights do not change
 * between calls (inference, or between optimiser steps): W (16,C,K) is repacked to (16,K,C),
 * rounded to TF32 (round to nearest), and a map of all-zero 64x32 weight blocks is built so
 * the kernel skips their loads and MMAs.  `prepared` is a caller-owned device buffer of
 * wg2x2_prepared_weights_bytes(C,K) bytes, 256-byte aligned.  wg2x2_conv_fwd with
 * WG2X2_MATH_TF32 does the same preparation into its workspace on every call.
 * Takes the place of the per-step `W * mask` and of the operand set-up before
 * cublasSgemmBatched (ResNet-18-var/winograd_conv.py:21-26, winograd2x2_conv_cuda.cu.cc:71-85).
 * Needs C % 4 == 0 (WG2X2_ERR_UNSUPPORTED otherwise).
 */
size_t wg2x2_prepared_weights_bytes(int C, int K);
int wg2x2_weights_prepare(const float *Wt, int C, int K, void *prepared, size_t prepared_bytes, void *stream);
int wg2x2_conv_fwd_prepared(const float *V, const void *prepared, float *Y, int B, int nH, int nW, int C, int K,
                            int out_h, int out_w, int layout, void *stream);
/*
 * wg2x2_conv_fwd_prepared with the epilogue extras Y = acc*out_scale[k] + out_shift[k] (+ residual), each optional
 * (NULL): the BatchNorm after a WinogradConv and the shortcut addition of a residual block
 * (ResNet-18-var/imagenet-resnet-transWino-prune.py:122-128) done while the result is still in registers.
 * `residual` has the shape and layout of Y.  out_scale/out_shift and residual must be 16-byte aligned.
 */
int wg2x2_conv_fwd_prepared_fused(const float *V, const void *prepared, float *Y, int B, int nH, int nW, int C, int K,
                                  int out_h, int out_w, int layout, const float *out_scale, const float *out_shift,
                                  const float *residual, void *stream);

/*
 * wg2x2_conv_fwd_prepared_fused with scratch memory, which lets layers with many channels (C, K >= 256) take
 * the wide path: the 16 products as GEMMs with 256 output channels per unit into `workspace` (16*P*K floats,
 * wg2x2_conv_fwd_prepared_workspace_bytes; 0 = the shape does not use it), then one pass for A^T m A — the
 * reference's own two-step structure (winograd2x2_conv_cuda.cu.cc:80-89) on tensor cores.  With workspace ==
 * NULL, or for smaller layers, the single-kernel path of wg2x2_conv_fwd_prepared_fused runs.
 */
int wg2x2_conv_fwd_prepared_ws(const float *V, const void *prepared, float *Y, int B, int nH, int nW, int C, int K,
                               int out_h, int out_w, int layout, const float *out_scale, const float *out_shift,
                               const float *residual, void *workspace, size_t workspace_bytes, void *stream);
size_t wg2x2_conv_fwd_prepared_workspace_bytes(int B, int nH, int nW, int C, int K);

/*
 * Gradient of the product/output-transform op for dY of size (B,H,W,K):
 *   dV_t = (A dY A^T)_t . W_t^T   (skipped when dV == NULL)
 *   dW_t = V_t^T . (A dY A^T)_t   (skipped when dW == NULL), multiplied by mask when mask != NULL
 * relu != 0 additionally zeroes dV where V <= 0, folding the ReluGrad of the layer wrapper
 * into this op.  Rows/columns of the tile grid beyond H, W count as zero gradient.
 * Replaces Winograd2x2ConvGradComputeLauncher (winograd2x2_conv_grad_op.cc:32,
 * winograd2x2_conv_grad_cuda.cu.cc:79-124) and the mask product autodiff derives from
 * ResNet-18-var/winograd_conv.py:23-26.
 */
int wg2x2_conv_bwd(const float *V, const float *Wt, const float *dY, const float *mask, float *dV,
                   float *dW, int B, int H, int W, int C, int K, int layout, int relu, int math,
                   void *workspace, size_t workspace_bytes, void *stream);
size_t wg2x2_conv_bwd_workspace_bytes(int B, int H, int W, int C, int K, int math, int want_dW);

/*
 * dW of wg2x2_conv_bwd (FP32 path) for callers that cannot allocate device memory: hooks
 * that receive only an op's inputs and outputs, processes that forbid cudaMalloc after
 * start-up, plug-ins of a host application that owns all device memory.  The split-P
 * partial sums go to a fixed 32 MiB array inside the library (held by every GPU that loads
 * it, until exit) instead of a caller workspace.  No counterpart in the reference, whose
 * caller always allocates the temporaries.
 *  - Limit: splits * 16*C*K floats <= wg2x2_conv_bwd_dw_noalloc_max_bytes()/4, with the same
 *    split count as wg2x2_conv_bwd; larger problems return WG2X2_ERR_WORKSPACE.
 *  - The first call on each device looks up the array's device address; make that call
 *    before any stream capture.  The call itself allocates nothing.  The address is kept for
 *    the life of the process: use the device's primary context, and do not call this entry
 *    point again after cudaDeviceReset (the kept address would be stale).
 *  - Every call shares the one array: calls that overlap on the GPU (two streams, two
 *    threads) race.  Nothing in it needs clearing: each call overwrites all it later reads.
 * Arguments as in wg2x2_conv_bwd; the result equals its dW bit for bit.
 */
int wg2x2_conv_bwd_dw_noalloc(const float *V, const float *dY, const float *mask, float *dW, int B, int H,
                              int W, int C, int K, int layout, void *stream);
size_t wg2x2_conv_bwd_dw_noalloc_max_bytes(void);

/*
 * Whole layer forward, X -> Y = conv(relu?(imtrans(X)), W): the call pair at
 * ResNet-18-var/imagenet-resnet-transWino-prune.py:118-119.  V_out, when not NULL, receives
 * the transformed (post-ReLU) input for a later backward pass; when NULL it lives in the
 * workspace.
 */
int wg2x2_layer_fwd(const float *X, const float *Wt, float *Y, float *V_out, int B, int H, int W, int C,
                    int K, int layout, int relu, int math, void *workspace, size_t workspace_bytes,
                    void *stream);
size_t wg2x2_layer_fwd_workspace_bytes(int B, int H, int W, int C, int K, int math, int keep_V);

/*
 * Whole layer forward with prepared weights (tensor-core path), the call pair of
 * ResNet-18-var/imagenet-resnet-transWino-prune.py:118-119 in its fastest form for the shape that needs no scratch
 * memory beyond V_scratch (wg2x2_layer_fwd_prepared_ws adds the wide path for C, K >= 256):
 *  - one kernel (wg2x2_layer_fwd_fused) where that is supported (NCHW, W % 4 == 0, C % 16 == 0, X and Y
 *    16-byte aligned) and either it is the faster one (K <= 128, or K <= 256 with C <= 64) or no V_scratch
 *    was given: both transforms and the ReLU happen on the SM, neither the transformed input nor the
 *    products are written to memory;
 *  - otherwise the two kernels with V_scratch (16*B*nH*nW*C floats) in between; WG2X2_ERR_WORKSPACE if NULL.
 * out_scale/out_shift/residual as in wg2x2_conv_fwd_prepared_fused (each may be NULL).
 */
int wg2x2_layer_fwd_prepared(const float *X, const void *prepared, float *Y, float *V_scratch, int B, int H, int W,
                             int C, int K, int layout, int relu, const float *out_scale, const float *out_shift,
                             const float *residual, void *stream);
/*
 * The same with scratch memory for the products, which lets layers with many channels (C, K >= 256) take their
 * fastest form too: input transform into V_scratch, then the wide path of wg2x2_conv_fwd_prepared_ws through
 * `workspace` (wg2x2_layer_fwd_prepared_workspace_bytes; 0 = the shape does not use one).  With workspace == NULL, or
 * for other shapes, this is wg2x2_layer_fwd_prepared.
 */
int wg2x2_layer_fwd_prepared_ws(const float *X, const void *prepared, float *Y, float *V_scratch, int B, int H, int W,
                                int C, int K, int layout, int relu, const float *out_scale, const float *out_shift,
                                const float *residual, void *workspace, size_t workspace_bytes, void *stream);
size_t wg2x2_layer_fwd_prepared_workspace_bytes(int B, int H, int W, int C, int K);
int wg2x2_layer_fwd_fused_supported(int B, int H, int W, int C, int K, int layout);
/* The one-kernel layer forward on its own (NCHW in and out); WG2X2_ERR_UNSUPPORTED outside the shapes above.
 * residual may be Y itself: the result is then added into Y in place (the TMA unit does the addition);
 * otherwise residual is first copied to Y on the same stream and must not overlap it. */
int wg2x2_layer_fwd_fused(const float *X, const void *prepared, float *Y, int B, int H, int W, int C, int K, int relu,
                          const float *out_scale, const float *out_shift, const float *residual, void *stream);
/*
 * The same with a per-input-channel affine map in front of the transform, x -> in_scale[c] * x + in_shift[c]
 * inside the image (the padding stays zero): BatchNorm -> WinogradImTrans(relu) -> WinogradConv
 * [-> BatchNorm + shortcut add] of ResNet-18-var/imagenet-resnet-transWino-prune.py:117-119 as one kernel.
 * in_scale / in_shift: C floats each, both or neither NULL.
 */
int wg2x2_layer_fwd_fused_affine(const float *X, const void *prepared, float *Y, int B, int H, int W, int C, int K,
                                 int relu, const float *in_scale, const float *in_shift, const float *out_scale,
                                 const float *out_shift, const float *residual, void *stream);

/*
 * 3x3 / stride 2 max-pooling with TensorFlow's SAME padding on an NCHW tensor (B,C,H,W) -> (B,C,ceil(H/2),ceil(W/2)):
 * the MaxPooling('pool*', l, 3, stride=2, padding='SAME') steps between the stages of the reference's ResNet-18-var
 * graph (ResNet-18-var/imagenet-resnet-transWino-prune.py:115,141,166,191).  Y_relu, when not NULL, also receives
 * max(relu_scale[c] * Y + relu_shift[c], 0) (scale 1 and shift 0 when those are NULL): what the next stage's shortcut
 * branch starts from -- BNReLU in the first stage (:126), a plain ReLU later (:151) -- so it costs no pass of its own.
 */
int wg2x2_maxpool3x3s2_same(const float *X, float *Y, float *Y_relu, const float *relu_scale, const float *relu_shift,
                            int B, int C, int H, int W, void *stream);
/* The same pooling of a channels-last input X (B,H,W,C) into NCHW outputs: the step after a stem convolution that runs
 * channels-last (ResNet-18-var/imagenet-resnet-transWino-prune.py:114-115) when the Winograd layers that follow take NCHW. */
int wg2x2_maxpool3x3s2_same_nhwc_in(const float *X, float *Y, float *Y_relu, const float *relu_scale,
                                    const float *relu_shift, int B, int C, int H, int W, void *stream);

/*
 * The dense head of the reference's ResNet-18-var graph as one kernel: Conv2D('conv1', image, 64, 7, stride=2) (no
 * bias, no activation) followed by MaxPooling('pool1', l, 3, stride=2, padding='SAME'), both with TensorFlow's SAME
 * padding (ResNet-18-var/imagenet-resnet-transWino-prune.py:112-114).  X (B,3,H,W) NCHW with H and W multiples of 4 and
 * W <= 224; Y (B,64,H/4,W/4) NCHW; Y_relu as in wg2x2_maxpool3x3s2_same.  The convolution runs on the tensor cores
 * with TF32 operands and FP32 accumulation and its (B,64,H/2,W/2) result never reaches memory.  Other sizes return
 * WG2X2_ERR_UNSUPPORTED (run a stock convolution and wg2x2_maxpool3x3s2_same instead).
 * wg2x2_stem_prepare arranges the (64,3,7,7) weights once into wg2x2_stem_prepared_floats() floats for the kernel.
 */
int wg2x2_stem_prepared_floats(void);
int wg2x2_stem_prepare(const float *W, float *Wp, void *stream);
int wg2x2_stem7x7s2_pool(const float *X, const float *Wp, float *Y, float *Y_relu, const float *relu_scale,
                         const float *relu_shift, int B, int H, int W, void *stream);

/*
 * Status word of the most recent kernel on this device that uses bounded waits
 * (the tcgen05 path): 0, or WG2X2_ERR_TIMEOUT with a code saying where it gave up.
 * Synchronises the given stream.
 */
int wg2x2_last_device_status(void *stream, unsigned int *where);

/*
 * Bounded waits.  Every device-side wait of the tensor-core kernels (on an mbarrier fed by a TMA copy, by
 * tcgen05.commit or by another warp) polls at most `polls` times; when one runs out, the role records where it
 * was, raises a CTA-wide flag that makes the other roles leave, the kernel frees its tensor memory and returns,
 * and wg2x2_last_device_status reports WG2X2_ERR_TIMEOUT once (reading clears it).  The outputs of such a launch
 * are incomplete: a caller that cannot afford that polls the status after its last launch.  polls = 0 restores
 * the default (4e7, about a second).  Process-wide; read by each launch when it is enqueued.
 * The reference has no counterpart: its kernels never wait on one another.
 */
int wg2x2_set_wait_limit(long long polls);
/*
 * Test hooks for the time-out path (they fault and hang nothing).  wg2x2_test_drop_load(n): in the next
 * launch of conv_fwd (row-walk) or layer_fwd_fused, CTA 0's weight producer stops before its n-th load, so the
 * MMA issuer's wait for that stage runs out; one-shot, n < 0 disarms.  wg2x2_test_wait_probe: a one-thread
 * kernel that waits `polls` polls on a barrier nobody arrives on and records `where`.
 */
int wg2x2_test_drop_load(int nth);
int wg2x2_test_wait_probe(long long polls, unsigned int where, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* WINOGRAD2X2_B200_H */
