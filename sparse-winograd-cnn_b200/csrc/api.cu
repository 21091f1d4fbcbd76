// C ABI of libwinograd2x2_b200.so: argument checks, workspace carving and dispatch to the
// kernels.  Declarations and per-function documentation are in include/winograd2x2_b200.h.
#include "wg_common.cuh"

namespace wg {
// imtrans.cu
int imtrans_fwd(const float *X, float *V, int B, int H, int W, int C, int layout, int relu, const float *scale, const float *shift,
                cudaStream_t st);
int imtrans_bwd(const float *dV, const float *Vm, float *dX, int B, int H, int W, int C, int layout, cudaStream_t st);
// conv_ffma.cu
int conv_fwd_ffma(const float *V, const float *Wt, float *Y, int B, int nH, int nW, int C, int K, int outH, int outW,
                  int layout, cudaStream_t st);
int conv_dv_ffma(const float *V, const float *Wt, const float *dY, float *dV, int B, int H, int W, int C, int K, int layout,
                 int relu, cudaStream_t st);
int conv_dw_splits(long long P, int C, int K);
size_t conv_dw_scratch_bytes(long long P, int C, int K);
int conv_dw_ffma(const float *V, const float *dY, const float *mask, float *dW, int B, int H, int W, int C, int K, int layout,
                 float *scratch, int splits, cudaStream_t st);
// conv_tc.cu
size_t conv_fwd_tc_workspace_bytes(int B, int nH, int nW, int C, int K);
int conv_fwd_tc(const float *V, const float *Wt, float *Y, int B, int nH, int nW, int C, int K, int outH, int outW, int layout,
                void *ws, size_t ws_bytes, cudaStream_t st);
int tc_last_device_status(cudaStream_t st, unsigned int *where);
int tc_set_wait_limit(long long polls);
int tc_test_drop_load(int nth);
int tc_wait_probe(long long polls, unsigned where, cudaStream_t st);
size_t prepared_weights_bytes(int C, int K);
int weights_prepare(const float *Wt, int C, int K, void *prepared, size_t bytes, cudaStream_t st);
int conv_fwd_tc_prepared(const float *V, const void *prepared, float *Y, int B, int nH, int nW, int C, int K, int outH, int outW,
                         int layout, const float *out_scale, const float *out_shift, const float *residual, cudaStream_t st);
bool conv_fwd_wide_preferred(int C, int K);
size_t conv_fwd_wide_workspace_bytes(long long P, int K);
int conv_fwd_tc_wide(const float *V, const void *prepared, float *Y, int B, int nH, int nW, int C, int K, int outH, int outW,
                     int layout, const float *out_scale, const float *out_shift, const float *residual, void *ws, size_t ws_bytes,
                     cudaStream_t st);
bool fused_fwd_supported(int B, int H, int W, int C, int K, int layout);
int layer_fwd_fused(const float *X, const void *prepared, float *Y, int B, int H, int W, int C, int K, int relu,
                    const float *in_scale, const float *in_shift, const float *out_scale, const float *out_shift,
                    const float *residual, cudaStream_t st);
size_t conv_bwd_tc_workspace_bytes(long long P, int C, int K, int want_dW);
int conv_bwd_tc(const float *V, const float *Wt, const float *dY, const float *mask, float *dV, float *dW, int B, int H, int W,
                int C, int K, int layout, int relu, void *ws, size_t ws_bytes, cudaStream_t st);
}  // namespace wg

using namespace wg;

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
static inline bool layout_ok(int l) { return l == WG2X2_NHWC || l == WG2X2_NCHW; }
static inline bool math_ok(int m) { return m == WG2X2_MATH_FP32 || m == WG2X2_MATH_TF32; }
static inline bool crop_ok(int out, int n) { return out == 2 * n || out == 2 * n - 1; }

extern "C" {

const char *wg2x2_status_string(int s)
{
    switch (s) {
        case WG2X2_OK: return "ok";
        case WG2X2_ERR_BAD_ARG: return "bad argument";
        case WG2X2_ERR_WORKSPACE: return "workspace missing or too small";
        case WG2X2_ERR_LAUNCH: return "CUDA launch error";
        case WG2X2_ERR_TIMEOUT: return "bounded device-side wait gave up";
        case WG2X2_ERR_UNSUPPORTED: return "shape not supported by this math mode";
    }
    return "unknown status";
}

int wg2x2_abi_version(void) { return 1; }

int wg2x2_imtrans_fwd(const float *X, float *V, int B, int H, int W, int C, int layout, int relu, void *stream)
{
    return imtrans_fwd(X, V, B, H, W, C, layout, relu, nullptr, nullptr, (cudaStream_t)stream);
}

int wg2x2_imtrans_fwd_affine(const float *X, const float *in_scale, const float *in_shift, float *V, int B, int H, int W, int C,
                             int layout, int relu, void *stream)
{
    if (!in_scale || !in_shift) return WG2X2_ERR_BAD_ARG;
    return imtrans_fwd(X, V, B, H, W, C, layout, relu, in_scale, in_shift, (cudaStream_t)stream);
}

int wg2x2_imtrans_bwd(const float *dV, const float *V_relu, float *dX, int B, int H, int W, int C, int layout, void *stream)
{
    return imtrans_bwd(dV, V_relu, dX, B, H, W, C, layout, (cudaStream_t)stream);
}

size_t wg2x2_conv_fwd_workspace_bytes(int B, int nH, int nW, int C, int K, int math)
{
    if (math == WG2X2_MATH_TF32) return conv_fwd_tc_workspace_bytes(B, nH, nW, C, K);
    return 0;
}

int wg2x2_conv_fwd(const float *V, const float *Wt, float *Y, int B, int nH, int nW, int C, int K, int out_h, int out_w,
                   int layout, int math, void *workspace, size_t workspace_bytes, void *stream)
{
    if (!V || !Wt || !Y || B <= 0 || nH <= 0 || nW <= 0 || C <= 0 || K <= 0) return WG2X2_ERR_BAD_ARG;
    if (!layout_ok(layout) || !math_ok(math) || !crop_ok(out_h, nH) || !crop_ok(out_w, nW)) return WG2X2_ERR_BAD_ARG;
    if (math == WG2X2_MATH_TF32)
        return conv_fwd_tc(V, Wt, Y, B, nH, nW, C, K, out_h, out_w, layout, workspace, workspace_bytes, (cudaStream_t)stream);
    return conv_fwd_ffma(V, Wt, Y, B, nH, nW, C, K, out_h, out_w, layout, (cudaStream_t)stream);
}

size_t wg2x2_prepared_weights_bytes(int C, int K)
{
    return (C > 0 && K > 0) ? prepared_weights_bytes(C, K) : 0;
}

int wg2x2_weights_prepare(const float *Wt, int C, int K, void *prepared, size_t prepared_bytes, void *stream)
{
    return weights_prepare(Wt, C, K, prepared, prepared_bytes, (cudaStream_t)stream);
}

int wg2x2_conv_fwd_prepared(const float *V, const void *prepared, float *Y, int B, int nH, int nW, int C, int K, int out_h,
                            int out_w, int layout, void *stream)
{
    if (!V || !prepared || !Y || B <= 0 || nH <= 0 || nW <= 0 || C <= 0 || K <= 0) return WG2X2_ERR_BAD_ARG;
    if (!layout_ok(layout) || !crop_ok(out_h, nH) || !crop_ok(out_w, nW)) return WG2X2_ERR_BAD_ARG;
    return conv_fwd_tc_prepared(V, prepared, Y, B, nH, nW, C, K, out_h, out_w, layout, nullptr, nullptr, nullptr, (cudaStream_t)stream);
}

int wg2x2_conv_fwd_prepared_fused(const float *V, const void *prepared, float *Y, int B, int nH, int nW, int C, int K, int out_h,
                                  int out_w, int layout, const float *out_scale, const float *out_shift, const float *residual,
                                  void *stream)
{
    if (!V || !prepared || !Y || B <= 0 || nH <= 0 || nW <= 0 || C <= 0 || K <= 0) return WG2X2_ERR_BAD_ARG;
    if (!layout_ok(layout) || !crop_ok(out_h, nH) || !crop_ok(out_w, nW)) return WG2X2_ERR_BAD_ARG;
    return conv_fwd_tc_prepared(V, prepared, Y, B, nH, nW, C, K, out_h, out_w, layout, out_scale, out_shift, residual,
                                (cudaStream_t)stream);
}

size_t wg2x2_conv_bwd_workspace_bytes(int B, int H, int W, int C, int K, int math, int want_dW)
{
    if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0) return 0;
    const long long P = (long long)B * ((H + 1) / 2) * ((W + 1) / 2);
    if (math == WG2X2_MATH_TF32) return conv_bwd_tc_workspace_bytes(P, C, K, want_dW);
    if (!want_dW) return 0;
    return conv_dw_scratch_bytes(P, C, K);
}

int wg2x2_conv_bwd(const float *V, const float *Wt, const float *dY, const float *mask, float *dV, float *dW, int B, int H,
                   int W, int C, int K, int layout, int relu, int math, void *workspace, size_t workspace_bytes, void *stream)
{
    if (!dY || B <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0) return WG2X2_ERR_BAD_ARG;
    if (!layout_ok(layout) || !math_ok(math)) return WG2X2_ERR_BAD_ARG;
    if (dV && !Wt) return WG2X2_ERR_BAD_ARG;
    if ((dW || (dV && relu)) && !V) return WG2X2_ERR_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    if (math == WG2X2_MATH_TF32)
        return conv_bwd_tc(V, Wt, dY, mask, dV, dW, B, H, W, C, K, layout, relu, workspace, workspace_bytes, st);
    if (dV) {
        const int s = conv_dv_ffma(V, Wt, dY, dV, B, H, W, C, K, layout, relu, st);
        if (s != WG2X2_OK) return s;
    }
    if (dW) {
        const long long P = (long long)B * ((H + 1) / 2) * ((W + 1) / 2);
        const int splits = conv_dw_splits(P, C, K);
        const size_t need = conv_dw_scratch_bytes(P, C, K);
        if (need && (!workspace || workspace_bytes < need)) return WG2X2_ERR_WORKSPACE;
        const int s = conv_dw_ffma(V, dY, mask, dW, B, H, W, C, K, layout, (float *)workspace, splits, st);
        if (s != WG2X2_OK) return s;
    }
    return WG2X2_OK;
}

size_t wg2x2_layer_fwd_workspace_bytes(int B, int H, int W, int C, int K, int math, int keep_V)
{
    if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0) return 0;
    const int nH = (H + 1) / 2, nW = (W + 1) / 2;
    size_t bytes = align_up(wg2x2_conv_fwd_workspace_bytes(B, nH, nW, C, K, math), 256);
    if (!keep_V) bytes += align_up((size_t)16 * B * nH * nW * C * sizeof(float), 256);
    return bytes;
}

int wg2x2_layer_fwd(const float *X, const float *Wt, float *Y, float *V_out, int B, int H, int W, int C, int K, int layout,
                    int relu, int math, void *workspace, size_t workspace_bytes, void *stream)
{
    if (!X || !Wt || !Y || B <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0) return WG2X2_ERR_BAD_ARG;
    if (!layout_ok(layout) || !math_ok(math)) return WG2X2_ERR_BAD_ARG;
    const int nH = (H + 1) / 2, nW = (W + 1) / 2;
    const size_t need = wg2x2_layer_fwd_workspace_bytes(B, H, W, C, K, math, V_out != NULL);
    if (need && (!workspace || workspace_bytes < need)) return WG2X2_ERR_WORKSPACE;
    const size_t conv_ws = align_up(wg2x2_conv_fwd_workspace_bytes(B, nH, nW, C, K, math), 256);
    float *Vbuf = V_out ? V_out : reinterpret_cast<float *>(static_cast<char *>(workspace) + conv_ws);
    int s = wg2x2_imtrans_fwd(X, Vbuf, B, H, W, C, layout, relu, stream);
    if (s != WG2X2_OK) return s;
    return wg2x2_conv_fwd(Vbuf, Wt, Y, B, nH, nW, C, K, H, W, layout, math, workspace, conv_ws, stream);
}

size_t wg2x2_conv_fwd_prepared_workspace_bytes(int B, int nH, int nW, int C, int K)
{
    if (B <= 0 || nH <= 0 || nW <= 0 || C <= 0 || K <= 0 || !conv_fwd_wide_preferred(C, K)) return 0;
    return conv_fwd_wide_workspace_bytes((long long)B * nH * nW, K);
}

int wg2x2_conv_fwd_prepared_ws(const float *V, const void *prepared, float *Y, int B, int nH, int nW, int C, int K, int out_h,
                               int out_w, int layout, const float *out_scale, const float *out_shift, const float *residual,
                               void *workspace, size_t workspace_bytes, void *stream)
{
    if (!V || !prepared || !Y || B <= 0 || nH <= 0 || nW <= 0 || C <= 0 || K <= 0) return WG2X2_ERR_BAD_ARG;
    if (!layout_ok(layout) || !crop_ok(out_h, nH) || !crop_ok(out_w, nW)) return WG2X2_ERR_BAD_ARG;
    if ((out_scale == nullptr) != (out_shift == nullptr)) return WG2X2_ERR_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    if (conv_fwd_wide_preferred(C, K) && workspace)
        return conv_fwd_tc_wide(V, prepared, Y, B, nH, nW, C, K, out_h, out_w, layout, out_scale, out_shift, residual, workspace,
                                workspace_bytes, st);
    return conv_fwd_tc_prepared(V, prepared, Y, B, nH, nW, C, K, out_h, out_w, layout, out_scale, out_shift, residual, st);
}

int wg2x2_layer_fwd_fused_supported(int B, int H, int W, int C, int K, int layout)
{
    return (B > 0 && H > 0 && W > 0 && C > 0 && K > 0 && fused_fwd_supported(B, H, W, C, K, layout)) ? 1 : 0;
}

int wg2x2_layer_fwd_prepared(const float *X, const void *prepared, float *Y, float *V_scratch, int B, int H, int W, int C, int K,
                             int layout, int relu, const float *out_scale, const float *out_shift, const float *residual,
                             void *stream)
{
    if (!X || !prepared || !Y || B <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0) return WG2X2_ERR_BAD_ARG;
    if (!layout_ok(layout)) return WG2X2_ERR_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    // The one-kernel path redoes the input transform for every block of 64 output channels, so it wins while
    // there are few of them (measured: K <= 128, or K <= 256 with C <= 64); beyond that the two-kernel path,
    // whose wide GEMM shares one transformed input among 256 output channels, is faster.
    const bool fused_pays = K <= 128 || (K <= 256 && C <= 64);
    const bool aligned16 = ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(Y)) & 15u) == 0;   // TMA both ways
    if (fused_fwd_supported(B, H, W, C, K, layout) && aligned16 && (fused_pays || !V_scratch))
        return layer_fwd_fused(X, prepared, Y, B, H, W, C, K, relu, nullptr, nullptr, out_scale, out_shift, residual, st);
    if (!V_scratch) return WG2X2_ERR_WORKSPACE;
    const int nH = (H + 1) / 2, nW = (W + 1) / 2;
    const int s = imtrans_fwd(X, V_scratch, B, H, W, C, layout, relu, nullptr, nullptr, st);
    if (s != WG2X2_OK) return s;
    return conv_fwd_tc_prepared(V_scratch, prepared, Y, B, nH, nW, C, K, H, W, layout, out_scale, out_shift, residual, st);
}

size_t wg2x2_layer_fwd_prepared_workspace_bytes(int B, int H, int W, int C, int K)
{
    if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0) return 0;
    return wg2x2_conv_fwd_prepared_workspace_bytes(B, (H + 1) / 2, (W + 1) / 2, C, K);
}

int wg2x2_layer_fwd_prepared_ws(const float *X, const void *prepared, float *Y, float *V_scratch, int B, int H, int W, int C, int K,
                                int layout, int relu, const float *out_scale, const float *out_shift, const float *residual,
                                void *workspace, size_t workspace_bytes, void *stream)
{
    if (!X || !prepared || !Y || B <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0) return WG2X2_ERR_BAD_ARG;
    if (!layout_ok(layout)) return WG2X2_ERR_BAD_ARG;
    // layers with many channels: input transform, then the products as wide GEMMs through the workspace
    if (conv_fwd_wide_preferred(C, K) && V_scratch && workspace) {
        const int nH = (H + 1) / 2, nW = (W + 1) / 2;
        const int s = imtrans_fwd(X, V_scratch, B, H, W, C, layout, relu, nullptr, nullptr, (cudaStream_t)stream);
        if (s != WG2X2_OK) return s;
        return wg2x2_conv_fwd_prepared_ws(V_scratch, prepared, Y, B, nH, nW, C, K, H, W, layout, out_scale, out_shift, residual, workspace,
                                          workspace_bytes, stream);
    }
    return wg2x2_layer_fwd_prepared(X, prepared, Y, V_scratch, B, H, W, C, K, layout, relu, out_scale, out_shift, residual, stream);
}

int wg2x2_layer_fwd_fused(const float *X, const void *prepared, float *Y, int B, int H, int W, int C, int K, int relu,
                          const float *out_scale, const float *out_shift, const float *residual, void *stream)
{
    if (!X || !prepared || !Y || B <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0) return WG2X2_ERR_BAD_ARG;
    return layer_fwd_fused(X, prepared, Y, B, H, W, C, K, relu, nullptr, nullptr, out_scale, out_shift, residual, (cudaStream_t)stream);
}

int wg2x2_layer_fwd_fused_affine(const float *X, const void *prepared, float *Y, int B, int H, int W, int C, int K, int relu,
                                 const float *in_scale, const float *in_shift, const float *out_scale, const float *out_shift,
                                 const float *residual, void *stream)
{
    if (!X || !prepared || !Y || B <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0) return WG2X2_ERR_BAD_ARG;
    return layer_fwd_fused(X, prepared, Y, B, H, W, C, K, relu, in_scale, in_shift, out_scale, out_shift, residual, (cudaStream_t)stream);
}

int wg2x2_last_device_status(void *stream, unsigned int *where)
{
    return tc_last_device_status((cudaStream_t)stream, where);
}

int wg2x2_set_wait_limit(long long polls) { return tc_set_wait_limit(polls); }

int wg2x2_test_drop_load(int nth) { return tc_test_drop_load(nth); }

int wg2x2_test_wait_probe(long long polls, unsigned int where, void *stream)
{
    return tc_wait_probe(polls, where, (cudaStream_t)stream);
}

}  // extern "C"
