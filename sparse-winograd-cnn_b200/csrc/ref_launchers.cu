// The reference's four launcher functions, by name and argument list, with C++ linkage as
// the reference's op files declare them (winograd2x2_imTrans_op.cc:30,
// winograd2x2_imTrans_grad_op.cc:29, winograd2x2_conv_op.cc:31, winograd2x2_conv_grad_op.cc:32),
// so that those op files link against this library unchanged.  Like the originals they
// return nothing, take NHWC tensors and enqueue on the default stream; unlike them they do
// not touch their inputs and need neither the product buffer nor the pointer table
// (tmp_data_buffer doubles as the dW split scratch, tmp_ptr_buffer is ignored).
#include "wg_common.cuh"

namespace wg {
int conv_dw_splits(long long P, int C, int K);
int conv_dw_ffma(const float *V, const float *dY, const float *mask, float *dW, int B, int H, int W, int C, int K, int layout,
                 float *scratch, int splits, cudaStream_t st);
}

void Winograd2x2ImTransComputeLauncher(const float *Input, float *TransIm, int C, int B, int H, int W, int pad_h, int pad_w)
{
    (void)pad_h; (void)pad_w;
    wg2x2_imtrans_fwd(Input, TransIm, B, H, W, C, WG2X2_NHWC, 0, nullptr);
}

void Winograd2x2ImTransGradComputeLauncher(const float *Output_grad, float *Input_grad, int C, int B, int H, int W, int pad_h,
                                           int pad_w)
{
    (void)pad_h; (void)pad_w;
    wg2x2_imtrans_bwd(Output_grad, nullptr, Input_grad, B, H, W, C, WG2X2_NHWC, nullptr);
}

void Winograd2x2ConvComputeLauncher(const float *Input, const float *Weight, float *Output, float *tmp_data_buffer,
                                    const long long *tmp_ptr_buffer, int C, int B, int nH, int nW, int K, int pad_h, int pad_w)
{
    (void)tmp_data_buffer; (void)tmp_ptr_buffer; (void)pad_h; (void)pad_w;
    wg2x2_conv_fwd(Input, Weight, Output, B, nH, nW, C, K, 2 * nH, 2 * nW, WG2X2_NHWC, WG2X2_MATH_FP32, nullptr, 0, nullptr);
}

void Winograd2x2ConvGradComputeLauncher(const float *TInput, const float *Weight, const float *Output_grad, float *TInput_grad,
                                        float *Weight_grad, float *tmp_data_buffer, long long *tmp_ptr_buffer, int C, int B, int H,
                                        int W, int K, int pad_h, int pad_w)
{
    (void)tmp_ptr_buffer; (void)pad_h; (void)pad_w;
    wg2x2_conv_bwd(TInput, Weight, Output_grad, nullptr, TInput_grad, nullptr, B, H, W, C, K, WG2X2_NHWC, 0, WG2X2_MATH_FP32,
                   nullptr, 0, nullptr);
    // dW: the caller's product buffer (16*P*K floats) serves as split scratch; it holds
    // floor(P/C) partial copies of dW (16*C*K floats each).
    const long long P = (long long)B * ((H + 1) / 2) * ((W + 1) / 2);
    int splits = wg::conv_dw_splits(P, C, K);
    const long long fit = tmp_data_buffer ? P / C : 1;
    if (splits > fit) splits = fit < 1 ? 1 : (int)fit;
    wg::conv_dw_ffma(TInput, Output_grad, nullptr, Weight_grad, B, H, W, C, K, WG2X2_NHWC, tmp_data_buffer, splits, nullptr);
}
