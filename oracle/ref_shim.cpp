// C-linkage doorway to the reference's four launcher functions, so that tests can reach
// them through ctypes.  The launchers themselves come from the upstream *.cu.cc files,
// compiled unmodified by oracle/Makefile (target "ref"); they have C++ linkage there
// (declared at winograd2x2_imTrans_op.cc:30, winograd2x2_imTrans_grad_op.cc:29,
// winograd2x2_conv_op.cc:31, winograd2x2_conv_grad_op.cc:32).  Test infrastructure only.
void Winograd2x2ImTransComputeLauncher(const float *Input, float *TransIm, int C, int B, int H, int W,
                                       int pad_h, int pad_w);
void Winograd2x2ImTransGradComputeLauncher(const float *Output_grad, float *Input_grad, int C, int B, int H,
                                           int W, int pad_h, int pad_w);
void Winograd2x2ConvComputeLauncher(const float *Input, const float *Weight, float *Output,
                                    float *tmp_data_buffer, const long long *tmp_ptr_buffer, int C, int B,
                                    int nH, int nW, int K, int pad_h, int pad_w);
void Winograd2x2ConvGradComputeLauncher(const float *TInput, const float *Weight, const float *Output_grad,
                                        float *TInput_grad, float *Weight_grad, float *tmp_data_buffer,
                                        long long *tmp_ptr_buffer, int C, int B, int H, int W, int K,
                                        int pad_h, int pad_w);

extern "C" {
void wgref_imtrans(const float *X, float *V, int C, int B, int H, int W)
{
    Winograd2x2ImTransComputeLauncher(X, V, C, B, H, W, 1, 1);
}
// The upstream gradient launcher overwrites its input (it transforms the incoming
// gradient in place), so callers pass a copy they can lose.
void wgref_imtrans_grad(float *dV_clobbered, float *dX, int C, int B, int H, int W)
{
    Winograd2x2ImTransGradComputeLauncher(dV_clobbered, dX, C, B, H, W, 1, 1);
}
void wgref_conv(const float *V, const float *Wt, float *Y, float *tmp, const long long *ptrs, int C, int B,
                int nH, int nW, int K)
{
    Winograd2x2ConvComputeLauncher(V, Wt, Y, tmp, ptrs, C, B, nH, nW, K, 1, 1);
}
void wgref_conv_grad(const float *V, const float *Wt, const float *dY, float *dV, float *dW, float *tmp,
                     long long *ptrs, int C, int B, int H, int W, int K)
{
    Winograd2x2ConvGradComputeLauncher(V, Wt, dY, dV, dW, tmp, ptrs, C, B, H, W, K, 1, 1);
}
}
